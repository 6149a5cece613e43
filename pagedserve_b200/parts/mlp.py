"""Dense feed-forward."""

from __future__ import annotations

import torch

from pagedserve_b200.parts.base import FeedForward, register_part
from pagedserve_b200.weights.loader import ParamSpec

ACTIVATIONS = ("gelu_tanh", "gelu_erf")


@register_part("feed_forward", "dense_mlp")
class DenseMLP(FeedForward):
    """residual += act(x W_up + b_up) W_down + b_down
    (reference: src/model/paged_decoder.py:178-179, 224-228, 273-280).
    params: hidden_size, inner_size, activation ('gelu_tanh' | 'gelu_erf'), has_bias,
    stored_in_out, up_name, down_name, init_std, out_init_std."""

    graph_safe = True
    accepts_deferred_norm = True       # x goes straight into ops.linear

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        if self.params["activation"] not in ACTIVATIONS:
            raise ValueError(f"unsupported activation {self.params['activation']!r}; one of {ACTIVATIONS}")

    def _matrix(self, name, n_out, n_in, std):
        flip = self.params.get("stored_in_out", False)
        stored = (n_in, n_out) if flip else (n_out, n_in)
        return (ParamSpec(self._n(name + ".weight"), stored, "matmul", transpose=flip), ("normal", std))

    def param_specs(self):
        p = self.params
        specs = [self._matrix(p["up_name"], p["inner_size"], p["hidden_size"], p.get("init_std", 0.02)),
                 self._matrix(p["down_name"], p["hidden_size"], p["inner_size"], p.get("out_init_std", 0.02))]
        if p.get("has_bias", True):
            specs.append((ParamSpec(self._n(p["up_name"] + ".bias"), (p["inner_size"],), "vector"),
                          ("normal", p.get("init_std", 0.02))))
            specs.append((ParamSpec(self._n(p["down_name"] + ".bias"), (p["hidden_size"],), "vector"),
                          ("normal", p.get("init_std", 0.02))))
        return specs

    def bind(self, tensors):
        p = self.params
        self.w_up = tensors[self._n(p["up_name"] + ".weight")]         # [I, H]
        self.w_down = tensors[self._n(p["down_name"] + ".weight")]     # [H, I]
        has_bias = p.get("has_bias", True)
        self.b_up = tensors[self._n(p["up_name"] + ".bias")] if has_bias else None
        self.b_down = tensors[self._n(p["down_name"] + ".bias")] if has_bias else None

    def forward(self, x, residual, ctx):
        p = self.params
        ops = self.env.ops
        inner = ops.empty((x.shape[0], p["inner_size"]), self.env.dtype, x.device)
        ops.linear(x, self.w_up, self.b_up, inner, act=p["activation"])
        ops.linear(inner, self.w_down, self.b_down, residual, accumulate=True)
