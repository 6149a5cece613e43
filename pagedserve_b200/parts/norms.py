"""Norm parts."""

from __future__ import annotations

import torch

from pagedserve_b200.parts.base import Norm, NormPrologue, register_part
from pagedserve_b200.weights.loader import ParamSpec


class DeferredNorm:
    """A norm that has been asked for but not computed: the consumer (a matrix product) may fold it
    into its own kernel, or call :meth:`materialize` to get the normed tensor."""

    def __init__(self, norm, x, rows=None):
        self.norm = norm
        self.x = x
        self.rows = rows
        count = rows.numel() if rows is not None else x.shape[0]
        self.shape = (count, x.shape[1])
        self.device = x.device

    def materialize(self, out=None):
        return self.norm.forward(self.x, out=out, rows=self.rows)


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * weight + bias over the last axis, in float32.

    reference: nn.LayerNorm at src/model/paged_decoder.py:170-177, 291-294 and the
    fused kernel src/kernels/triton_residual_layernorm.py:25-40.
    params: width, eps, name, has_mean (False gives the RMS form), has_bias, init_std.
    """

    graph_safe = True

    def param_specs(self):
        p = self.params
        specs = [(ParamSpec(self._n(p["name"] + ".weight"), (p["width"],), "vector"),
                  ("ones_plus_normal", p.get("init_std", 0.0)))]
        if p.get("has_bias", True):
            specs.append((ParamSpec(self._n(p["name"] + ".bias"), (p["width"],), "vector"),
                          ("normal", p.get("init_std", 0.0))))
        return specs

    def bind(self, tensors):
        p = self.params
        self.weight = tensors[self._n(p["name"] + ".weight")]
        self.bias = tensors[self._n(p["name"] + ".bias")] if p.get("has_bias", True) else None

    def defer(self, x, rows=None):
        return DeferredNorm(self, x, rows)

    def fused_prologue(self):
        return NormPrologue(self.weight, self.bias, float(self.params["eps"]), bool(self.params.get("has_mean", True)))

    def forward(self, x, out=None, rows=None, out_dtype=None):
        n_rows = rows.numel() if rows is not None else x.shape[0]
        if out is None:
            out = self.env.ops.empty((n_rows, x.shape[1]), out_dtype or self.env.dtype, x.device)
        return self.env.ops.layernorm(x, self.weight, self.bias, float(self.params["eps"]), out, rows=rows,
                                      has_mean=self.params.get("has_mean", True))
