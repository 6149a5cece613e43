"""Causal self-attention over the paged cache."""

from __future__ import annotations

import torch

from pagedserve_b200.cache.manager import KVNeed
from pagedserve_b200.parts.base import Mixer, register_part
from pagedserve_b200.weights.loader import ParamSpec


@register_part("mixer", "causal_attention")
class CausalSelfAttention(Mixer):
    """Packed QKV projection, causal attention over the request's pages, output projection.

    qkv = x W + b, split q|k|v in that order, head j = columns [j*hd, (j+1)*hd)
    (reference: src/model/paged_decoder.py:49-53, 63-69);
    s = (q.k) * scale, keys after the query masked, softmax in float32, o = p v
    (reference: src/model/paged_attention.py:262-295);
    residual += o W_o + b_o (reference: src/model/paged_decoder.py:135, 184).

    The step's keys and values are written to the pages first; queries then read
    everything, old and new, from the pages.  A token's result therefore does not
    depend on how its prompt was cut into steps.

    params: hidden_size, n_heads, n_kv_heads, head_dim, scale, window (None = all keys),
    has_bias, stored_in_out (True: matrices stored [in, out]), qkv_name, out_name,
    init_std, out_init_std, write_cache (False: this run only reads a cache layer that another
    run of the schedule has written in the same step).
    """

    graph_safe = True
    accepts_deferred_norm = True       # x goes straight into ops.linear_qkv

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        if p["n_heads"] % p["n_kv_heads"] != 0:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if not (0 < p["head_dim"] <= 256):
            # multiples of 16 run on the tensor-core kernels in bfloat16; other sizes on the CUDA-core ones
            raise ValueError(f"head_dim {p['head_dim']} is not supported: at most 256")
        self.q_width = p["n_heads"] * p["head_dim"]
        self.kv_width = p["n_kv_heads"] * p["head_dim"]

    def cache_need(self):
        p = self.params
        return KVNeed(p["n_kv_heads"], p["head_dim"], p.get("window"))

    def _matrix(self, name, n_out, n_in, std):
        stored = (n_in, n_out) if self.params.get("stored_in_out", False) else (n_out, n_in)
        return (ParamSpec(self._n(name + ".weight"), stored, "matmul",
                          transpose=self.params.get("stored_in_out", False)), ("normal", std))

    def param_specs(self):
        p = self.params
        total = self.q_width + 2 * self.kv_width
        specs = [self._matrix(p["qkv_name"], total, p["hidden_size"], p.get("init_std", 0.02)),
                 self._matrix(p["out_name"], p["hidden_size"], self.q_width, p.get("out_init_std", 0.02))]
        if p.get("has_bias", True):
            specs.append((ParamSpec(self._n(p["qkv_name"] + ".bias"), (total,), "vector"),
                          ("normal", p.get("init_std", 0.02))))
            specs.append((ParamSpec(self._n(p["out_name"] + ".bias"), (p["hidden_size"],), "vector"),
                          ("normal", p.get("init_std", 0.02))))
        return specs

    def bind(self, tensors):
        p = self.params
        self.w_qkv = tensors[self._n(p["qkv_name"] + ".weight")]       # [q+2kv, H]
        self.w_out = tensors[self._n(p["out_name"] + ".weight")]       # [H, q]
        has_bias = p.get("has_bias", True)
        self.b_qkv = tensors[self._n(p["qkv_name"] + ".bias")] if has_bias else None
        self.b_out = tensors[self._n(p["out_name"] + ".bias")] if has_bias else None

    def forward(self, x, residual, ctx, layer):
        p = self.params
        ops = self.env.ops
        tokens = x.shape[0]
        from pagedserve_b200.parts.base import PositionEncoding

        qkv = ops.empty((tokens, self.q_width + 2 * self.kv_width), self.env.dtype, x.device)
        write_cache = p.get("write_cache", True)
        # keys may go from the projection straight into the pages unless the position encoding
        # still has to transform them
        no_rotation = type(layer.positions).rotate is PositionEncoding.rotate
        written = ops.linear_qkv(x, self.w_qkv, self.b_qkv, qkv, ctx, layer, self.q_width, self.kv_width,
                                 p["head_dim"], scatter=write_cache and no_rotation)
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if not no_rotation:
            layer.positions.rotate(q, k, ctx)
        context = ops.empty((tokens, self.q_width), self.env.dtype, x.device)
        ops.attention(q, k, v, context, ctx, layer, p["n_heads"], p["n_kv_heads"], p["head_dim"],
                      p.get("window"), float(p["scale"]), write_cache=write_cache and not written)
        ops.linear(context, self.w_out, self.b_out, residual, accumulate=True)
