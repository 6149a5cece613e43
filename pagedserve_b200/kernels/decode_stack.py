"""Host side of the persistent decode kernel (csrc/decode_stack.cu).

A model qualifies when every scheduled layer is the pre-norm arrangement of a causal-attention mixer
and a dense MLP with LayerNorm-type norms, all layers have the same sizes, there is one cache group,
positions are a learned table or none, and the compute dtype is bfloat16.  Nothing here names a model:
the check reads the parts' kinds and constants.  Other models, float32 runs and batches above 64 use the
general path (one kernel per operation, captured as a CUDA graph).
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from pagedserve_b200.kernels.build import load as _load_library
from pagedserve_b200.kernels.ops import KernelError, _ACT_CODE

_p = ctypes.c_void_p
_i = ctypes.c_int


class _LayerWeights(ctypes.Structure):
    _fields_ = [(name, _p) for name in (
        "ln1_g", "ln1_b", "ln2_g", "ln2_b", "w_qkv", "b_qkv", "w_out", "b_out", "w_up", "b_up", "w_down",
        "b_down", "k_pool", "v_pool")]


class _Params(ctypes.Structure):
    _fields_ = (
        [(name, _i) for name in ("B", "H", "n_heads", "n_kv_heads", "head_dim", "I", "V", "n_layers", "page_size",
                                 "window", "act", "n_positions", "ln_has_mean", "stage_in_smem", "n_steps",
                                 "want_logits", "do_sample")]
        + [("eps", ctypes.c_float), ("scale_log2", ctypes.c_float), ("page_stride", ctypes.c_longlong)]
        + [(name, _p) for name in ("layers", "wte", "wpe", "lnf_g", "lnf_b", "lm_head", "token_ids", "positions",
                                   "kv_len", "block_table")]
        + [("bt_stride", _i)]
        + [(name, _p) for name in ("h", "xn", "q", "attn", "inner", "part_acc", "part_ml", "counters")]
        + [("chunk_keys", _i), ("split_chunks", _i), ("n_splits", _i)]
        + [(name, _p) for name in ("logits", "temperature", "seed", "best", "sampled", "history", "step_counter")]
        + [("max_steps", _i)]
        + [("barrier", _p), ("status", _p), ("skip_mask", _i), ("ctas_per_sm", _i)]
    )


def _ptr(tensor: Optional[torch.Tensor]) -> int:
    return tensor.data_ptr() if tensor is not None else 0


class DecodeStack:
    MAX_BATCH = 64
    STAGE_LIMIT = 64 * 1024          # staged activations beyond this go through a global buffer

    def __init__(self, model, cache, device):
        self.lib = _load_library("stack")
        layer_bytes, params_bytes = _i(0), _i(0)
        self.lib.ps_decode_stack_sizes(ctypes.byref(layer_bytes), ctypes.byref(params_bytes))
        if layer_bytes.value != ctypes.sizeof(_LayerWeights) or params_bytes.value != ctypes.sizeof(_Params):
            raise KernelError("decode_stack: the host mirror of the kernel's parameter block is out of date")
        self.model, self.cache, self.device = model, cache, device
        spec = model.spec
        first = model.blocks[spec.schedule[0].layer]
        mp, fp = first.mixer.params, first.feed_forward.params
        self.H, self.I, self.V = spec.hidden_size, fp["inner_size"], spec.vocab_size
        self.n_heads, self.n_kv_heads, self.head_dim = mp["n_heads"], mp["n_kv_heads"], mp["head_dim"]
        self.window = mp.get("window") or 0
        self.scale = float(mp["scale"])
        self.act = _ACT_CODE[fp["activation"]]
        norm = first.norms["pre_mixer"].params
        self.eps, self.has_mean = float(norm["eps"]), bool(norm.get("has_mean", True))
        group = cache.groups[0]
        self.group = group
        rows = []
        for entry in spec.schedule:
            block = model.blocks[entry.layer]
            k_pool, v_pool = group.layer_views(entry.cache_layer)
            n1, n2 = block.norms["pre_mixer"], block.norms["pre_feed_forward"]
            rows.append(_LayerWeights(
                _ptr(n1.weight), _ptr(n1.bias), _ptr(n2.weight), _ptr(n2.bias),
                _ptr(block.mixer.w_qkv), _ptr(block.mixer.b_qkv), _ptr(block.mixer.w_out), _ptr(block.mixer.b_out),
                _ptr(block.feed_forward.w_up), _ptr(block.feed_forward.b_up),
                _ptr(block.feed_forward.w_down), _ptr(block.feed_forward.b_down),
                k_pool.data_ptr(), v_pool.data_ptr()))
        array = (_LayerWeights * len(rows))(*rows)
        raw = bytes(array)
        self.layers = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.n_layers = len(rows)
        table = model.positions.embedding_table()
        self.wpe = table
        self.n_positions = table.shape[0] if table is not None else (1 << 30)
        self.wte = model.embedding.table
        self.lm_head = model.head.table if model.head.table is not None else model.embedding.table
        B = self.MAX_BATCH
        q_width = self.n_heads * self.head_dim
        f32, bf16 = torch.float32, torch.bfloat16
        self.h = torch.empty(B, self.H, dtype=f32, device=device)
        self.xn = torch.empty(B, self.H, dtype=bf16, device=device)
        self.q = torch.empty(B, q_width, dtype=bf16, device=device)
        self.attn = torch.empty(B, q_width, dtype=bf16, device=device)
        self.inner = torch.empty(B, self.I, dtype=bf16, device=device)
        self.counters = torch.zeros(B * self.n_heads, dtype=torch.int32, device=device)
        self.best = torch.zeros(B, dtype=torch.int64, device=device)
        self.barrier = torch.zeros(64, dtype=torch.int32, device=device)
        self.skip_mask = 0          # timing aid (see csrc/decode_stack.cu); results are wrong when non-zero
        self.ctas_per_sm = int(os.environ.get("PAGEDSERVE_B200_STACK_CTAS", "0"))
        self.logits = None
        self.part_acc = self.part_ml = None
        self.sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.launches = 0

    # ------------------------------------------------------------------ qualification
    @classmethod
    def build_if_possible(cls, model, cache, device) -> Optional["DecodeStack"]:
        spec = model.spec
        if model.env.dtype != torch.bfloat16 or len(cache.groups) != 1 or cache.state:
            return None
        if spec.embedding.kind != "token_embedding" or spec.head.kind != "lm_head" or \
                spec.positions.kind not in ("learned_absolute", "none") or spec.final_norm.kind != "layernorm":
            return None
        reference = None
        for entry in spec.schedule:
            layer = spec.layers[entry.layer]
            if layer.block.kind != "pre_norm" or layer.mixer.kind != "causal_attention" or \
                    layer.feed_forward.kind != "dense_mlp" or any(n.kind != "layernorm" for n in layer.norms.values()):
                return None
            if not layer.mixer.params.get("write_cache", True):
                return None
            m, f, n = layer.mixer.params, layer.feed_forward.params, layer.norms["pre_mixer"].params
            n2 = layer.norms["pre_feed_forward"].params
            key = (m["hidden_size"], m["n_heads"], m["n_kv_heads"], m["head_dim"], m.get("window"), float(m["scale"]),
                   f["inner_size"], f["activation"], float(n["eps"]), n.get("has_mean", True),
                   float(n2["eps"]), n2.get("has_mean", True))
            if reference is None:
                reference = key
            elif key != reference:
                return None
        final = spec.final_norm.params
        if reference is None or (float(final["eps"]), final.get("has_mean", True)) != (reference[8], reference[9]):
            return None
        hidden, inner, head_dim = reference[0], reference[6], reference[3]
        if hidden % 8 or inner % 8 or head_dim % 16 or head_dim > 256 or (reference[1] * head_dim) % 8:
            return None
        return cls(model, cache, device)

    # ------------------------------------------------------------------ one call = n_steps decode steps
    def run(self, ctx, n_steps: int, want_logits: bool, do_sample: bool, sampled=None, history=None,
            step_counter=None, max_steps: int = 0, max_kv_len: int = 0):
        from pagedserve_b200.kernels.ops import Ops

        B = ctx.num_items
        if B > self.MAX_BATCH or ctx.num_tokens != B:
            raise KernelError("decode_stack takes decode-only batches of at most 64 requests")
        group = self.group
        chunk = Ops.attention_chunk_keys(self.head_dim, group.page_size)
        grid = self.sms * (self.ctas_per_sm or 3)
        chunks = max(1, -(-int(max_kv_len) // chunk))
        wanted = max(1, -(-grid // (B * self.n_heads)))
        split_chunks = max(1, -(-chunks // wanted))
        n_splits = -(-chunks // split_chunks)
        if n_splits > 1:
            need = B * self.n_heads * n_splits
            if self.part_acc is None or self.part_acc.shape[0] < need:
                self.part_acc = torch.empty(need, self.head_dim, dtype=torch.float32, device=self.device)
                self.part_ml = torch.empty(need, 2, dtype=torch.float32, device=self.device)
        logits = None
        if want_logits:
            logits = torch.empty(B, self.V, dtype=torch.float32, device=self.device)
        tok = 8 * (1 if B <= 8 else 2 if B <= 16 else 4 if B <= 32 else 8)
        stage = tok * (self.H + 8) * 2 <= self.STAGE_LIMIT
        params = _Params(
            B, self.H, self.n_heads, self.n_kv_heads, self.head_dim, self.I, self.V, self.n_layers, group.page_size,
            self.window, self.act, self.n_positions, 1 if self.has_mean else 0, 1 if stage else 0, n_steps,
            1 if want_logits else 0, 1 if do_sample else 0,
            self.eps, self.scale * 1.4426950408889634, group.page_stride,
            _ptr(self.layers), _ptr(self.wte), _ptr(self.wpe), _ptr(self.model.final_norm.weight),
            _ptr(self.model.final_norm.bias), _ptr(self.lm_head), _ptr(ctx.token_ids), _ptr(ctx.positions),
            _ptr(ctx.kv_len), _ptr(ctx.block_tables[0]), ctx.block_tables[0].stride(0),
            _ptr(self.h), _ptr(self.xn), _ptr(self.q), _ptr(self.attn), _ptr(self.inner), _ptr(self.part_acc),
            _ptr(self.part_ml), _ptr(self.counters), chunk, split_chunks, n_splits,
            _ptr(logits), _ptr(ctx.temperature if do_sample else None), _ptr(ctx.seed if do_sample else None),
            _ptr(self.best), _ptr(sampled), _ptr(history), _ptr(step_counter), max_steps,
            _ptr(self.barrier), _ptr(ctx.status), self.skip_mask, self.ctas_per_sm)
        status = self.lib.ps_decode_stack(ctypes.byref(params), _i(0),
                                          _p(torch.cuda.current_stream().cuda_stream))
        if status != 0:
            raise KernelError(f"decode_stack: launch failed with status {status}")
        self.launches += 1
        return logits
