"""Python wrappers of the CUDA entry points.

Every wrapper checks device, dtype, contiguity and sizes on the host, passes raw
pointers and the current CUDA stream to the ``extern "C"`` function and raises
:class:`KernelError` on a non-zero status.  There is no CPU fallback: a tensor
that is not on a CUDA device, or a library that cannot be built or loaded, is
an error.
"""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from pagedserve_b200.kernels.build import load as _load_library

PS_F32, PS_BF16 = 0, 1
_DTYPE_CODE = {torch.float32: PS_F32, torch.bfloat16: PS_BF16}
_ACT_CODE = {None: 0, "none": 0, "gelu_tanh": 1, "gelu_erf": 2}
_STATUS = {1: "bad argument", 2: "unsupported size or dtype", 3: "kernel launch failed"}

_c_void_p = ctypes.c_void_p
_c_int = ctypes.c_int
_c_float = ctypes.c_float
_c_ll = ctypes.c_longlong


class KernelError(RuntimeError):
    pass


def _ptr(tensor):
    """Device address of a tensor (or of a :class:`MappedHostBuffer`); None stays a null pointer."""
    if tensor is None:
        return None
    if isinstance(tensor, MappedHostBuffer):
        return tensor.device_ptr
    return tensor.data_ptr()


class MappedHostBuffer:
    """Page-locked host memory of ``count`` int32 that kernels write directly (see csrc/host_io.cu);
    ``array`` is the host's numpy view of it."""

    def __init__(self, lib, count: int):
        host, device = ctypes.c_void_p(), ctypes.c_void_p()
        _check(lib.ps_host_alloc_mapped(count * 4, ctypes.byref(host), ctypes.byref(device)), "host_alloc_mapped")
        self._lib = lib
        self.host_ptr = host.value
        self.device_ptr = device.value
        self.count = count
        self.array = np.ctypeslib.as_array((ctypes.c_int32 * count).from_address(self.host_ptr))

    def close(self):
        if self.host_ptr:
            self.array = None
            self._lib.ps_host_free(self.host_ptr)
            self.host_ptr = self.device_ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# Argument types of the entry points, declared once: ctypes then converts plain Python ints, floats and
# None itself, which is several times cheaper per call than building c_int / c_void_p objects.
_P, _I, _F, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
_SIGNATURES = {
    "core": {
        "ps_embed": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
        "ps_layernorm": [_P, _P, _I, _I, _P, _P, _F, _I, _P, _I, _P],
        "ps_gemm_simt": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
        "ps_kv_append": [_P, _P, _I, _P, _P, _P, _I, _P, _P, _L, _I, _I, _I, _I, _I, _P],
        "ps_paged_attention_simt": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
        "ps_sample": [_P, _I, _I, _I, _P, _P, _P, _I, _P, _P],
        "ps_step_shape": [_I, _P, _P, _P, _I, _I, _I, _I, _P],
        "ps_step_fill": [_I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _P, _I, _I, _I, _I, _P],
        "ps_step_begin": [_P, _P, _P, _P, _P, _P],
        "ps_step_end": [_P, _P, _P, _P, _P, _P, _I, _I, _P, _P, _P],
        "ps_host_alloc_mapped": [_L, _P, _P],
        "ps_host_free": [_P],
        "ps_copy_h2d": [_P, _P, _L, _P],
    },
    "bf16": {
        "ps_gemm_skinny": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                           _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "ps_gemm_skinny_fused": [_P, _I, _P, _P, _P, _F, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                 _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "ps_paged_attention_decode_checked": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                              _F, _I, _I, _P, _P, _P, _P, _P],
        "ps_paged_attention_decode_ex": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I,
                                         _I, _I, _F, _I, _I, _I, _P, _P, _P, _P, _P],
        "ps_prefill_attention": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F,
                                 _P],
    },
    "tc": {
        "ps_gemm_tc": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P],
        "ps_gemm_rows_tc": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I,
                            _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "ps_gemm_tc_qkv": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "ps_prefill_attention_tc": [_P, _I, _I, _P, _I, _P, _L, _L, _L, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I,
                                    _I, _I, _F, _I, _P, _P],
    },
}


def _declare(lib, name: str):
    for function, argtypes in _SIGNATURES[name].items():
        handle = getattr(lib, function)
        handle.argtypes = argtypes
        handle.restype = ctypes.c_int
    return lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle (the fast private lookup when torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _require(tensor: torch.Tensor, name: str, dtype=None):
    if not tensor.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")


def _check(status: int, what: str):
    if status != 0:
        raise KernelError(f"{what}: {_STATUS.get(status, f'status {status}')}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype not in _DTYPE_CODE:
        raise KernelError(f"unsupported dtype {dtype}")
    return _DTYPE_CODE[dtype]


class StepArena:
    """Memory for the tensors that live for one step only (activations, scratch).

    A step asks for the same sizes in the same order every time it runs, so its tensors are handed out from a
    few large chunks by moving an offset, which is set back when the next step begins. Nothing is given back to
    the allocator and, once the chunks have grown to the largest step, nothing is asked of it: a CUDA graph
    capture whose tensors came from the allocator's graph pool cost 6 to 14 ms and now and then 60 to 80 ms
    (fresh device memory for every tensor of the step), which a serving loop shows as one very long step.
    What a step returns to its caller is copied out of the arena first; tensors of the arena are valid until the
    next step starts on the same stream."""

    CHUNK_BYTES = 64 << 20
    ALIGN = 256

    def __init__(self):
        self.chunks = []             # uint8 tensors, never freed
        self.chunk = 0
        self.offset = 0

    def reset(self) -> None:
        self.chunk = 0
        self.offset = 0

    def mark(self):
        """The current place; ``release(mark)`` hands everything asked for since then out again (kernels run
        in stream order, so a later tensor may lie where an earlier, finished one lay)."""
        return (self.chunk, self.offset)

    def release(self, mark) -> None:
        self.chunk, self.offset = mark

    def empty(self, shape, dtype, device):
        count = 1
        for extent in shape:
            count *= int(extent)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        if nbytes == 0:
            return torch.empty(tuple(shape), dtype=dtype, device=device)
        size = -(-nbytes // self.ALIGN) * self.ALIGN
        while True:
            if self.chunk < len(self.chunks):
                chunk = self.chunks[self.chunk]
                start = self.offset + (-(chunk.data_ptr() + self.offset)) % self.ALIGN     # an aligned address
                if chunk.device == torch.device(device) and start + size <= chunk.numel():
                    piece = chunk[start:start + nbytes]
                    self.offset = start + size
                    return piece.view(dtype).view(tuple(shape))
                self.chunk += 1
                self.offset = 0
                continue
            if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                # a capture runs the step that an eager run made room for just before; if it asks for more
                # all the same, the graph's own pool serves it
                return torch.empty(tuple(shape), dtype=dtype, device=device)
            self.chunks.append(torch.empty(max(self.CHUNK_BYTES, size) + self.ALIGN, dtype=torch.uint8, device=device))


class Ops:
    """The kernel set for one compute dtype (``torch.float32`` or ``torch.bfloat16``)."""

    def __init__(self, dtype: torch.dtype):
        if dtype not in _DTYPE_CODE:
            raise KernelError(f"unsupported compute dtype {dtype}")
        self.dtype = dtype
        self.code = _DTYPE_CODE[dtype]
        self.core = _declare(_load_library("core"), "core")
        self.fast = _declare(_load_library("bf16"), "bf16") if dtype == torch.bfloat16 else None
        self._tc = None              # tcgen05 library, loaded when a product first needs it
        self.status = None
        self._counters = None        # zeroed int32 scratch of the split attention kernel
        self.launches = 0            # count of kernel launches issued through this object
        self.arena = None            # a StepArena once a runner has attached one: see ``empty``

    def empty(self, shape, dtype, device):
        """An uninitialised tensor that lives until the next step begins (from the step arena if a runner
        attached one, else from the allocator): what parts use for activations and kernels for scratch."""
        if self.arena is not None:
            return self.arena.empty(shape, dtype, device)
        return torch.empty(tuple(shape), dtype=dtype, device=device)

    # ------------------------------------------------------------------ embedding
    def embed(self, ids, positions, wte, wpe, out, status=None):
        """out[t] = wte[ids[t]] (+ wpe[positions[t]]) as float32 [T, H]."""
        T, H = out.shape
        _require(out, "out", torch.float32)
        _require(ids, "ids", torch.int32)
        _require(wte, "wte", self.dtype)
        if wpe is not None:
            _require(wpe, "wpe", self.dtype)
            _require(positions, "positions", torch.int32)
            if wpe.shape[1] != H:
                raise KernelError("wpe width does not match the hidden size")
        if wte.shape[1] != H or ids.numel() != T:
            raise KernelError("embed: shapes do not match")
        self.launches += 1
        _check(self.core.ps_embed(_ptr(ids), _ptr(positions if wpe is not None else None), _ptr(wte), _ptr(wpe),
                                  _ptr(out), T, H, wte.shape[0],
                                  wpe.shape[0] if wpe is not None else 0, self.code,
                                  _ptr(status), _stream()), "embed")
        return out

    # ------------------------------------------------------------------ norm
    def layernorm(self, x, gamma, beta, eps, out, rows=None, has_mean=True):
        """out[r] = norm(x[rows[r]] or x[r]); x float32 [*, H]; out compute dtype or float32."""
        _require(x, "x", torch.float32)
        _require(gamma, "gamma", torch.float32)
        H = x.shape[-1]
        n_rows = out.shape[0]
        if rows is not None:
            _require(rows, "rows", torch.int32)
            if rows.numel() != n_rows:
                raise KernelError("layernorm: rows and out disagree")
        elif x.shape[0] != n_rows:
            raise KernelError("layernorm: x and out disagree")
        if out.shape[-1] != H or gamma.numel() != H or (beta is not None and beta.numel() != H):
            raise KernelError("layernorm: widths disagree")
        if not x.is_contiguous() or not out.is_contiguous():
            raise KernelError("layernorm: tensors must be contiguous")
        self.launches += 1
        _check(self.core.ps_layernorm(_ptr(x), _ptr(rows), n_rows, H, _ptr(gamma), _ptr(beta),
                                      eps, 1 if has_mean else 0, _ptr(out),
                                      dtype_code(out.dtype), _stream()), "layernorm")
        return out

    # ------------------------------------------------------------------ matrix product
    def linear_simt(self, a, w, bias, out, act=None, accumulate=False):
        """out = act(a @ w.T + bias) on CUDA cores (float32 accumulation, fixed K order)."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError(f"linear: shapes do not match: a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
        _require(a, "a")
        _require(w, "w", a.dtype)
        _require(out, "out")
        if bias is not None:
            _require(bias, "bias", torch.float32)
            if bias.numel() != N:
                raise KernelError("linear: bias length")
        if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear: innermost stride must be 1")
        if accumulate and out.dtype != torch.float32:
            raise KernelError("linear: accumulate needs a float32 output")
        self.launches += 1
        _check(self.core.ps_gemm_simt(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias),
                                      _ptr(out), out.stride(0), M, N, K,
                                      dtype_code(a.dtype), dtype_code(out.dtype),
                                      _ACT_CODE[act], 1 if accumulate else 0, _stream()),
               "gemm_simt")
        return out

    def linear_skinny(self, a, w, bias, out, act=None, accumulate=False, kv=None):
        """Weight-streaming product for at most 64 rows of ``a`` (bfloat16 operands).  ``kv`` =
        (ctx, layer, q_width, kv_width, head_dim) sends the key and value columns of a packed q|k|v
        projection into the pages instead of ``out``."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError("linear_skinny: shapes do not match")
        _require(a, "a", torch.bfloat16)
        _require(w, "w", torch.bfloat16)
        _require(out, "out")
        if bias is not None:
            _require(bias, "bias", torch.float32)
        if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear_skinny: innermost stride must be 1")
        self.launches += 1
        _check(self.fast.ps_gemm_skinny(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias),
                                        _ptr(out), out.stride(0), M, N, K,
                                        dtype_code(out.dtype), _ACT_CODE[act],
                                        1 if accumulate else 0, *self._kv_arguments(kv, N), _stream()), "gemm_skinny")
        return out

    def linear_tc(self, a, w, bias, out, act=None, accumulate=False, status=None, bn=0):
        """tcgen05 / TMA / TMEM product (bfloat16 operands, float32 accumulation); any M."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError("linear_tc: shapes do not match")
        _require(a, "a", torch.bfloat16)
        _require(w, "w", torch.bfloat16)
        _require(out, "out")
        if bias is not None:
            _require(bias, "bias", torch.float32)
        if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear_tc: innermost stride must be 1")
        if self._tc is None:
            self._tc = _declare(_load_library("tc"), "tc")
        if status is None:
            status = self.status_flag(a.device)
        self.launches += 1
        _check(self._tc.ps_gemm_tc(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
                                   out.stride(0), M, N, K,
                                   dtype_code(out.dtype), _ACT_CODE[act],
                                   1 if accumulate else 0, _ptr(status), bn, _stream()), "gemm_tc")
        return out

    def linear_rows_tc(self, a, w, bias, out, act=None, accumulate=False, kv=None, status=None, splits=0):
        """tcgen05 product for at most 64 rows of ``a`` with the operands swapped: weight rows on the 128-row
        side of the MMA, K split over the CTAs of a thread-block cluster (csrc/gemm_rows_tc.cu).  ``kv`` as in
        :meth:`linear_skinny`; ``splits`` 0 lets the kernel choose."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError("linear_rows_tc: shapes do not match")
        _require(a, "a", torch.bfloat16)
        _require(w, "w", torch.bfloat16)
        _require(out, "out")
        if bias is not None:
            _require(bias, "bias", torch.float32)
        if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear_rows_tc: innermost stride must be 1")
        if self._tc is None:
            self._tc = _declare(_load_library("tc"), "tc")
        if status is None:
            status = self.status_flag(a.device)
        self.launches += 1
        _check(self._tc.ps_gemm_rows_tc(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
                                        out.stride(0), M, N, K, dtype_code(out.dtype), _ACT_CODE[act],
                                        1 if accumulate else 0, _ptr(status), splits,
                                        *self._kv_arguments(kv, N), _stream()), "gemm_rows_tc")
        return out

    @staticmethod
    def tc_ok(a, w):
        K = a.shape[1]
        return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    @staticmethod
    def skinny_ok(a, w):
        K = a.shape[1]
        return (a.shape[0] <= 64 and K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    FUSED_NORM_ROWS = 32          # most rows for which the norm is folded into the skinny product
    FUSED_NORM_COLUMNS = 16 * 2 * 148   # and most output columns

    def _fused_norm_ok(self, a, w):
        prologue = getattr(a.norm, "fused_prologue", lambda: None)()
        if prologue is None:
            return False                  # this norm cannot be written as the product's prologue
        # every CTA (16 output columns) recomputes the statistics: worth it only while the product is narrow
        rows = 8 if a.shape[0] <= 8 else 16 if a.shape[0] <= 16 else 32
        # the normed rows and the norm's scale and shift are staged in shared memory
        if rows * (a.shape[1] + 8) * 2 + 8 * a.shape[1] > 96 * 1024:
            return False
        # one CTA per 16 output columns, two CTAs per SM: beyond one wave of CTAs the repeated norm costs more
        # than a norm kernel of its own
        return (self.dtype == torch.bfloat16 and a.shape[0] <= self.FUSED_NORM_ROWS
                and w.shape[0] <= self.FUSED_NORM_COLUMNS
                and a.x.dtype == torch.float32 and prologue.weight.dtype == torch.float32
                and a.shape[1] % 8 == 0 and a.x.stride(0) % 4 == 0 and a.x.stride(1) == 1
                and w.stride(0) % 8 == 0 and w.stride(1) == 1 and w.dtype == torch.bfloat16
                and a.x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
                and prologue.weight.data_ptr() % 16 == 0
                and (prologue.bias is None or prologue.bias.data_ptr() % 16 == 0))

    @staticmethod
    def _kv_arguments(kv, N):
        """The cache-write arguments of a product's epilogue; ``kv`` None = no cache write."""
        if kv is None:
            return (None, None, 0, None, None, None, 0, N, 0, 1, 1)
        ctx, layer, q_width, kv_width, head_dim = kv
        return (_ptr(layer.k_pool), _ptr(layer.v_pool), layer.page_stride, _ptr(ctx.token_slot),
                _ptr(ctx.positions), _ptr(layer.block_table), layer.block_table.stride(0),
                q_width, kv_width, head_dim, layer.page_size)

    def status_flag(self, device) -> torch.Tensor:
        """The device int32 that kernels of this object set non-zero when a bounded wait ran out or an input
        was bad, unless the caller hands them a flag of its own."""
        if self.status is None:
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
        return self.status

    def reset_after_fault(self) -> None:
        """After a kernel gave up a wait: the split attention kernel's arrival counters may not be back at
        zero (the CTA that would have reset them stopped), and later steps would merge too early."""
        if self._counters is not None:
            self._counters.zero_()

    def linear_skinny_fused(self, a, w, bias, out, act=None, accumulate=False, kv=None):
        """out = act(norm(x)[rows] @ w.T + bias) with the norm computed inside the product's kernel
        (``a`` is a DeferredNorm); ``kv`` = (ctx, layer, q_width, kv_width, head_dim) also sends the key
        and value columns of the result straight into the pages."""
        norm = a.norm.fused_prologue()
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError("linear_skinny_fused: shapes do not match")
        _require(out, "out")
        kv_args = self._kv_arguments(kv, N)
        self.launches += 1
        _check(self.fast.ps_gemm_skinny_fused(
            _ptr(a.x), a.x.stride(0), _ptr(a.rows), _ptr(norm.weight), _ptr(norm.bias),
            float(norm.eps), 1 if norm.has_mean else 0,
            _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(0), M, N,
            K, dtype_code(out.dtype), _ACT_CODE[act], 1 if accumulate else 0,
            *kv_args, _stream()), "gemm_skinny_fused")
        return out

    def linear_qkv(self, a, w, bias, out, ctx, layer, q_width, kv_width, head_dim, scatter=True):
        """The packed q|k|v projection.  Returns True when the key and value columns were written into
        the pages by the product's own epilogue (then no separate cache write is needed)."""
        if scatter and layer.k_pool is not None and self.dtype == torch.bfloat16 and head_dim % 16 == 0:
            if hasattr(a, "materialize") and self._fused_norm_ok(a, w):
                self.linear_skinny_fused(a, w, bias, out, kv=(ctx, layer, q_width, kv_width, head_dim))
                return True
            if hasattr(a, "materialize"):
                a = a.materialize()
            from pagedserve_b200.kernels import tensorcore

            # a few dozen rows of a large matrix: the few-rows tcgen05 product writes the pages from its epilogue
            if tensorcore.prefers_rows(self, a, w) and q_width % 4 == 0 and kv_width % 4 == 0:
                self.linear_rows_tc(a, w, bias, out, kv=(ctx, layer, q_width, kv_width, head_dim))
                return True
            # many rows: the tcgen05 product, whose TMA-store epilogue sends the key and value columns to the pages
            if tensorcore.prefers_tc(self, a, w):
                if (q_width % 64 == 0 and head_dim % 8 == 0 and out.data_ptr() % 16 == 0
                        and out.stride(0) % 8 == 0 and out.dtype == torch.bfloat16):
                    self.linear_tc_qkv(a, w, bias, out, ctx, layer, q_width, kv_width, head_dim)
                    return True
            elif self.skinny_ok(a, w):
                self.linear_skinny(a, w, bias, out, kv=(ctx, layer, q_width, kv_width, head_dim))
                return True
        self.linear(a, w, bias, out)
        return False

    def linear_tc_qkv(self, a, w, bias, out, ctx, layer, q_width, kv_width, head_dim):
        """tcgen05 q|k|v projection: query columns to ``out``, key and value columns into the pages."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError("linear_tc_qkv: shapes do not match")
        _require(a, "a", torch.bfloat16)
        _require(w, "w", torch.bfloat16)
        _require(out, "out", torch.bfloat16)
        if self._tc is None:
            self._tc = _declare(_load_library("tc"), "tc")
        self.launches += 1
        _check(self._tc.ps_gemm_tc_qkv(
            _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(0), M, N, K,
            _ptr(self.status_flag(a.device)), _ptr(layer.k_pool), _ptr(layer.v_pool), layer.page_stride,
            _ptr(ctx.token_slot), _ptr(ctx.positions), _ptr(layer.block_table), layer.block_table.stride(0),
            q_width, kv_width, head_dim, layer.page_size, _stream()), "gemm_tc_qkv")
        return out

    def linear(self, a, w, bias, out, act=None, accumulate=False):
        """The matrix product of the model: float32 runs on FFMA, bfloat16 on tensor cores.
        ``a`` may be a DeferredNorm: it is folded into the product where a kernel can, else evaluated."""
        if hasattr(a, "materialize"):
            if self._fused_norm_ok(a, w):
                return self.linear_skinny_fused(a, w, bias, out, act, accumulate)
            a = a.materialize()
        if self.dtype == torch.float32:
            return self.linear_simt(a, w, bias, out, act, accumulate)
        from pagedserve_b200.kernels import tensorcore

        return tensorcore.linear(self, a, w, bias, out, act, accumulate)

    # ------------------------------------------------------------------ cache + attention
    def kv_append(self, k_src, v_src, token_item, positions, block_table, k_pool, v_pool, page_stride,
                  n_kv_heads, head_dim, page_size):
        """Copy this step's K/V rows ([T, n_kv_heads*head_dim] views) into their pages."""
        T = k_src.shape[0]
        _require(k_src, "k", self.dtype)
        _require(v_src, "v", self.dtype)
        _require(k_pool, "k_pool", self.dtype)
        if k_src.stride(1) != 1 or v_src.stride(1) != 1 or k_src.stride(0) != v_src.stride(0):
            raise KernelError("kv_append: k and v must be row views with equal row stride")
        self.launches += 1
        _check(self.core.ps_kv_append(_ptr(k_src), _ptr(v_src), k_src.stride(0), _ptr(token_item),
                                      _ptr(positions), _ptr(block_table), block_table.stride(0),
                                      _ptr(k_pool), _ptr(v_pool), page_stride, T,
                                      n_kv_heads, head_dim, page_size,
                                      self.code, _stream()), "kv_append")

    def paged_attention_simt(self, q, out, k_pool, v_pool, page_stride, token_item, positions, block_table,
                             n_heads, n_kv_heads, head_dim, page_size, window, scale):
        """out[t, h] = softmax(q[t,h] . K[<=pos]) V over the request's pages; CUDA cores."""
        T = q.shape[0]
        _require(q, "q", self.dtype)
        _require(out, "out", self.dtype)
        if q.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("attention: innermost stride must be 1")
        self.launches += 1
        _check(self.core.ps_paged_attention_simt(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pool), _ptr(v_pool),
            page_stride, _ptr(token_item), _ptr(positions), _ptr(block_table),
            block_table.stride(0), T, n_heads, n_kv_heads, head_dim,
            page_size, window or 0, scale, self.code, _stream()),
            "paged_attention_simt")
        return out

    @staticmethod
    def attention_chunk_keys(head_dim, page_size):
        """Keys per shared-memory chunk of the split attention kernel (mirrors the CUDA side)."""
        keys = 128 if head_dim <= 64 else 64 if head_dim <= 128 else 32
        return max(keys, page_size)

    def attention_split_plan(self, T, n_heads, head_dim, page_size, max_kv_len, target_ctas=1184):
        """(split_tiles, n_splits): how the keys of a token are cut over CTAs.

        A split is a whole number of chunks; splits are made as short as one chunk while the grid
        stays below ``target_ctas`` CTAs (8 per SM), so that small batches still fill the GPU."""
        chunk = self.attention_chunk_keys(head_dim, page_size)
        chunks = max(1, -(-int(max_kv_len) // chunk))
        wanted = max(1, target_ctas // max(1, T * n_heads))
        split_chunks = max(1, -(-chunks // wanted))
        n_splits = -(-chunks // split_chunks)
        return split_chunks * chunk // 32, n_splits

    def attention_cluster_plan(self, T, n_heads, head_dim, page_size, max_kv_len, target_ctas=1184, largest=8):
        """(split_tiles, cluster) if the splits of a (token, head) can be one thread-block cluster of at most
        ``largest`` CTAs without leaving much of the GPU idle, else None."""
        chunk = self.attention_chunk_keys(head_dim, page_size)
        chunks = max(1, -(-int(max_kv_len) // chunk))
        wanted = min(chunks, max(1, target_ctas // max(1, T * n_heads)))
        if wanted > largest and chunks > 2 * largest:
            return None                                  # a long context at a small batch: more splits pay
        cluster = 1
        while cluster < min(largest, wanted):
            cluster *= 2                                 # the power of two at or above the wanted splits ...
        if cluster > 1 and T * n_heads * cluster > target_ctas:
            cluster //= 2                                # ... unless that makes more CTAs than are resident at once
        split_chunks = -(-chunks // cluster)
        return split_chunks * chunk // 32, cluster

    def paged_attention_decode(self, q, out, k_pool, v_pool, page_stride, token_item, positions, block_table,
                               n_heads, n_kv_heads, head_dim, page_size, window, scale, max_kv_len,
                               target_ctas=1184, status=None, q_start=None, kv_len=None, merge="global",
                               largest_cluster=8, token_row=None):
        """Split-key attention for few query tokens (bfloat16).  ``max_kv_len`` bounds the context of
        every token in the call; it fixes the grid, so a CUDA graph passes the model's maximum.
        ``q_start`` / ``kv_len`` (the step's per-item arrays) let the kernel fetch keys older than this step
        before the kernel that precedes it has finished.  ``merge``: "global" (the splits of a token and head
        merge through scratch in global memory) or "cluster" (they are a thread-block cluster and merge
        through shared memory; falls back to "global" where more than ``largest_cluster`` splits pay).
        ``block_table`` rows are indexed by ``token_row[t]`` (a table kept by request slot) or, without it, by
        ``token_item[t]``."""
        T = q.shape[0]
        _require(q, "q", torch.bfloat16)
        _require(out, "out", torch.bfloat16)
        plan = None
        if merge == "cluster":
            plan = self.attention_cluster_plan(T, n_heads, head_dim, page_size, max_kv_len, target_ctas,
                                               largest_cluster)
        part_acc = part_ml = counters = None
        if plan is not None:
            split_tiles, cluster = plan
            n_splits = cluster
        else:
            cluster = 1
            split_tiles, n_splits = self.attention_split_plan(T, n_heads, head_dim, page_size, max_kv_len,
                                                              target_ctas)
            if n_splits > 1:
                if self._counters is None or self._counters.numel() < T * n_heads:
                    self._counters = torch.zeros(max(1024, T * n_heads), dtype=torch.int32, device=q.device)
                counters = self._counters
                part_acc = self.empty((T * n_heads * n_splits, head_dim), torch.float32, q.device)
                part_ml = self.empty((T * n_heads * n_splits, 2), torch.float32, q.device)
        self.launches += 1
        _check(self.fast.ps_paged_attention_decode_ex(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pool), _ptr(v_pool),
            page_stride, _ptr(token_item), _ptr(token_row), _ptr(positions), _ptr(block_table),
            block_table.stride(0), _ptr(q_start), _ptr(kv_len), T, n_heads, n_kv_heads, head_dim,
            page_size, window or 0, scale, split_tiles, n_splits, cluster,
            _ptr(part_acc), _ptr(part_ml), _ptr(counters), _ptr(status), _stream()), "paged_attention_decode")
        return out

    def prefill_attention(self, q, out, k_pool, v_pool, page_stride, q_start, kv_len, block_table, first_item,
                          n_items, max_blocks, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                          item_row=None):
        """Tensor-core causal attention of prompt portions (bfloat16): items ``first_item ..`` of the step,
        ``max_blocks`` >= the number of 64-query blocks they make up.  ``q`` / ``out`` are the step's flat
        token arrays (row 0 = token 0).  ``item_row``: the block-table row of each item (a table kept by request
        slot); without it item i uses row i."""
        _require(q, "q", torch.bfloat16)
        _require(out, "out", torch.bfloat16)
        if head_dim > 128:
            raise KernelError("prefill_attention: head sizes above 128 are not supported")
        self.launches += 1
        _check(self.fast.ps_prefill_attention(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_pool), _ptr(v_pool),
            page_stride, _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0), _ptr(item_row),
            first_item, n_items, max_blocks, n_heads, n_kv_heads,
            head_dim, page_size, window or 0, scale, _stream()),
            "prefill_attention")
        return out

    @staticmethod
    def prefill_tc_ok(head_dim, page_size, q, out, pool):
        return (head_dim in (64, 128) and 8 <= page_size <= 64 and pool is not None and q.stride(0) % 8 == 0
                and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)

    def prefill_attention_tc(self, q, out, pool, cache_layer_local, q_start, kv_len, block_table, first_item,
                             n_items, max_blocks, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                             status=None, row_threads=0, item_row=None):
        """tcgen05 causal attention of prompt portions (bfloat16, head size 64 or 128).  ``pool`` is the cache
        group's whole pool ``[pages, layers, 2, kv heads, page size, head dim]``; ``cache_layer_local`` the
        layer's index inside it; ``max_blocks`` >= the number of 128-query blocks of the items.
        ``row_threads``: 1 or 2 threads per query row (0: the kernel's launcher decides)."""
        _require(q, "q", torch.bfloat16)
        _require(out, "out", torch.bfloat16)
        if self._tc is None:
            self._tc = _declare(_load_library("tc"), "tc")
        if status is None:
            status = self.status_flag(q.device)
        pages, layers, two, kv_heads, ps, hd = pool.shape
        rows_per_tensor = kv_heads * ps                      # rows of one (layer, k or v) inside a page
        page_rows = layers * 2 * rows_per_tensor
        self.launches += 1
        _check(self._tc.ps_prefill_attention_tc(
            _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(pool), pages * page_rows,
            (cache_layer_local * 2) * rows_per_tensor, (cache_layer_local * 2 + 1) * rows_per_tensor, page_rows,
            _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0), _ptr(item_row), first_item,
            n_items, max_blocks, n_heads, n_kv_heads, head_dim, page_size, window or 0, scale, row_threads,
            _ptr(status), _stream()),
            "prefill_attention_tc")
        return out

    def attention(self, q, k, v, out, ctx, layer, n_heads, n_kv_heads, head_dim, window, scale,
                  write_cache=True):
        """Write the step's keys and values into the pages, then attend from the pages."""
        if write_cache:
            self.kv_append(k, v, ctx.token_slot, ctx.positions, layer.block_table, layer.k_pool, layer.v_pool,
                           layer.page_stride, n_kv_heads, head_dim, layer.page_size)
        if self.dtype == torch.float32 or head_dim % 16 != 0:
            # the CUDA-core kernel takes every head size; the tensor-core kernels want multiples of 16
            return self.paged_attention_simt(q, out, layer.k_pool, layer.v_pool, layer.page_stride,
                                             ctx.token_slot, ctx.positions, layer.block_table, n_heads,
                                             n_kv_heads, head_dim, layer.page_size, window, scale)
        from pagedserve_b200.kernels import tensorcore

        return tensorcore.attention(self, q, out, ctx, layer, n_heads, n_kv_heads, head_dim, window, scale)

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, seed, position, out, pos_offset=0):
        """out[r] = argmax (temperature 0) or a Gumbel-max draw keyed by (seed[r], position[r] + pos_offset);
        logits float32 [R, V]."""
        R, V = logits.shape
        _require(logits, "logits", torch.float32)
        _require(out, "out", torch.int32)
        if temperature is not None:
            _require(temperature, "temperature", torch.float32)
            _require(seed, "seed", torch.int64)
            _require(position, "position", torch.int32)
        self.launches += 1
        _check(self.core.ps_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature),
                                   _ptr(seed), _ptr(position), pos_offset, _ptr(out), _stream()),
               "sample")
        return out

    def mapped_host_buffer(self, count: int) -> MappedHostBuffer:
        """``count`` int32 of page-locked host memory that kernels can write (a result the host reads in
        place after a stream synchronisation, without a copy of its own)."""
        return MappedHostBuffer(self.core, count)

    def copy_h2d(self, dst: torch.Tensor, src_host_ptr: int, nbytes: int) -> None:
        """One asynchronous copy of ``nbytes`` from page-locked host memory into ``dst`` on the current
        stream (the plain runtime call: a fraction of the host time of a tensor ``copy_``)."""
        _check(self.core.ps_copy_h2d(dst.data_ptr(), src_host_ptr, nbytes, _stream()), "copy_h2d")

    # ------------------------------------------------------------------ the host side of a step, natively
    def step_shape(self, counts, starts, want_counts, long_entry, pad, pad_short, pad_long):
        """(T, I, R, short items, short tokens, long blocks, real rows, longest entry, longest context) of the
        flat batch that ``engine.batch.arrange_step`` would lay out; ``counts`` / ``starts`` int64 and
        ``want_counts`` int32 per entry in the caller's order (host arrays, no device work)."""
        shape = np.empty(9, dtype=np.int32)
        _check(self.core.ps_step_shape(len(counts), counts.ctypes.data, starts.ctypes.data, want_counts.ctypes.data,
                                       long_entry, 1 if pad else 0, pad_short, pad_long, shape.ctypes.data),
               "step_shape")
        return shape.tolist()

    def step_fill(self, counts, starts, want_counts, tokens, slots, wants, long_entry, pad, pad_short, pad_long,
                  scratch_slot, vocab_size, staging_ptr, layout):
        """Write slots, item starts, wanted rows and token ids of the flat batch into the step's staging buffer
        (``staging_ptr``: host address) at ``layout``'s offsets.  Returns None, or the first token id outside
        the vocabulary."""
        bad = ctypes.c_longlong(0)
        status = self.core.ps_step_fill(len(counts), counts.ctypes.data, starts.ctypes.data, want_counts.ctypes.data,
                                        tokens.ctypes.data, slots.ctypes.data, wants.ctypes.data, long_entry,
                                        1 if pad else 0, pad_short, pad_long, scratch_slot, vocab_size, staging_ptr,
                                        layout.item_slot, layout.q_start, layout.logit_rows, layout.token_ids,
                                        ctypes.addressof(bad))
        if status == 1 and (bad.value < 0 or bad.value >= vocab_size):
            return bad.value
        _check(status, "step_fill")
        return None

    def step_begin(self, slots, layout, meta, status=None):
        """The first kernel of a step: apply the uploaded corrections to the slot store (``slots``, a
        :class:`pagedserve_b200.cache.slots.SlotStore`) and derive the step's per-token and per-item arrays
        in ``meta`` (the packed metadata buffer laid out by ``layout``) from the slots' state."""
        self.launches += 1
        _check(self.core.ps_step_begin(_ptr(slots.store), slots.layout_words.ctypes.data, _ptr(meta),
                                       layout.words.ctypes.data, _ptr(status), _stream()), "step_begin")

    def step_end(self, slots, layout, meta, sampled, history, max_steps, status=None, status_index=None):
        """The last kernel of a decode step that sampled on the device: the sampled tokens go into the slots
        (the next step's inputs if it feeds back) and into ``history``; ``status`` (device int32) is copied to
        ``history[status_index]`` for the host to read with the tokens."""
        B = sampled.numel()
        self.launches += 1
        copy_to = None if status is None else _ptr(history) + 4 * status_index
        _check(self.core.ps_step_end(_ptr(slots.store), slots.layout_words.ctypes.data, _ptr(meta),
                                     layout.words.ctypes.data, _ptr(sampled), _ptr(history), B, max_steps,
                                     _ptr(status), copy_to, _stream()), "step_end")
