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
_ACT_CODE = {None: 0, "none": 0, "gelu_tanh": 1, "gelu_erf": 2, "relu_squared": 3, "silu": 4, "tanh": 5}
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
        "ps_paged_attention_simt": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _F, _P,
                                    _I, _P],
        "ps_rotary_cache_write": [_P, _I, _P, _I, _P, _I, _P, _I, _I, _P, _P, _P, _I, _P, _P, _L, _I, _I, _I, _I, _I,
                                  _I, _P],
        "ps_token_shift_mix": [_P, _I, _P, _I, _P, _L, _I, _P, _P, _P, _P, _L, _I, _I, _I, _I, _P],
        "ps_wkv_prepare": [_P, _I, _P, _F, _P, _P, _L, _I, _P, _P, _P, _P, _I, _I, _P, _I, _P, _I, _P, _L, _I, _P, _I, _I,
                           _I, _I, _P],
        "ps_wkv_recurrence": [_P, _P, _P, _P, _P, _I, _P, _P, _F, _P, _I, _I, _P, _L, _I, _P, _P, _P, _I, _I, _I, _I,
                              _I, _P],
        "ps_sample": [_P, _I, _I, _I, _P, _P, _P, _I, _P, _P],
        "ps_embed_pair": [_P, _P, _P, _P, _P, _P, _F, _P, _I, _L, _L, _P, _P, _I, _I, _I, _I, _P, _P],
        "ps_hyper_begin": [_P, _P, _P, _P, _P, _L, _I, _P],
        "ps_hyper_step": [_P, _P, _P, _P, _P, _P, _L, _I, _P],
        "ps_latent_prepare": [_P, _I, _P, _I, _P, _F, _P, _I, _P, _P, _P, _I, _P, _L, _I, _P, _I, _I, _I, _I, _I, _I,
                              _I, _P],
        "ps_sigmoid_gate": [_P, _I, _P, _I, _I, _I, _I, _I, _P],
        "ps_moe_route": [_P, _I, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _F, _I, _I, _P, _P],
        "ps_moe_gate_mul": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _P],
        "ps_head_norm_rotary_cache_write": [_P, _I, _P, _I, _P, _I, _P, _P, _F, _P, _I, _I, _P, _P, _P, _I, _P, _P, _L,
                                            _I, _I, _I, _I, _I, _I, _I, _F, _P],
        "ps_group_rms_norm": [_P, _L, _I, _P, _I, _I, _I, _P, _F, _P, _L, _I, _P],
        "ps_post_norm_add": [_P, _P, _I, _I, _I, _P, _F, _P, _I, _P, _L, _I, _P, _P],
        "ps_depth_begin": [_P, _P, _P, _I, _P, _L, _P],
        "ps_mingru_scan": [_P, _L, _I, _P, _L, _P, _P, _I, _P, _L, _I, _I, _P],
        "ps_short_conv": [_P, _L, _P, _I, _I, _I, _P, _L, _P, _P, _P, _P, _L, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P],
        "ps_short_conv_keep": [_P, _L, _I, _I, _P, _L, _P, _P, _I, _P],
        "ps_moe_plan": [_P, _P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P],
        "ps_moe_gather": [_P, _I, _P, _P, _I, _I, _I, _I, _P],
        "ps_moe_gate_mul_rows": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _F, _P],
        "ps_moe_combine": [_P, _I, _P, _I, _P, _I, _I, _I, _P],
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
        "ps_gemm_skinny_grouped": [_P, _I, _L, _P, _I, _P, _P, _I, _L, _I, _I, _I, _I, _I, _I, _I, _P],
        "ps_paged_attention_decode_checked": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I,
                                              _F, _I, _I, _P, _P, _P, _P, _P],
        "ps_paged_attention_decode_ex": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I,
                                         _I, _I, _F, _I, _I, _I, _P, _P, _P, _P, _F, _P, _P],
        "ps_shared_position_attention": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _P, _I, _P],
        "ps_prefill_attention": [_P, _I, _P, _I, _P, _P, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F,
                                 _F, _P, _P],
    },
    "tc": {
        "ps_gemm_tc": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P],
        "ps_gemm_rows_tc": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I,
                            _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "ps_gemm_tc_groups": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
        "ps_gemm_tc_experts": [_P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P],
        "ps_gemm_tc_qkv": [_P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "ps_prefill_attention_tc": [_P, _I, _I, _P, _I, _P, _L, _L, _L, _L, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I,
                                    _I, _I, _F, _I, _P, _F, _P, _P],
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

    GROUPED_ROWS = 32             # most rows for which equal products run as one grouped launch

    def linear_grouped(self, a, w, out, act=None, act_from_group=0, max_rows=None):
        """``out[g] = a[g] @ w[g * cols:(g + 1) * cols].T`` for every group g: ``a`` [G, M, K], ``w`` the stacked
        weights [G * cols, K], ``out`` [G, M, cols]; ``act`` is applied to the groups from ``act_from_group`` on.
        Few rows in bfloat16 run as one launch of the weight-streaming kernel (up to ``max_rows``, at most 64;
        default GROUPED_ROWS: large matrices do better as products of their own from there); everything else as G
        products."""
        groups, M, K = a.shape
        cols = out.shape[2]
        if w.shape != (groups * cols, K) or out.shape[:2] != (groups, M):
            raise KernelError("linear_grouped: shapes do not match")
        one_launch = (self.dtype == torch.bfloat16 and a.dtype == torch.bfloat16
                      and M <= min(64, max_rows or self.GROUPED_ROWS)
                      and cols % 16 == 0 and K % 8 == 0 and a.stride(2) == 1 and out.stride(2) == 1
                      and w.stride(1) == 1 and a.stride(1) % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
                      and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
        if not one_launch and act is None and self._column_groups_ok(a, w, out):
            return self.linear_column_groups(a, w, out)
        if not one_launch:
            for g in range(groups):
                self.linear(a[g], w[g * cols:(g + 1) * cols], None, out[g], act=act if g >= act_from_group else None)
            return out
        _require(w, "w", torch.bfloat16)
        _require(out, "out")
        self.launches += 1
        _check(self.fast.ps_gemm_skinny_grouped(_ptr(a), a.stride(1), a.stride(0), _ptr(w), w.stride(0), None,
                                                _ptr(out), out.stride(1), out.stride(0), M, cols, groups, K,
                                                dtype_code(out.dtype), _ACT_CODE[act], act_from_group, _stream()),
               "gemm_skinny_grouped")
        return out

    def _column_groups_ok(self, a, w, out):
        """Whether the groups of a grouped product are column blocks of two row-major matrices that the tcgen05
        kernel can walk in one launch: many rows, bfloat16, and TMA's alignment."""
        groups, M, K = a.shape
        return (self.dtype == torch.bfloat16 and a.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and M > 64 and groups > 1 and a.stride(2) == 1 and out.stride(2) == 1 and w.is_contiguous()
                and a.stride(0) >= K and a.stride(0) % 8 == 0 and a.stride(1) % 8 == 0 and K % 8 == 0
                and a.stride(1) >= (groups - 1) * a.stride(0) + K
                and out.stride(0) >= out.shape[2] and out.stride(1) >= (groups - 1) * out.stride(0) + out.shape[2]
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def linear_column_groups(self, a, w, out, status=None):
        """The grouped product where group g's rows are the columns ``[g * a.stride(0), + K)`` of one row-major
        matrix and its results the columns ``[g * out.stride(0), + cols)`` of another (the heads of a layer): one
        launch of the tcgen05 kernel over (row tile, group) pairs (csrc/gemm_tc.cu: ColumnGroups)."""
        groups, M, K = a.shape
        cols = out.shape[2]
        if self._tc is None:
            self._tc = _declare(_load_library("tc"), "tc")
        if status is None:
            status = self.status_flag(a.device)
        self.launches += 1
        _check(self._tc.ps_gemm_tc_groups(_ptr(a), a.stride(1), _ptr(w), w.stride(0), _ptr(out), out.stride(1), M, cols,
                                          K, groups, a.stride(0), out.stride(0), dtype_code(out.dtype), _ptr(status),
                                          _stream()), "gemm_tc_groups")
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
                             n_heads, n_kv_heads, head_dim, page_size, window, scale, softcap=None, sink=None):
        """out[t, h] = softmax(q[t,h] . K[<=pos]) V over the request's pages; CUDA cores.  ``softcap``:
        scores become softcap * tanh(score / softcap); ``sink``: float32 [n_heads], exp(sink[h]) joins the
        softmax's denominator."""
        if sink is not None:
            _require(sink, "sink", torch.float32)
            if sink.numel() != n_heads:
                raise KernelError("attention: one sink per query head")
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
            page_size, window or 0, scale, float(softcap or 0.0), _ptr(sink), self.code, _stream()),
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
                               largest_cluster=8, token_row=None, softcap=None, sink=None):
        """Split-key attention for few query tokens (bfloat16).  ``max_kv_len`` bounds the context of
        every token in the call; it fixes the grid, so a CUDA graph passes the model's maximum.
        ``q_start`` / ``kv_len`` (the step's per-item arrays) let the kernel fetch keys older than this step
        before the kernel that precedes it has finished.  ``merge``: "global" (the splits of a token and head
        merge through scratch in global memory) or "cluster" (they are a thread-block cluster and merge
        through shared memory; falls back to "global" where more than ``largest_cluster`` splits pay).
        ``block_table`` rows are indexed by ``token_row[t]`` (a table kept by request slot) or, without it, by
        ``token_item[t]``.  ``softcap`` / ``sink`` as in :meth:`paged_attention_simt`."""
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
            _ptr(part_acc), _ptr(part_ml), _ptr(counters), _ptr(status), float(softcap or 0.0), _ptr(sink),
            _stream()), "paged_attention_decode")
        return out

    def prefill_attention(self, q, out, k_pool, v_pool, page_stride, q_start, kv_len, block_table, first_item,
                          n_items, max_blocks, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                          item_row=None, softcap=None, sink=None):
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
            head_dim, page_size, window or 0, scale, float(softcap or 0.0), _ptr(sink), _stream()),
            "prefill_attention")
        return out

    def shared_position_attention(self, q, out, k_pool, v_pool, page_stride, positions, block_table, token_row,
                                  heads, head_dim, page_size, window, scale, max_kv_len=None):
        """Attention of single tokens whose ``heads`` query heads all read one key/value head (bfloat16, head
        sizes that are multiples of 16 up to 128): the heads of a token are the query rows of one tile, so its
        keys are fetched once.  ``q`` / ``out`` [T, heads * head_dim]; token t stands at ``positions[t]`` and
        reads the pages of block-table row ``token_row[t]``.  With few tokens the key tiles of a token are shared
        out over several CTAs (a rule of T and ``max_kv_len``, the longest context any token of the call may have)
        whose partial results a second kernel merges."""
        T = q.shape[0]
        _require(q, "q", torch.bfloat16)
        _require(out, "out", torch.bfloat16)
        if (q.shape[1] != heads * head_dim or out.shape != q.shape or not q.is_contiguous()
                or not out.is_contiguous()):
            raise KernelError("shared_position_attention: q and out must be contiguous [T, heads * head_dim]")
        extent = abs(window or 0)                                     # a chunked mask (negative) bounds the keys alike
        seen = min(max_kv_len, extent) if (extent and max_kv_len) else (max_kv_len or extent or 0)
        tiles = -(-seen // 64) + 1 if seen else 1                      # 64-key tiles a token can touch
        splits = max(1, min(8, 296 // max(T, 1), tiles)) if heads <= 64 else 1
        partial = self.empty((T * splits * heads * (head_dim + 2),), torch.float32, q.device) if splits > 1 else None
        self.launches += 2 if splits > 1 else 1
        _check(self.fast.ps_shared_position_attention(
            _ptr(q), head_dim, _ptr(out), head_dim, _ptr(k_pool), _ptr(v_pool), page_stride, _ptr(positions),
            _ptr(block_table), block_table.stride(0), _ptr(token_row), T, heads, head_dim, page_size, window or 0,
            scale, _ptr(partial), splits, _stream()), "shared_position_attention")
        return out

    @staticmethod
    def prefill_tc_ok(head_dim, page_size, q, out, pool):
        return (head_dim in (64, 128) and 8 <= page_size <= 64 and pool is not None and q.stride(0) % 8 == 0
                and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)

    def prefill_attention_tc(self, q, out, pool, cache_layer_local, q_start, kv_len, block_table, first_item,
                             n_items, max_blocks, n_heads, n_kv_heads, head_dim, page_size, window, scale,
                             status=None, row_threads=0, item_row=None, softcap=None, sink=None):
        """tcgen05 causal attention of prompt portions (bfloat16, head size 64 or 128).  ``pool`` is the cache
        group's whole pool ``[pages, layers, planes, kv heads, page size, head dim]`` (one plane: the values are the keys); ``cache_layer_local`` the
        layer's index inside it; ``max_blocks`` >= the number of 128-query blocks of the items.
        ``row_threads``: 1 or 2 threads per query row (0: the kernel's launcher decides)."""
        _require(q, "q", torch.bfloat16)
        _require(out, "out", torch.bfloat16)
        if self._tc is None:
            self._tc = _declare(_load_library("tc"), "tc")
        if status is None:
            status = self.status_flag(q.device)
        pages, layers, planes, kv_heads, ps, hd = pool.shape
        rows_per_tensor = kv_heads * ps                      # rows of one (layer, k or v) inside a page
        page_rows = layers * planes * rows_per_tensor
        self.launches += 1
        _check(self._tc.ps_prefill_attention_tc(
            _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(pool), pages * page_rows,
            (cache_layer_local * planes) * rows_per_tensor,
            (cache_layer_local * planes + planes - 1) * rows_per_tensor, page_rows,
            _ptr(q_start), _ptr(kv_len), _ptr(block_table), block_table.stride(0), _ptr(item_row), first_item,
            n_items, max_blocks, n_heads, n_kv_heads, head_dim, page_size, window or 0, scale, row_threads,
            _ptr(status), float(softcap or 0.0), _ptr(sink), _stream()),
            "prefill_attention_tc")
        return out

    def attention(self, q, k, v, out, ctx, layer, n_heads, n_kv_heads, head_dim, window, scale,
                  write_cache=True, softcap=None, sink=None, chunk=None):
        """Write the step's keys and values into the pages, then attend from the pages.  ``softcap`` and
        ``sink`` as in :meth:`paged_attention_simt`.  Besides "no later key", a query sees the last ``window``
        keys, or (``chunk`` C instead of a window) the keys j of its own run of C positions,
        ``j // C == i // C``, runs counted from position 0 of the sequence; neither: every earlier key.  Below
        this method the two travel as one integer: the window, or minus the chunk."""
        if chunk:
            if window:
                raise KernelError("attention: a window or a chunked mask, not both")
            window = -int(chunk)
        if write_cache:
            self.kv_append(k, v, ctx.token_slot, ctx.positions, layer.block_table, layer.k_pool, layer.v_pool,
                           layer.page_stride, n_kv_heads, head_dim, layer.page_size)
        from pagedserve_b200.kernels import tensorcore

        if self.dtype == torch.float32 or head_dim % 16 != 0 or head_dim > 256:
            # the CUDA-core kernel takes every head size (up to 1,024); the tensor-core kernels want multiples of 16
            # up to 256
            return self.paged_attention_simt(q, out, layer.k_pool, layer.v_pool, layer.page_stride,
                                             ctx.token_slot, ctx.positions, layer.block_table, n_heads,
                                             n_kv_heads, head_dim, layer.page_size, window, scale, softcap, sink)
        return tensorcore.attention(self, q, out, ctx, layer, n_heads, n_kv_heads, head_dim, window, scale,
                                    softcap=softcap, sink=sink)

    # ------------------------------------------------------------------ rotary positions + cache write
    def rotary_cache_write(self, q, k, v, inv_freq, rot_dims, interleaved, ctx, layer, n_heads, n_kv_heads,
                           head_dim, write_cache=True):
        """Turn the queries in place by position and send the step's keys (turned) and values into the pages
        in one launch.  ``q`` [T, n_heads * head_dim], ``k`` [T, n_kv_heads * head_dim] (row views);
        ``v`` None: the values are the keys as projected, before they are turned.  ``inv_freq``: float32
        [rot_dims / 2]; the first ``rot_dims`` dimensions of a head turn, as neighbours (2i, 2i + 1) when
        ``interleaved`` else as (i, i + rot_dims / 2)."""
        T = q.shape[0]
        _require(q, "q", self.dtype)
        _require(k, "k", self.dtype)
        if v is not None:
            _require(v, "v", self.dtype)
        if rot_dims:
            _require(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() != rot_dims // 2:
                raise KernelError("rotary: one frequency per pair of turning dimensions")
        if q.stride(1) != 1 or k.stride(1) != 1 or (v is not None and v.stride(1) != 1):
            raise KernelError("rotary: innermost stride must be 1")
        if q.shape[1] != n_heads * head_dim or k.shape[1] != n_kv_heads * head_dim:
            raise KernelError("rotary: widths do not match the head counts")
        pools = write_cache and layer is not None and layer.k_pool is not None
        if pools:
            _require(layer.k_pool, "k_pool", self.dtype)
        self.launches += 1
        _check(self.core.ps_rotary_cache_write(
            _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0) if v is not None else 0,
            _ptr(inv_freq) if rot_dims else None, rot_dims, 1 if interleaved else 0,
            _ptr(ctx.token_slot) if pools else None, _ptr(ctx.positions),
            _ptr(layer.block_table) if pools else None, layer.block_table.stride(0) if pools else 0,
            _ptr(layer.k_pool) if pools else None, _ptr(layer.v_pool) if pools else None,
            layer.page_stride if pools else 0, T, n_heads, n_kv_heads, head_dim,
            layer.page_size if pools else 1, self.code, _stream()), "rotary_cache_write")

    def head_norm_rotary_cache_write(self, q, k, v, q_gain, k_gain, eps, inv_freq, rot_dims, interleaved, dim, ctx,
                                     layer, n_heads, n_kv_heads, head_dim, write_cache=True, amplitude=1.0):
        """As :meth:`rotary_cache_write` for heads that are normed before they turn: per head, its first ``dim``
        numbers (of ``head_dim``; the rest is padding) are divided by their root mean square (eps inside the root)
        and multiplied by ``q_gain`` / ``k_gain`` (float32 [dim], one for all heads of a kind; None: no norm), then
        the first ``rot_dims`` turn.  Queries in place, keys into the key pages, the rows of ``v`` into the value
        pages.  ``k`` and ``v`` None: a layer that reads another layer's cache prepares its queries only.
        ``inv_freq``: float32 [rot_dims / 2, 2] as (high, low) parts (``RotaryPositions.inv_freq_split``);
        ``amplitude`` multiplies every sine and cosine (a rotation stretched to longer contexts has one above 1)."""
        T = q.shape[0]
        _require(q, "q", self.dtype)
        if (k is None) != (v is None):
            raise KernelError("head_norm_rotary: keys and values come together")
        for name, tensor in (("k", k), ("v", v)):
            if tensor is not None:
                _require(tensor, name, self.dtype)
                if tensor.stride(1) != 1 or tensor.shape[1] != n_kv_heads * head_dim:
                    raise KernelError("head_norm_rotary: keys and values must be rows of n_kv_heads * head_dim")
        for name, gain in (("q_gain", q_gain), ("k_gain", k_gain)):
            if gain is not None:
                _require(gain, name, torch.float32)
                if gain.numel() != dim or not gain.is_contiguous():
                    raise KernelError("head_norm_rotary: one gain per normed dimension")
        if rot_dims:
            _require(inv_freq, "inv_freq", torch.float32)
            if inv_freq.shape != (rot_dims // 2, 2) or not inv_freq.is_contiguous():
                raise KernelError("head_norm_rotary: one (high, low) frequency per pair of turning dimensions")
        if q.stride(1) != 1 or q.shape[1] != n_heads * head_dim:
            raise KernelError("head_norm_rotary: queries must be rows of n_heads * head_dim")
        pools = write_cache and k is not None and layer is not None and layer.k_pool is not None
        if pools:
            _require(layer.k_pool, "k_pool", self.dtype)
        self.launches += 1
        _check(self.core.ps_head_norm_rotary_cache_write(
            _ptr(q), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0, _ptr(v),
            v.stride(0) if v is not None else 0, _ptr(q_gain), _ptr(k_gain), float(eps),
            _ptr(inv_freq) if rot_dims else None, rot_dims, 1 if interleaved else 0,
            _ptr(ctx.token_slot) if pools else None, _ptr(ctx.positions),
            _ptr(layer.block_table) if pools else None, layer.block_table.stride(0) if pools else 0,
            _ptr(layer.k_pool) if pools else None, _ptr(layer.v_pool) if pools else None,
            layer.page_stride if pools else 0, T, n_heads, n_kv_heads, head_dim, dim,
            layer.page_size if pools else 1, self.code, float(amplitude), _stream()), "head_norm_rotary_cache_write")

    # ------------------------------------------------------------------ linear recurrence with decay ("wkv")
    def token_shift_mix(self, x, mu, state, prev_offset, ctx, out):
        """out[s, t] = x[t] + (x[t-1] - x[t]) * mu[s]: ``x`` [T, W] (compute dtype), ``mu`` float32 [S, W],
        ``out`` [S, T, W]; x[t-1] of an entry's first token is the request's stored last input
        (``state[slot, prev_offset:prev_offset + W]``, float32)."""
        T, W = x.shape
        _require(x, "x", self.dtype)
        _require(out, "out", self.dtype)
        _require(mu, "mu", torch.float32)
        _require(state, "state", torch.float32)
        if out.shape != (mu.shape[0], T, W) or not out.is_contiguous() or x.stride(1) != 1 or mu.shape[1] != W:
            raise KernelError("token_shift_mix: shapes do not match")
        self.launches += 1
        _check(self.core.ps_token_shift_mix(_ptr(x), x.stride(0), _ptr(mu), mu.shape[0], _ptr(state),
                                            state.stride(0), prev_offset, _ptr(ctx.token_item), _ptr(ctx.q_start),
                                            _ptr(ctx.item_slot), _ptr(out), out.stride(0), out.stride(1), T, W,
                                            self.code, _stream()), "token_shift_mix")
        return out

    def wkv_prepare(self, hidden, gain, eps, mu, state, prev_offset, ctx, w1, w2, w0, blends, decay):
        """From the float32 residual rows to the wkv mixer's inputs in one launch: the RMS norm (``gain``, ``eps``),
        the blends with the token before (``mu`` float32 [5, W]; ``blends`` [5, T, W]: blocks 0..3 the first four
        blends, block 4 the normed rows), and the decay's argument ``w2 @ tanh(w1 @ blend_4) + w0`` into
        ``decay`` (float32 [T, inner] rows)."""
        T, W = hidden.shape
        _require(hidden, "hidden", torch.float32)
        _require(gain, "gain", torch.float32)
        _require(mu, "mu", torch.float32)
        _require(state, "state", torch.float32)
        _require(w1, "w1", self.dtype)
        _require(w2, "w2", self.dtype)
        _require(w0, "w0", torch.float32)
        _require(blends, "blends", self.dtype)
        _require(decay, "decay", torch.float32)
        rank, inner = w1.shape[0], w2.shape[0]
        if (blends.shape != (5, T, W) or blends.stride(2) != 1 or mu.shape != (5, W) or not mu.is_contiguous()
                or w1.shape[1] != W or w2.shape[1] != rank or w1.stride(1) != 1 or w2.stride(1) != 1
                or decay.shape != (T, inner) or decay.stride(1) != 1 or hidden.stride(1) != 1 or w0.numel() != inner):
            raise KernelError("wkv_prepare: shapes do not match")
        self.launches += 1
        _check(self.core.ps_wkv_prepare(_ptr(hidden), hidden.stride(0), _ptr(gain), float(eps), _ptr(mu), _ptr(state),
                                        state.stride(0), prev_offset, _ptr(ctx.token_item), _ptr(ctx.q_start),
                                        _ptr(ctx.item_slot), _ptr(w1), w1.stride(0), rank, _ptr(w2), w2.stride(0),
                                        _ptr(w0), inner, _ptr(blends), blends.stride(0), blends.stride(1), _ptr(decay),
                                        decay.stride(0), T, W, self.code, _stream()), "wkv_prepare")

    def wkv_recurrence(self, r, k, v, decay, gate, u, gain, eps, x, state, prev_offset, ctx, out, heads, head_dim):
        """The recurrence of every entry of the step, tokens in order, from and into the slots' state (see
        csrc/wkv.cu).  ``r, k, v, decay, gate``: float32 [T, heads * head_dim] of equal row stride; ``u``,
        ``gain``: float32 [heads * head_dim]; ``x`` [T, W] the mixer's input, whose newest row per entry is
        kept in the slot; ``out`` [T, heads * head_dim] in the compute dtype."""
        inner = heads * head_dim
        for name, tensor in (("r", r), ("k", k), ("v", v), ("decay", decay), ("gate", gate)):
            _require(tensor, name, torch.float32)
            if tensor.shape[1] != inner or tensor.stride(1) != 1 or tensor.stride(0) != r.stride(0):
                raise KernelError("wkv: r, k, v, decay and gate must be rows of equal stride")
        _require(u, "u", torch.float32)
        _require(gain, "gain", torch.float32)
        _require(state, "state", torch.float32)
        _require(x, "x", self.dtype)
        _require(out, "out", self.dtype)
        if u.numel() != inner or gain.numel() != inner or state.shape[1] < prev_offset + x.shape[1]:
            raise KernelError("wkv: sizes do not match")
        if head_dim > 128:
            raise KernelError("wkv: head sizes above 128 are not supported")
        self.launches += 1
        _check(self.core.ps_wkv_recurrence(_ptr(r), _ptr(k), _ptr(v), _ptr(decay), _ptr(gate), r.stride(0), _ptr(u),
                                           _ptr(gain), float(eps), _ptr(x), x.stride(0), x.shape[1], _ptr(state),
                                           state.stride(0), prev_offset, _ptr(ctx.q_start), _ptr(ctx.item_slot),
                                           _ptr(out), out.stride(0), ctx.num_items, heads, head_dim, self.code,
                                           _stream()), "wkv_recurrence")
        return out

    # ------------------------------------------------------------------ embedding with a hashed pair table
    def embed_pair(self, ctx, table, scale, pair, buckets, mul_prev, mul_cur, newest, out):
        """out[t] = scale * table[id_t] + pair[row_t] as float32 [T, H]; row_t is the hash
        (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets, or ``buckets`` for a sequence's first token.  The token
        before an entry's first token is read from ``newest`` (int32, one per slot), which then receives the
        entry's last token.  ``pair`` None: no pair table."""
        T, H = out.shape
        _require(out, "out", torch.float32)
        _require(table, "table", self.dtype)
        if table.shape[1] != H or ctx.token_ids.numel() != T:
            raise KernelError("embed_pair: shapes do not match")
        if pair is not None:
            _require(pair, "pair", self.dtype)
            _require(newest, "newest", torch.int32)
            if pair.shape != (buckets + 1, H) or not pair.is_contiguous():
                raise KernelError("embed_pair: the pair table must hold buckets + 1 rows of the model's width")
        if not table.is_contiguous() or not out.is_contiguous():
            raise KernelError("embed_pair: tensors must be contiguous")
        self.launches += 1
        _check(self.core.ps_embed_pair(_ptr(ctx.token_ids), _ptr(ctx.positions), _ptr(ctx.token_item),
                                       _ptr(ctx.q_start), _ptr(ctx.item_slot), _ptr(table), float(scale), _ptr(pair),
                                       int(buckets), int(mul_prev) % max(int(buckets), 1),
                                       int(mul_cur) % max(int(buckets), 1), _ptr(newest), _ptr(out), T, H,
                                       table.shape[0], self.code, _ptr(ctx.status), _stream()), "embed_pair")
        return out

    # ------------------------------------------------------------------ several residual streams
    def hyper_begin(self, x0, w_in, streams, u, y):
        """streams[s] = x0 for every s; u = sum_s w_in[s] * x0; y = 0.  All float32; ``streams`` [S, T, W]."""
        S = streams.shape[0]
        for name, tensor in (("x0", x0), ("w_in", w_in), ("streams", streams), ("u", u), ("y", y)):
            _require(tensor, name, torch.float32)
        if (streams.shape[1:] != x0.shape or u.shape != x0.shape or y.shape != x0.shape or w_in.numel() != S
                or not (x0.is_contiguous() and streams.is_contiguous() and u.is_contiguous() and y.is_contiguous())):
            raise KernelError("hyper_begin: shapes do not match")
        self.launches += 1
        _check(self.core.ps_hyper_begin(_ptr(x0), _ptr(w_in), _ptr(streams), _ptr(u), _ptr(y), x0.numel(), S,
                                        _stream()), "hyper_begin")

    def hyper_step(self, streams, y, mix, w_out, w_in_next, u):
        """Finish a sublayer and open the next: x_t <- sum_s mix[s, t] x_s + w_out[t] y for every stream t, then
        u = sum_t w_in_next[t] x_t (``w_in_next`` None: ones) and y = 0.  All float32."""
        S = streams.shape[0]
        for name, tensor in (("streams", streams), ("y", y), ("mix", mix), ("w_out", w_out), ("u", u)):
            _require(tensor, name, torch.float32)
        if w_in_next is not None:
            _require(w_in_next, "w_in_next", torch.float32)
        if (streams.shape[1:] != y.shape or u.shape != y.shape or mix.shape != (S, S) or w_out.numel() != S
                or (w_in_next is not None and w_in_next.numel() != S) or not mix.is_contiguous()
                or not (streams.is_contiguous() and u.is_contiguous() and y.is_contiguous())):
            raise KernelError("hyper_step: shapes do not match")
        self.launches += 1
        _check(self.core.ps_hyper_step(_ptr(streams), _ptr(y), _ptr(mix), _ptr(w_out), _ptr(w_in_next), _ptr(u),
                                       y.numel(), S, _stream()), "hyper_step")

    # ------------------------------------------------------------------ latent attention
    def latent_prepare(self, q, down, gain, eps, inv_freq, rot_dims, ctx, layer, q_out, n_heads, flat, turning,
                       rank, write_cache=True):
        """Between the input projection and attention of a latent-attention layer (csrc/latent.cu): the latent
        (``down[:, :rank]``, unit RMS times ``gain``) and the turned shared key part (``down[:, rank:]``) go into
        the token's place of the layer's single cache plane; the turning part of every query head (the last
        ``turning`` of its ``flat + turning`` numbers in ``q``) is turned into the last ``turning`` of the head's
        ``rank + turning`` numbers in ``q_out``.  ``inv_freq``: float32 [rot_dims / 2, 2], each frequency as a
        float and the float nearest to the rest (``RotaryPositions.inv_freq_split``)."""
        T = q.shape[0]
        for name, tensor in (("q", q), ("down", down), ("q_out", q_out)):
            _require(tensor, name, self.dtype)
            if tensor.stride(1) != 1:
                raise KernelError("latent_prepare: innermost stride must be 1")
        _require(gain, "gain", torch.float32)
        if (q.shape[1] != n_heads * (flat + turning) or down.shape[1] != rank + turning
                or q_out.shape[1] != n_heads * (rank + turning) or gain.numel() != rank):
            raise KernelError("latent_prepare: widths do not match")
        if rot_dims:
            _require(inv_freq, "inv_freq", torch.float32)
            if inv_freq.shape != (rot_dims // 2, 2) or not inv_freq.is_contiguous():
                raise KernelError("latent_prepare: one (high, low) frequency per pair of turning dimensions")
        pools = write_cache and layer is not None and layer.k_pool is not None
        if pools:
            _require(layer.k_pool, "k_pool", self.dtype)
            if layer.k_pool.shape[-1] != rank + turning or layer.k_pool.shape[-3] != 1:
                raise KernelError("latent_prepare: the cache plane must hold one row of rank + turning per token")
        self.launches += 1
        _check(self.core.ps_latent_prepare(
            _ptr(q), q.stride(0), _ptr(down), down.stride(0), _ptr(gain), float(eps),
            _ptr(inv_freq) if rot_dims else None, rot_dims, _ptr(ctx.token_slot) if pools else None,
            _ptr(ctx.positions), _ptr(layer.block_table) if pools else None,
            layer.block_table.stride(0) if pools else 0, _ptr(layer.k_pool) if pools else None,
            layer.page_stride if pools else 0, layer.page_size if pools else 1, _ptr(q_out), q_out.stride(0), T,
            n_heads, flat, turning, rank, self.code, _stream()), "latent_prepare")

    def sigmoid_gate(self, heads, g, span=1):
        """heads[:, j] *= sigmoid(g[:, j // span]) in float32; ``heads`` [rows, width] and ``g`` [rows, width / span]
        are row views of the compute type (span 1: a gate per number; a head's size: one gate per head)."""
        _require(heads, "heads", self.dtype)
        _require(g, "g", self.dtype)
        if (heads.shape[0] != g.shape[0] or heads.shape[1] != g.shape[1] * span or heads.stride(1) != 1
                or g.stride(1) != 1):
            raise KernelError("sigmoid_gate: shapes do not match")
        self.launches += 1
        _check(self.core.ps_sigmoid_gate(_ptr(heads), heads.stride(0), _ptr(g), g.stride(0), heads.shape[0],
                                         heads.shape[1], int(span), self.code, _stream()), "sigmoid_gate")
        return heads

    # ------------------------------------------------------------------ norms in groups, sums behind a norm
    def group_rms_norm(self, x, gain, eps, groups, out, rows=None):
        """out[r] = x[rows[r]] (or x[r]) with each of its ``groups`` equal runs divided by the run's root mean square
        (eps inside the root), times ``gain`` (float32 [H]); csrc/post_norm.cu.  ``x`` rows of float32 or the compute
        type, ``out`` rows of either; a row may be normed in place."""
        _require(x, "x")
        _require(out, "out")
        _require(gain, "gain", torch.float32)
        H = x.shape[-1]
        n_rows = out.shape[0]
        if rows is not None:
            _require(rows, "rows", torch.int32)
            if rows.numel() != n_rows:
                raise KernelError("group_rms_norm: rows and out disagree")
        elif x.shape[0] != n_rows:
            raise KernelError("group_rms_norm: x and out disagree")
        if (out.shape[-1] != H or gain.numel() != H or x.stride(-1) != 1 or out.stride(-1) != 1 or groups <= 0
                or H % groups or not gain.is_contiguous()):
            raise KernelError("group_rms_norm: widths disagree")
        self.launches += 1
        _check(self.core.ps_group_rms_norm(_ptr(x), x.stride(0), dtype_code(x.dtype), _ptr(rows), n_rows, H, int(groups),
                                           _ptr(gain), float(eps), _ptr(out), out.stride(0), dtype_code(out.dtype),
                                           _stream()), "group_rms_norm")
        return out

    def post_norm_add(self, y, x, gain, eps, groups, x_cast=None, history=None, n_history=0, weight=None):
        """x += group_rms_norm(y) * gain, y = 0 (all float32 [T, H]); with ``history`` [n, T, H] the sum is stored as
        entry ``n_history - 1`` and x becomes sum_j weight[j] * history[j] over the first ``n_history`` entries;
        ``x_cast`` (compute type) receives a copy of the new x."""
        for name, tensor in (("y", y), ("x", x)):
            _require(tensor, name, torch.float32)
        _require(gain, "gain", torch.float32)
        T, H = x.shape
        if y.shape != x.shape or not (x.is_contiguous() and y.is_contiguous()) or gain.numel() != H or H % groups:
            raise KernelError("post_norm_add: shapes do not match")
        if x_cast is not None and (x_cast.shape != x.shape or not x_cast.is_contiguous()):
            raise KernelError("post_norm_add: the copy must have the rows' shape")
        stride = 0
        if history is not None:
            _require(history, "history", torch.float32)
            _require(weight, "weight", torch.float32)
            if (history.shape[1:] != x.shape or not history.is_contiguous() or not (0 < n_history <= history.shape[0])
                    or weight.numel() != n_history or not weight.is_contiguous()):
                raise KernelError("post_norm_add: the history does not fit")
            stride = history.stride(0)
        self.launches += 1
        _check(self.core.ps_post_norm_add(_ptr(y), _ptr(x), T, H, int(groups), _ptr(gain), float(eps), _ptr(x_cast),
                                          dtype_code(x_cast.dtype) if x_cast is not None else PS_F32, _ptr(history),
                                          stride, int(n_history), _ptr(weight), _stream()), "post_norm_add")

    def depth_begin(self, x, first, x_cast, y):
        """first = x (if given), x_cast = x in the compute type (if given), y = 0; float32 rows of one shape."""
        _require(x, "x", torch.float32)
        _require(y, "y", torch.float32)
        if y.shape != x.shape or not (x.is_contiguous() and y.is_contiguous()):
            raise KernelError("depth_begin: shapes do not match")
        for tensor in (first, x_cast):
            if tensor is not None and (tensor.shape != x.shape or not tensor.is_contiguous()):
                raise KernelError("depth_begin: shapes do not match")
        self.launches += 1
        _check(self.core.ps_depth_begin(_ptr(x), _ptr(first), _ptr(x_cast),
                                        dtype_code(x_cast.dtype) if x_cast is not None else PS_F32, _ptr(y), x.numel(),
                                        _stream()), "depth_begin")

    # ------------------------------------------------------------------ minGRU
    def mingru_scan(self, zug, width, state, ctx, out):
        """The gated recurrence of every entry of the step from and into the slots' state (csrc/mingru.cu).  ``zug``
        float32 [T, 3 * width]: the update gate's, the candidate's and the output gate's projections side by side;
        ``state`` float32 [slots, width]; ``out`` [T, width] in the compute type."""
        _require(zug, "zug", torch.float32)
        _require(state, "state", torch.float32)
        _require(out, "out", self.dtype)
        T = zug.shape[0]
        if (zug.shape[1] != 3 * width or out.shape != (T, width) or state.shape[1] != width or zug.stride(1) != 1
                or out.stride(1) != 1 or state.stride(1) != 1):
            raise KernelError("mingru_scan: shapes do not match")
        # long entries are cut into runs of tokens that are folded side by side (a rule of the step's shape)
        longest = max(1, int(ctx.max_q_len))
        segments = 1
        while segments < 64 and segments * 16 < longest:
            segments *= 2
        self.launches += 1
        _check(self.core.ps_mingru_scan(_ptr(zug), zug.stride(0), width, _ptr(state), state.stride(0), _ptr(ctx.q_start),
                                        _ptr(ctx.item_slot), ctx.num_items, _ptr(out), out.stride(0), segments,
                                        self.code, _stream()), "mingru_scan")
        return out

    # ------------------------------------------------------------------ short convolution over time
    def short_conv(self, u, weight, taps, conv_channels, state, ctx, out, blend=None):
        """out[t, c] = sum_j weight[c, j] * u[t - taps + 1 + j, c] for the first ``conv_channels`` channels, the rest
        passed through; what lies before an entry's first token comes from ``state`` (float32
        [slots, (taps - 1) * conv_channels]: a request's last projected rows), which is then brought up to date
        (csrc/short_conv.cu).  ``u`` float32 [T, channels], ``out`` the same shape in the compute type.
        ``blend`` = (mode, first channel, heads, head slot, head values, shared float32 [T, heads * head values],
        mix float32 scalar): mode "store" leaves the convolved values of those heads in ``shared``, "mix" blends
        them, v <- (1 - mix) v + mix * shared."""
        _require(u, "u", torch.float32)
        _require(out, "out", self.dtype)
        T, channels = u.shape
        if out.shape != u.shape or u.stride(1) != 1 or out.stride(1) != 1 or not (0 <= conv_channels <= channels):
            raise KernelError("short_conv: shapes do not match")
        if conv_channels:
            _require(weight, "weight", torch.float32)
            if weight.shape != (conv_channels, taps) or not weight.is_contiguous():
                raise KernelError("short_conv: one row of taps per convolved channel")
        if taps > 1 and conv_channels:
            _require(state, "state", torch.float32)
            if state.shape[1] != (taps - 1) * conv_channels or state.stride(1) != 1:
                raise KernelError("short_conv: the state holds taps - 1 rows of the convolved channels")
        else:
            state = None
        mode, lo, heads, slot, values, shared, mix = 0, 0, 0, 1, 1, None, None
        if blend is not None:
            kind, lo, heads, slot, values, shared, mix = blend
            mode = {"store": 1, "mix": 2}[kind]
            _require(shared, "shared", torch.float32)
            if shared.shape != (T, heads * values) or not shared.is_contiguous() or lo + heads * slot > conv_channels:
                raise KernelError("short_conv: the shared values do not fit")
            if mode == 2:
                _require(mix, "mix", torch.float32)
        self.launches += 1
        _check(self.core.ps_short_conv(_ptr(u), u.stride(0), _ptr(weight), taps, conv_channels, channels, _ptr(state),
                                       state.stride(0) if state is not None else 0, _ptr(ctx.token_item),
                                       _ptr(ctx.q_start), _ptr(ctx.item_slot), _ptr(out), out.stride(0), mode, lo, heads,
                                       slot, values, _ptr(shared), _ptr(mix) if mode == 2 else None, T, self.code,
                                       _stream()), "short_conv")
        if state is not None:
            self.launches += 1
            _check(self.core.ps_short_conv_keep(_ptr(u), u.stride(0), taps, conv_channels, _ptr(state), state.stride(0),
                                                _ptr(ctx.q_start), _ptr(ctx.item_slot), ctx.num_items, _stream()),
                   "short_conv_keep")
        return out

    # ------------------------------------------------------------------ routed experts
    def moe_route(self, x, router, shared_gate_w, dense, chosen, chosen_w, shared_gate, top, groups, keep, norm=None,
                  score="softmax", normalize=True, correction=None):
        """The router of a layer of experts (csrc/moe.cu): softmax of ``x @ router.T`` in float32, the ``top``
        largest among the experts of the ``keep`` best of ``groups`` groups (0 or 1 groups: all experts stand),
        weights normalised to sum 1.  ``dense`` float32 [T, E] gets the weights (0 where not chosen), ``chosen``
        int32 / ``chosen_w`` float32 [T, top] the election, ``shared_gate`` float32 [T] = sigmoid(x . shared_gate_w)
        where ``shared_gate_w`` [W] is given.  ``norm`` = (raw float32 [T, W], gain float32 [W], eps): the kernel
        first writes the RMS norm of ``raw`` into ``x`` (the rows the experts' products then read) instead of
        reading ``x``.  ``score`` "sigmoid": the scores are sigmoid(z) expert by expert instead of the softmax;
        ``normalize`` False: the weights are the chosen scores themselves.  ``correction`` float32 [E]: added to the
        scores for the election only (the weights stay the scores)."""
        if correction is not None:
            _require(correction, "correction", torch.float32)
            if correction.numel() != router.shape[0] or not correction.is_contiguous():
                raise KernelError("moe_route: one correction per expert")
        if score not in ("softmax", "sigmoid"):
            raise KernelError(f"moe_route: unknown score {score!r}")
        T, W = x.shape
        E = router.shape[0]
        _require(x, "x", self.dtype)
        _require(router, "router", self.dtype)
        _require(dense, "dense", torch.float32)
        _require(chosen, "chosen", torch.int32)
        _require(chosen_w, "chosen_w", torch.float32)
        if shared_gate_w is not None:
            _require(shared_gate_w, "shared_gate_w", self.dtype)
            _require(shared_gate, "shared_gate", torch.float32)
            if shared_gate_w.numel() != W or not shared_gate_w.is_contiguous() or shared_gate.numel() != T:
                raise KernelError("moe_route: the shared gate does not fit")
        if (router.shape[1] != W or x.stride(1) != 1 or router.stride(1) != 1 or dense.shape != (T, E)
                or chosen.shape != (T, top) or chosen_w.shape != (T, top)
                or not (dense.is_contiguous() and chosen.is_contiguous() and chosen_w.is_contiguous())):
            raise KernelError("moe_route: shapes do not match")
        raw = gain = None
        eps = 0.0
        if norm is not None:
            raw, gain, eps = norm
            _require(raw, "raw", torch.float32)
            _require(gain, "gain", torch.float32)
            if raw.shape != (T, W) or raw.stride(1) != 1 or gain.numel() != W or not gain.is_contiguous():
                raise KernelError("moe_route: the rows to norm do not fit")
        self.launches += 1
        _check(self.core.ps_moe_route(_ptr(x), x.stride(0), _ptr(router), router.stride(0), _ptr(shared_gate_w),
                                      _ptr(dense), _ptr(chosen), _ptr(chosen_w), _ptr(shared_gate), T, W, E, top,
                                      int(groups or 0), int(keep or 0), self.code, _ptr(raw),
                                      raw.stride(0) if raw is not None else 0, _ptr(gain), float(eps),
                                      1 if score == "sigmoid" else 0, 1 if normalize else 0, _ptr(correction),
                                      _stream()), "moe_route")

    @staticmethod
    def _gate_form(form):
        """(kind, limit, shared limit, alpha) of the inner activation: None / "silu" = silu(g) * u * weight;
        ("clamped_swish", limit, shared_limit, alpha): g' = min(weight * g, limit), u' = clamp(weight * u, +-limit),
        g' * sigmoid(alpha * g') * (u' + 1): the weight scales the expert's input."""
        if form is None or form == "silu":
            return 0, 0.0, 0.0, 0.0
        kind, limit, shared_limit, alpha = form
        if kind != "clamped_swish":
            raise KernelError(f"unknown gated form {kind!r}")
        return 1, float(limit), float(shared_limit if shared_limit is not None else limit), float(alpha)

    def moe_gate_mul(self, gate_up, dense, shared_gate, inner, n_experts, expert_ff, form=None):
        """inner[t, c] = silu(gate) * up * weight over the stacked product ``gate_up`` [T, 2 C], C = inner.shape[1]:
        expert e's block of 2 * expert_ff columns is its gates, then its ups, and the shared expert's block follows;
        the weight of inner's column c is ``dense[t, c // expert_ff]`` for the experts' columns and
        ``shared_gate[t]`` (None: 1) from column ``n_experts * expert_ff`` on (csrc/moe.cu).  ``n_experts`` 0: the
        product of a shared expert alone, or of a dense gated feed-forward.  ``form``: see :meth:`_gate_form`."""
        T, C = inner.shape
        _require(gate_up, "gate_up", self.dtype)
        _require(inner, "inner", self.dtype)
        if (gate_up.shape != (T, 2 * C) or gate_up.stride(1) != 1 or inner.stride(1) != 1
                or (n_experts and (dense.shape != (T, n_experts) or not dense.is_contiguous()))):
            raise KernelError("moe_gate_mul: shapes do not match")
        if n_experts:
            _require(dense, "dense", torch.float32)
        if shared_gate is not None:
            _require(shared_gate, "shared_gate", torch.float32)
        self.launches += 1
        _check(self.core.ps_moe_gate_mul(_ptr(gate_up), gate_up.stride(0), _ptr(dense) if n_experts else None,
                                         _ptr(shared_gate), _ptr(inner), inner.stride(0), T, C, n_experts, expert_ff,
                                         self.code, *self._gate_form(form), _stream()),
               "moe_gate_mul")
        return inner

    EXPERT_TILE = 128             # rows of a tile of the tcgen05 product: runs of rows of one expert start on these

    def expert_rows(self, tokens, top, experts):
        """Rows of the buffer in which (token, expert) pairs are sorted by expert, every expert's run padded to whole
        tiles: enough for any election."""
        tile = self.EXPERT_TILE
        return -(-(tokens * top + experts * (tile - 1)) // tile) * tile

    def moe_plan(self, chosen, chosen_w, experts, row_of, row_token, row_weight, tile_expert):
        """Sort the (token, chosen expert) pairs of ``chosen`` [T, top] by expert (csrc/moe.cu: moe_plan)."""
        T, top = chosen.shape
        rows_cap = row_token.numel()
        _require(chosen, "chosen", torch.int32)
        _require(chosen_w, "chosen_w", torch.float32)
        for name, tensor in (("row_of", row_of), ("row_token", row_token), ("tile_expert", tile_expert)):
            _require(tensor, name, torch.int32)
        _require(row_weight, "row_weight", torch.float32)
        if (row_of.numel() != T * top or row_weight.numel() != rows_cap
                or tile_expert.numel() != rows_cap // self.EXPERT_TILE or not chosen.is_contiguous()
                or not chosen_w.is_contiguous()):
            raise KernelError("moe_plan: shapes do not match")
        self.launches += 1
        _check(self.core.ps_moe_plan(_ptr(chosen), _ptr(chosen_w), T, top, experts, self.EXPERT_TILE, rows_cap,
                                     _ptr(row_of), _ptr(row_token), _ptr(row_weight), _ptr(tile_expert), _stream()),
               "moe_plan")

    def moe_gather(self, x, row_token, rows):
        """rows[r] = x[row_token[r]], zeros where row_token[r] < 0."""
        _require(x, "x", self.dtype)
        _require(rows, "rows", self.dtype)
        _require(row_token, "row_token", torch.int32)
        if rows.shape != (row_token.numel(), x.shape[1]) or x.stride(1) != 1 or rows.stride(1) != 1:
            raise KernelError("moe_gather: shapes do not match")
        self.launches += 1
        _check(self.core.ps_moe_gather(_ptr(x), x.stride(0), _ptr(row_token), _ptr(rows), rows.stride(0),
                                       rows.shape[0], x.shape[1], self.code, _stream()), "moe_gather")
        return rows

    def moe_gate_mul_rows(self, gate_up, row_weight, inner, form=None):
        """inner[r, j] = silu(gate_up[r, j]) * gate_up[r, F + j] * row_weight[r], or the other ``form`` of
        :meth:`_gate_form` (with the routed experts' limit)."""
        R, F = inner.shape
        _require(gate_up, "gate_up", self.dtype)
        _require(inner, "inner", self.dtype)
        _require(row_weight, "row_weight", torch.float32)
        if gate_up.shape != (R, 2 * F) or row_weight.numel() != R or gate_up.stride(1) != 1 or inner.stride(1) != 1:
            raise KernelError("moe_gate_mul_rows: shapes do not match")
        self.launches += 1
        kind, limit, _, alpha = self._gate_form(form)
        _check(self.core.ps_moe_gate_mul_rows(_ptr(gate_up), gate_up.stride(0), _ptr(row_weight), _ptr(inner),
                                              inner.stride(0), R, F, self.code, kind, limit, alpha, _stream()),
               "moe_gate_mul_rows")
        return inner

    def moe_combine(self, down, row_of, top, y):
        """y[t] += sum_k down[row_of[t * top + k]] (float32; k in rising order, rows < 0 skipped)."""
        T, W = y.shape
        _require(down, "down", torch.float32)
        _require(y, "y", torch.float32)
        _require(row_of, "row_of", torch.int32)
        if down.shape[1] != W or row_of.numel() != T * top or down.stride(1) != 1 or y.stride(1) != 1:
            raise KernelError("moe_combine: shapes do not match")
        self.launches += 1
        _check(self.core.ps_moe_combine(_ptr(down), down.stride(0), _ptr(row_of), top, _ptr(y), y.stride(0), T, W,
                                        _stream()), "moe_combine")
        return y

    def linear_experts(self, a, w, out, tile_expert, experts, along_k=False, act=None, status=None):
        """tcgen05 product of rows sorted by expert: tile t of ``a`` (EXPERT_TILE rows) times the matrix of expert
        ``tile_expert[t]``, skipped where that is negative.  ``w``: the experts' [N, K] matrices stacked by rows
        ([experts * N, K]) or, with ``along_k``, side by side ([N, experts * K])."""
        M, K = a.shape
        N = out.shape[1]
        want = (N, experts * K) if along_k else (experts * N, K)
        if tuple(w.shape) != want or out.shape[0] != M or tile_expert.numel() != -(-M // self.EXPERT_TILE):
            raise KernelError("linear_experts: shapes do not match")
        _require(a, "a", torch.bfloat16)
        _require(w, "w", torch.bfloat16)
        _require(out, "out")
        _require(tile_expert, "tile_expert", torch.int32)
        if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
            raise KernelError("linear_experts: innermost stride must be 1")
        if self._tc is None:
            self._tc = _declare(_load_library("tc"), "tc")
        if status is None:
            status = self.status_flag(a.device)
        self.launches += 1
        _check(self._tc.ps_gemm_tc_experts(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N,
                                           K, dtype_code(out.dtype), _ACT_CODE[act], _ptr(tile_expert), experts,
                                           1 if along_k else 0, _ptr(status), _stream()), "gemm_tc_experts")
        return out

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
