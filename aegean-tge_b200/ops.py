"""Bindings of the CUDA kernels: torch tensors in, raw pointers to the libraries.

Every function here launches hand-written sm_100a code from ``csrc/`` on the
current CUDA stream.  There is no CPU path and no library attention or model
code behind any of them: if the libraries cannot be built or loaded, the
first call raises.  Tensors are checked (device, dtype, contiguity) before a
pointer leaves Python.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Dict, Optional, Tuple

import torch

from .csrc import build as _build

GEMM_STORE, GEMM_STORE_F32, GEMM_ADD_F32, GEMM_SWIGLU, GEMM_GELU, GEMM_GELU_TANH, GEMM_GLU_CLAMPED = 0, 1, 2, 3, 4, 5, 6
STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a page id outside the pool",
               4: "a row index outside the batch", 8: "a bounded device-side wait gave up"}

_c_int, _c_ll, _c_float, _c_ptr = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or a launch failed."""


class DeviceStatusError(RuntimeError):
    """A kernel recorded a fault in the status word (bad token, bad page, ...)."""


# ----------------------------------------------------------------------------
# libraries
# ----------------------------------------------------------------------------
_core_lib: Optional[ctypes.CDLL] = None
_attn_libs: Dict[Tuple[int, int], ctypes.CDLL] = {}

# Set to False to send bfloat16 products through the CUDA-core kernel (for A/B checks).
USE_TCGEN05 = os.environ.get("TGE_NO_TCGEN05", "") == ""
# Set to False to send bfloat16 attention through the CUDA-core kernel.
USE_MMA_ATTENTION = os.environ.get("TGE_NO_MMA_ATTENTION", "") == ""


def _declare(lib: ctypes.CDLL, name: str, argtypes) -> None:
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = _c_int


def core() -> ctypes.CDLL:
    global _core_lib
    if _core_lib is None:
        path = _build.build_core()
        lib = ctypes.CDLL(path)
        lib.tge_last_error.restype = ctypes.c_char_p
        _declare(lib, "tge_embedding", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr])
        _declare(lib, "tge_rmsnorm", [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float,
                                      _c_ptr, _c_ptr])
        _declare(lib, "tge_add_to_stream", [_c_ptr, _c_ptr, _c_int, _c_ll, _c_float, _c_ptr])
        _declare(lib, "tge_rope_kv_store", [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                            _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_gemm_simt", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int, _c_int,
                                        _c_int, _c_int, _c_float, _c_int, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                                           _c_int, _c_int, _c_ptr, _c_ll, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                                           _c_int, _c_float, _c_float, _c_int, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_add_defer", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int,
                                                     _c_int, _c_int, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll,
                                                     _c_ptr, _c_float, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_defer_slices", [_c_int])
        _declare(lib, "tge_scale_rows", [_c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_float, _c_ptr, _c_ll, _c_int,
                                         _c_int, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_add_norm", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                                                    _c_int, _c_ptr, _c_float, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr,
                                                    _c_float, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_qkv_rope", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                                                    _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                                    _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                    _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr])
        _declare(lib, "tge_gemm_tcgen05_qkv_norm_act", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_int,
                                                        _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ll,
                                                        _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ll,
                                                        _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr])
        lib.tge_gemm_tcgen05_pair_mode.argtypes = [_c_int]
        lib.tge_gemm_tcgen05_pair_mode.restype = None
        lib.tge_gemm_tcgen05_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.tge_gemm_tcgen05_scratch_floats.restype = _c_ll
        _declare(lib, "tge_attention_simt", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr,
                                             _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                                             _c_float, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                             _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_attention_pooled_merge", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr,
                                                     _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_int,
                                                     _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_int, _c_ptr,
                                                     _c_ptr])
        _declare(lib, "tge_group_norm", [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                                         _c_ptr, _c_ptr, _c_ptr, _c_ptr])
        _declare(lib, "tge_token_shift", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                          _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_latent_prepare", [_c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_float,
                                             _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                             _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_head_linear", [_c_ptr, _c_ll, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_int, _c_ll, _c_int,
                                          _c_int, _c_int, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_rotate_interleaved", [_c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ptr, _c_int, _c_int,
                                                 _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_latent_gather", [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                                            _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_latent_scatter", [_c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr,
                                             _c_int, _c_ptr])
        _declare(lib, "tge_gate_rows", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_router_topk", [_c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr,
                                          _c_ptr])
        _declare(lib, "tge_activation", [_c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr])
        _declare(lib, "tge_experts_direct", [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_experts_dense_weigh", [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_int,
                                                  _c_int, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_experts_group", [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_ptr])
        _declare(lib, "tge_experts_combine_add", [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_int,
                                                  _c_int, _c_ptr])
        _declare(lib, "tge_to_run_dtype", [_c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr])
        _declare(lib, "tge_scale_add_norm", [_c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_float,
                                             _c_float, _c_ptr])
        _declare(lib, "tge_decay_scan", [_c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                         _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                         _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr])
        _declare(lib, "tge_gated_norm", [_c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int, _c_int,
                                         _c_float, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_conv_norm_rope_store", [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                                   _c_ptr, _c_float, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr,
                                                   _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ll, _c_int,
                                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_pool_kv", [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                      _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                                      _c_ptr])
        _declare(lib, "tge_qk_norm_kv_store", [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_float, _c_int, _c_ptr, _c_int,
                                               _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int,
                                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_soft_cap", [_c_ptr, _c_ll, _c_int, _c_int, _c_float, _c_ptr])
        _declare(lib, "tge_sample", [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_apply_penalty", [_c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_sample_cuts", [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                          _c_int, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_random_fill", [_c_ptr, _c_int, _c_ll, _c_ll, ctypes.c_ulonglong, _c_int, _c_float, _c_int,
                                          ctypes.c_uint, _c_ptr])
        _declare(lib, "tge_wait_gives_up", [_c_ptr, _c_ll, _c_ptr, _c_ptr])
        _declare(lib, "tge_gated_prepare", [_c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr,
                                            _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_float, _c_ptr,
                                            _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_gated_rule_scan", [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                                              _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr])
        _declare(lib, "tge_norm_scale_add", [_c_ptr, _c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_float, _c_float, _c_ptr])
        _declare(lib, "tge_qk_temp_store", [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_float, _c_float, _c_int, _c_ptr,
                                            _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_int, _c_ptr, _c_ptr])
        _declare(lib, "tge_gated_clamp_act", [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_float, _c_float,
                                              _c_float, _c_ptr])
        _declare(lib, "tge_concat_rows", [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr])
        lib.tge_device_sm_count.argtypes = []
        lib.tge_device_sm_count.restype = _c_int
        lib.tge_sample_cuts_padded.argtypes = [_c_int]
        lib.tge_sample_cuts_padded.restype = _c_ll
        _core_lib = lib
    return _core_lib


def attention_lib(head_dim: int, value_dim: int = 0) -> ctypes.CDLL:
    value_dim = value_dim or head_dim
    if (head_dim, value_dim) not in _attn_libs:
        path = _build.build_attention(head_dim, value_dim)
        lib = ctypes.CDLL(path)
        lib.tge_last_error.restype = ctypes.c_char_p
        _declare(lib, "tge_attention_mma", [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr,
                                            _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_int,
                                            _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr,
                                            _c_int, _c_int, _c_ptr, _c_int, _c_ptr])
        lib.tge_attention_mma_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.tge_attention_mma_scratch_floats.restype = _c_ll
        if lib.tge_attention_mma_head_dim() != head_dim or lib.tge_attention_mma_value_dim() != value_dim:
            raise KernelError(f"{path} was built for another head size")
        _attn_libs[(head_dim, value_dim)] = lib
    return _attn_libs[(head_dim, value_dim)]


def mma_attention_supports(head_dim: int, heads: int, kv_heads: int, page_size: int, value_dim: int = 0) -> bool:
    value_dim = value_dim or head_dim
    return (head_dim % 16 == 0 and 16 <= head_dim <= 256 and value_dim % 16 == 0 and 16 <= value_dim <= 256
            and heads % kv_heads == 0 and heads // kv_heads <= 64 and 64 % page_size == 0)


def loaded_libraries() -> Tuple[str, ...]:
    names = []
    if _core_lib is not None:
        names.append(_core_lib._name)
    names.extend(lib._name for lib in _attn_libs.values())
    return tuple(names)


UNSUPPORTED = -100
launches = 0          # kernels launched through this module since import (or since the caller reset it)


def _check(rc: int, lib: ctypes.CDLL) -> int:
    """Raises on an error code; otherwise counts and returns the number of kernels launched."""
    global launches
    if rc == UNSUPPORTED:
        return rc
    if rc < 0:
        raise KernelError(lib.tge_last_error().decode("utf-8", "replace"))
    launches += rc
    return rc


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (asked on every launch: a graph capture switches streams)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _want(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (this engine has no CPU path)")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _rows_2d(t: torch.Tensor, name: str) -> int:
    """Row stride (elements) of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with dense rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


_FLOAT = (torch.float32, torch.bfloat16)

# ----------------------------------------------------------------------------
# status word and scratch
# ----------------------------------------------------------------------------
_status: Dict[int, torch.Tensor] = {}
_scratch: Dict[int, torch.Tensor] = {}
_outgrown: Dict[int, list] = {}       # earlier scratch buffers, kept alive for the graphs that hold their address


def status_word(device: Optional[torch.device] = None) -> torch.Tensor:
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _status:
        _status[index] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{index}")
    return _status[index]


def check_status() -> None:
    """Reads the status word (synchronises) and raises if a kernel recorded a fault."""
    word = status_word()
    value = int(word.item())
    if value:
        word.zero_()
        what = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise DeviceStatusError("a kernel met " + " and ".join(what or [f"status {value}"]))


def wait_gives_up(limit_ns: int = 1_000_000) -> Tuple[bool, int]:
    """Launches one thread that waits, with the product kernels' bounded wait and a limit of ``limit_ns``
    (at most 10 ms), on a barrier nothing arrives at.  Returns (whether the wait claimed success, nanoseconds
    it took); the status word then carries the time-out bit until :func:`check_status` reads it."""
    lib = core()
    outcome = torch.zeros(2, dtype=torch.int64, device=f"cuda:{torch.cuda.current_device()}")
    _check(lib.tge_wait_gives_up(status_word().data_ptr(), int(limit_ns), outcome.data_ptr(), _stream()), lib)
    arrived, took = outcome.tolist()
    return bool(arrived), int(took)


def scratch_floats(count: int) -> torch.Tensor:
    """A float32 scratch buffer of at least ``count`` elements, reused between calls.

    The buffer grows when a call needs more (never while a CUDA graph is being captured).  A buffer that
    was outgrown is kept, not freed: a graph captured earlier has its address in its kernels and goes on
    writing partial sums there whenever it is replayed.  Buffers at least double, so what is kept is less
    than what is in use.
    """
    index = torch.cuda.current_device()
    have = _scratch.get(index)
    if have is None or have.numel() < count:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("scratch memory must be sized before a CUDA graph is captured "
                              f"(need {count} floats, have {0 if have is None else have.numel()})")
        size = max(count, 1 << 22, 0 if have is None else 2 * have.numel())
        if have is not None:
            _outgrown.setdefault(index, []).append(have)
        _scratch[index] = torch.empty(size, dtype=torch.float32, device=f"cuda:{index}")
    return _scratch[index]


# ----------------------------------------------------------------------------
# kernels
# ----------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = float32(table[ids[t], :]) * scale"""
    _want(table, "embedding table", _FLOAT)
    _want(ids, "token ids", torch.int32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    _want(out, "embedding output", torch.float32)
    lib = core()
    _check(lib.tge_embedding(table.data_ptr(), int(table.dtype == torch.bfloat16), ids.data_ptr(), out.data_ptr(),
                             tokens, hidden, vocab, float(scale), status_word().data_ptr(), _stream()), lib)
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows (optionally gathered by ``rows``) into ``out_dtype``."""
    _want(x, "norm input", torch.float32)
    _want(weight, "norm weight", torch.float32)
    src_rows, hidden = x.shape
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {hidden}")
    out_rows = src_rows if rows is None else rows.numel()
    if rows is not None:
        _want(rows, "norm row index", torch.int32)
    if out is None:
        out = torch.empty((out_rows, hidden), dtype=out_dtype, device=x.device)
    _want(out, "norm output", _FLOAT)
    lib = core()
    _check(lib.tge_rmsnorm(x.data_ptr(), weight.data_ptr(), _ptr(rows), out.data_ptr(),
                           int(out.dtype == torch.bfloat16), out_rows, src_rows, hidden, float(eps),
                           status_word().data_ptr(), _stream()), lib)
    return out


def add_to_stream(x: torch.Tensor, y: torch.Tensor, alpha: float = 1.0) -> None:
    """x (float32) += alpha * y (run dtype), same shape."""
    _want(x, "stream", torch.float32)
    _want(y, "addend", _FLOAT)
    if x.shape != y.shape:
        raise KernelError(f"add_to_stream: shapes differ, {tuple(x.shape)} and {tuple(y.shape)}")
    lib = core()
    _check(lib.tge_add_to_stream(x.data_ptr(), y.data_ptr(), int(y.dtype == torch.bfloat16), x.numel(), float(alpha),
                                 _stream()), lib)


def rope_kv_store(qkv: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary: int,
                  positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                  k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], heads: int, kv_heads: int,
                  head_dim: int) -> None:
    """Rotates q (in place) and k, and stores k and v into their pages.

    qkv: [T, >= (heads + 2*kv_heads) * head_dim].  cos/sin: float32 [positions, rotary/2]
    (None with rotary == 0: no rotation).  Pages: [num_pages, kv_heads, page_size, head_dim];
    None: nothing is stored (a layer that reads another layer's cache).
    """
    _want(qkv, "qkv", _FLOAT, contiguous=False)
    stride = _rows_2d(qkv, "qkv")
    tokens = qkv.shape[0]
    store = k_pages is not None
    if rotary > 0:
        _want(cos, "cos table", torch.float32)
        _want(sin, "sin table", torch.float32)
        if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != rotary // 2:
            raise KernelError(f"rotary tables must be [positions, {rotary // 2}], got {tuple(cos.shape)}")
    _want(positions, "positions", torch.int32)
    _want(seq_of_token, "seq_of_token", torch.int32)
    num_pages = page_size = max_pages = 0
    if store:
        _want(k_pages, "k pages", qkv.dtype)
        _want(v_pages, "v pages", qkv.dtype)
        _want(block_table, "block table", torch.int32)
        if k_pages.shape != v_pages.shape or k_pages.dim() != 4 or k_pages.shape[1] != kv_heads or k_pages.shape[3] != head_dim:
            raise KernelError(f"pages must be [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pages.shape)}")
        num_pages, _, page_size, _ = k_pages.shape
        max_pages = block_table.shape[1]
    lib = core()
    _check(lib.tge_rope_kv_store(qkv.data_ptr(), int(qkv.dtype == torch.bfloat16), stride, _ptr(cos), _ptr(sin),
                                 0 if cos is None else cos.shape[0], positions.data_ptr(), seq_of_token.data_ptr(),
                                 _ptr(block_table), max_pages, _ptr(k_pages), _ptr(v_pages), num_pages, page_size,
                                 tokens, heads, kv_heads if store else 0, head_dim, rotary, int(store),
                                 status_word().data_ptr(), _stream()), lib)


def qk_norm_kv_store(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                     per_head: bool, positions: torch.Tensor, seq_of_token: torch.Tensor,
                     block_table: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
                     v_pages: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int, value_dim: int,
                     v_other: Optional[torch.Tensor] = None, blend: Optional[torch.Tensor] = None) -> None:
    """RMS norm of the q and k projections (float32 statistics), an optional blend of the values with another
    layer's, and the store of k and v into their pages, all in place on the fused rows ``qkv`` [T, q | k | v].

    The norm runs over a token's whole projection (weights float32 [heads*head_dim] and [kv_heads*head_dim]) or,
    with ``per_head``, over each head (weights [head_dim]); a weight of None leaves that projection alone.
    ``v_other`` [T, kv_heads*value_dim] (dense rows, any row stride) and ``blend`` (a float32 scalar on the
    device): v <- (1 - blend) v + blend v_other before the store.  Pages None: nothing is stored.
    """
    _want(qkv, "qkv", _FLOAT, contiguous=False)
    stride = _rows_2d(qkv, "qkv")
    tokens = qkv.shape[0]
    for name, t, n in (("q norm weight", q_weight, heads), ("k norm weight", k_weight, kv_heads)):
        if t is not None:
            _want(t, name, torch.float32)
            if t.numel() != (head_dim if per_head else n * head_dim):
                raise KernelError(f"{name} has {t.numel()} elements")
    _want(positions, "positions", torch.int32)
    _want(seq_of_token, "seq_of_token", torch.int32)
    if (v_other is None) != (blend is None):
        raise KernelError("qk_norm_kv_store: a blend needs the other values and its weight")
    other_stride = 0
    if v_other is not None:
        _want(v_other, "other values", qkv.dtype, contiguous=False)
        _want(blend, "blend weight", torch.float32)
        other_stride = _rows_2d(v_other, "other values")
        if tuple(v_other.shape) != (tokens, kv_heads * value_dim) or blend.numel() != 1:
            raise KernelError(f"other values must be [{tokens}, {kv_heads * value_dim}], got {tuple(v_other.shape)}")
    store = k_pages is not None
    num_pages = page_size = max_pages = 0
    if store:
        _want(k_pages, "k pages", qkv.dtype)
        _want(v_pages, "v pages", qkv.dtype)
        _want(block_table, "block table", torch.int32)
        num_pages, _, page_size, _ = k_pages.shape
        if (tuple(k_pages.shape) != (num_pages, kv_heads, page_size, head_dim)
                or tuple(v_pages.shape) != (num_pages, kv_heads, page_size, value_dim)):
            raise KernelError(f"pages must be [pages, {kv_heads}, page_size, {head_dim} | {value_dim}], got "
                              f"{tuple(k_pages.shape)} and {tuple(v_pages.shape)}")
        max_pages = block_table.shape[1]
    lib = core()
    _check(lib.tge_qk_norm_kv_store(qkv.data_ptr(), int(qkv.dtype == torch.bfloat16), stride, _ptr(q_weight),
                                    _ptr(k_weight), float(eps), int(per_head), _ptr(v_other), other_stride, _ptr(blend),
                                    positions.data_ptr(), seq_of_token.data_ptr(), _ptr(block_table), max_pages,
                                    _ptr(k_pages), _ptr(v_pages), num_pages, page_size, tokens, heads, kv_heads,
                                    head_dim, value_dim, int(store), status_word().data_ptr(), _stream()), lib)


def linear_qkv_norm_act_store(x, w: torch.Tensor, heads: int, kv_heads: int, head_dim: int, value_dim: int,
                              q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                              positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                              k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                              v_other: Optional[torch.Tensor] = None, blend: Optional[torch.Tensor] = None,
                              act_out: Optional[torch.Tensor] = None, activation: int = GEMM_GELU) -> Optional[torch.Tensor]:
    """For a small bfloat16 batch, the q/k/v product of a layer that normalises q and k over their whole
    projections, with what follows it in one kernel: the product's partial sums are added, q and k normalised
    (float32), the values blended with ``v_other`` and k and v stored (as :func:`qk_norm_kv_store` does).  The
    weight may carry more rows below q, k and v, a feed-forward's up rows: their GELU goes to ``act_out``
    [T, up rows] (dense rows, any row stride).  Returns the qkv buffer [T, q | k | v], or None when the batch or
    the shape is not one for this path: the caller then runs the separate kernels."""
    deferred = x if isinstance(x, DeferredRows) else None
    if deferred is not None:
        x = deferred.rows
    M, K = x.shape
    N = w.shape[0]
    n_qkv = heads * head_dim + kv_heads * (head_dim + value_dim)
    if not (x.dtype == torch.bfloat16 and USE_TCGEN05 and M <= FUSED_MAX_TOKENS) or (N > n_qkv) != (act_out is not None):
        return None
    if deferred is not None and M > DEFER_MAX_TOKENS:
        return None
    _want(x, "linear input", torch.bfloat16, contiguous=False)
    _want(w, "linear weight", torch.bfloat16, contiguous=False)
    for name, t in (("positions", positions), ("seq_of_token", seq_of_token)):
        _want(t, name, torch.int32)
    for name, t, count in (("q norm weight", q_weight, heads * head_dim), ("k norm weight", k_weight, kv_heads * head_dim)):
        if t is not None:
            _want(t, name, torch.float32)
            if t.numel() != count:
                raise KernelError(f"{name} has {t.numel()} elements, the projection {count}")
    store = k_pages is not None
    num_pages = page_size = max_pages = 0
    if store:
        _want(k_pages, "k pages", torch.bfloat16)
        _want(v_pages, "v pages", torch.bfloat16)
        _want(block_table, "block table", torch.int32)
        num_pages, _, page_size, _ = k_pages.shape
        if (tuple(k_pages.shape) != (num_pages, kv_heads, page_size, head_dim)
                or tuple(v_pages.shape) != (num_pages, kv_heads, page_size, value_dim) or w.shape[1] != K):
            raise KernelError("linear_qkv_norm_act_store: shapes do not fit")
        max_pages = block_table.shape[1]
    other_stride = act_stride = 0
    if (v_other is None) != (blend is None):
        raise KernelError("linear_qkv_norm_act_store: a blend needs the other values and its weight")
    if v_other is not None:
        _want(v_other, "other values", torch.bfloat16, contiguous=False)
        _want(blend, "blend weight", torch.float32)
        other_stride = _rows_2d(v_other, "other values")
        if tuple(v_other.shape) != (M, kv_heads * value_dim):
            raise KernelError("linear_qkv_norm_act_store: the other values do not fit")
    if act_out is not None:
        _want(act_out, "activated rows", torch.bfloat16, contiguous=False)
        act_stride = _rows_2d(act_out, "activated rows")
        if tuple(act_out.shape) != (M, N - n_qkv):
            raise KernelError("linear_qkv_norm_act_store: the activated rows do not fit")
    lib = core()
    need = max(lib.tge_gemm_tcgen05_scratch_floats(M, N, K), M * N)
    scratch = scratch_floats(need)
    qkv = torch.empty((M, n_qkv), dtype=torch.bfloat16, device=x.device)
    rc = lib.tge_gemm_tcgen05_qkv_norm_act(x.data_ptr(), _rows_2d(x, "linear input"), w.data_ptr(), _rows_2d(w, "linear weight"),
                                           qkv.data_ptr(), n_qkv, _ptr(act_out), act_stride, int(activation), M, N, K,
                                           _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(v_other), other_stride,
                                           _ptr(blend), positions.data_ptr(), seq_of_token.data_ptr(), _ptr(block_table),
                                           max_pages, _ptr(k_pages), _ptr(v_pages), num_pages, page_size, heads, kv_heads,
                                           head_dim, value_dim, int(store), scratch.data_ptr(), scratch.numel(),
                                           status_word().data_ptr(),
                                           *(_NO_FACTOR if deferred is None else deferred.factor_args()), _stream())
    return None if _check(rc, lib) == UNSUPPORTED else qkv


def soft_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    """z (float32 [R, V], dense rows) <- cap * tanh(z / cap), in place."""
    _want(z, "scores", torch.float32, contiguous=False)
    ld = _rows_2d(z, "scores")
    lib = core()
    _check(lib.tge_soft_cap(z.data_ptr(), ld, z.shape[0], z.shape[1], float(cap), _stream()), lib)
    return z


DEFER_MAX_TOKENS = 128      # rows that may travel without their norm factor (the small-batch products)


class DeferredRows:
    """Rows ``stream * norm_weight`` in bfloat16 that still lack their RMSNorm factor.

    ``sums`` (float32 [slices, M]) holds each row's sum of squares in slices; the factor of row m is
    ``1 / sqrt(sum over slices / width + eps)``.  The product that takes these rows multiplies its result
    by it (``linear`` and ``linear_qkv_rope_store`` do); ``complete()`` gives the normalised rows.
    """

    def __init__(self, rows: torch.Tensor, sums: torch.Tensor, width: int, eps: float):
        self.rows, self.sums, self.width, self.eps = rows, sums, int(width), float(eps)

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    @property
    def device(self):
        return self.rows.device

    def factor_args(self):
        return self.sums.data_ptr(), self.sums.shape[0], self.width, self.eps

    def complete(self) -> torch.Tensor:
        lib = core()
        M, N = self.rows.shape
        out = torch.empty_like(self.rows)
        _check(lib.tge_scale_rows(self.rows.data_ptr(), _rows_2d(self.rows, "rows"), self.sums.data_ptr(),
                                  self.sums.shape[0], self.width, self.eps, out.data_ptr(), N, M, N, _stream()), lib)
        return out


_NO_FACTOR = (None, 0, 0, 0.0)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int,
           out: Optional[torch.Tensor] = None, force_simt: bool = False, force_bn: int = 0,
           force_splits: int = 0, alpha: float = 1.0, act_from: int = 0) -> torch.Tensor:
    """out = x . w^T with an epilogue.

    x [M, K] and w [N, K] in the run dtype; bias float32 [N] or None.
    GEMM_STORE: out [M, N] run dtype.  GEMM_STORE_F32: out [M, N] float32.
    GEMM_ADD_F32: ``out`` (float32 [M, N], required) += product.
    GEMM_SWIGLU: w rows interleaved (gate_i, up_i); out [M, N/2] run dtype.
    GEMM_GLU_CLAMPED: the same rows, both halves clamped at L = ``alpha``: out = min(g, L) sigmoid(1.702 min(g, L))
    (clamp(u, -L, L) + 1).
    GEMM_GELU / GEMM_GELU_TANH: out [M, N] run dtype = gelu(product + bias) in the erf / the tanh form for the
    columns from ``act_from`` on, the plain product below (for row-concatenated weights).
    ``alpha`` multiplies product + bias in the store and add epilogues (a residual multiplier, a logit scale).
    bfloat16 goes to the tcgen05 kernel when the shape allows TMA, else (and all of
    float32) to the CUDA-core kernel.
    """
    deferred = x if isinstance(x, DeferredRows) else None
    if deferred is not None:
        x = deferred.rows
    _want(x, "linear input", _FLOAT, contiguous=False)
    _want(w, "linear weight", x.dtype, contiguous=False)
    ldx, ldw = _rows_2d(x, "linear input"), _rows_2d(w, "linear weight")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"linear: input has {K} columns, weight has {w.shape[1]}")
    if bias is not None:
        _want(bias, "linear bias", torch.float32)
        if bias.numel() != N:
            raise KernelError(f"linear: bias has {bias.numel()} elements for {N} rows")
    if epilogue == GEMM_ADD_F32:
        if out is None:
            raise KernelError("linear: the residual epilogue needs the stream as `out`")
        want_shape, want_dtype = (M, N), torch.float32
    elif epilogue == GEMM_STORE_F32:
        want_shape, want_dtype = (M, N), torch.float32
    elif epilogue in (GEMM_SWIGLU, GEMM_GLU_CLAMPED):
        want_shape, want_dtype = (M, N // 2), x.dtype
    elif epilogue in (GEMM_STORE, GEMM_GELU, GEMM_GELU_TANH):
        want_shape, want_dtype = (M, N), x.dtype
    else:
        raise KernelError(f"linear: unknown epilogue {epilogue}")
    if out is None:
        out = torch.empty(want_shape, dtype=want_dtype, device=x.device)
    _want(out, "linear output", want_dtype, contiguous=False)
    if tuple(out.shape) != want_shape:
        raise KernelError(f"linear: output must be {want_shape}, got {tuple(out.shape)}")
    ldo = _rows_2d(out, "linear output")
    lib = core()
    if x.dtype == torch.bfloat16 and USE_TCGEN05 and not force_simt and (deferred is None or M <= DEFER_MAX_TOKENS):
        need = lib.tge_gemm_tcgen05_scratch_floats(M, N, K) if force_splits == 0 else force_splits * M * N
        scratch = scratch_floats(need) if need > 0 else None
        factor = _NO_FACTOR if deferred is None else deferred.factor_args()
        rc = lib.tge_gemm_tcgen05(x.data_ptr(), ldx, w.data_ptr(), ldw, _ptr(bias), out.data_ptr(), ldo, M, N, K,
                                  epilogue, _ptr(scratch), 0 if scratch is None else scratch.numel(), force_bn,
                                  force_splits, status_word().data_ptr(), *factor, float(alpha), int(act_from), _stream())
        if _check(rc, lib) != UNSUPPORTED:
            return out
    if deferred is not None:
        x = deferred.complete()
        ldx = _rows_2d(x, "linear input")
    _check(lib.tge_gemm_simt(x.data_ptr(), ldx, w.data_ptr(), ldw, _ptr(bias), out.data_ptr(), ldo, M, N, K,
                             int(x.dtype == torch.bfloat16), epilogue, float(alpha), int(act_from), _stream()), lib)
    return out


def set_pair_gemm(mode: int) -> None:
    """Whether the bfloat16 product may pair two SMs on one tile: 0 never, 1 where it is expected to be
    faster (the default), 2 wherever the kernel can run (tests)."""
    core().tge_gemm_tcgen05_pair_mode(int(mode))


# Small batches: the product leaves partial sums and one kernel per token row adds them, normalises or rotates and
# stores; larger ones use the product's own epilogue and separate kernels.  Prompts of 144 / 160 / 256 tokens at the
# 7B shape took 4.40 / 4.66 / 5.32 ms the first way and 4.54 / 4.56 / 5.04 ms the second (14B: 8.4 / 9.1 / 11.0 and
# 8.6 / 9.0 / 10.9), so the change is made between 144 and 160.  (The kernels themselves take up to 256 rows.)
FUSED_MAX_TOKENS = 144


def linear_add_norm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], stream: torch.Tensor,
                    norm_weight: torch.Tensor, eps: float, out_dtype: torch.dtype, defer: bool = False,
                    alpha: float = 1.0):
    """stream (float32 [M, N]) += alpha * (x . w^T (+ bias)); returns RMSNorm(stream) * norm_weight in ``out_dtype``.

    For a small bfloat16 batch the partial sums of the product are added into the stream and the new
    rows normalised by one kernel; otherwise the product and the norm run as separate kernels.
    With ``defer`` (the caller knows that ``linear`` or ``linear_qkv_rope_store`` takes the result) up to 128
    rows may come back as :class:`DeferredRows`: without the norm's factor, which their taker applies.
    """
    M, K = x.shape
    N = w.shape[0]
    if x.dtype == torch.bfloat16 and USE_TCGEN05 and M <= FUSED_MAX_TOKENS and out_dtype == torch.bfloat16:
        _want(x, "linear input", torch.bfloat16, contiguous=False)
        _want(w, "linear weight", torch.bfloat16, contiguous=False)
        _want(stream, "stream", torch.float32, contiguous=False)
        _want(norm_weight, "norm weight", torch.float32)
        if bias is not None:
            _want(bias, "linear bias", torch.float32)
        if tuple(stream.shape) != (M, N) or w.shape[1] != K or norm_weight.numel() != N:
            raise KernelError("linear_add_norm: shapes do not fit")
        lib = core()
        need = max(lib.tge_gemm_tcgen05_scratch_floats(M, N, K), M * N)
        scratch = scratch_floats(need)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        if defer and M <= DEFER_MAX_TOKENS and N % 8 == 0:
            # the taker of these rows applies the norm's factor: no block waits for a whole row here
            sums = torch.empty((lib.tge_gemm_tcgen05_defer_slices(N), M), dtype=torch.float32, device=x.device)
            rc = lib.tge_gemm_tcgen05_add_defer(x.data_ptr(), _rows_2d(x, "linear input"), w.data_ptr(),
                                                _rows_2d(w, "linear weight"), _ptr(bias), stream.data_ptr(),
                                                _rows_2d(stream, "stream"), M, N, K, norm_weight.data_ptr(),
                                                out.data_ptr(), N, sums.data_ptr(), scratch.data_ptr(),
                                                scratch.numel(), status_word().data_ptr(), float(alpha), _stream())
            if _check(rc, lib) != UNSUPPORTED:
                return DeferredRows(out, sums, N, eps)
        rc = lib.tge_gemm_tcgen05_add_norm(x.data_ptr(), _rows_2d(x, "linear input"), w.data_ptr(),
                                           _rows_2d(w, "linear weight"), _ptr(bias), stream.data_ptr(),
                                           _rows_2d(stream, "stream"), M, N, K, norm_weight.data_ptr(), float(eps),
                                           out.data_ptr(), N, scratch.data_ptr(), scratch.numel(),
                                           status_word().data_ptr(), float(alpha), _stream())
        if _check(rc, lib) != UNSUPPORTED:
            return out
    linear(x, w, bias, GEMM_ADD_F32, out=stream, alpha=alpha)
    return rmsnorm(stream, norm_weight, eps, out_dtype)


def linear_qkv_rope_store(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                          sin: Optional[torch.Tensor], rotary: int, positions: torch.Tensor,
                          seq_of_token: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                          v_pages: torch.Tensor, heads: int, kv_heads: int, head_dim: int) -> torch.Tensor:
    """The fused q/k/v product of an attention layer followed by rotation and the cache store.

    Returns the qkv buffer [T, (heads + 2 kv_heads) * head_dim] whose first heads*head_dim columns hold the
    rotated queries.  For a small bfloat16 batch one kernel per token row adds the product's partial sums,
    rotates and stores; otherwise the product and the rotate-and-store kernel run one after the other
    (then the k and v columns of the buffer are filled as well).
    """
    deferred = x if isinstance(x, DeferredRows) else None
    if deferred is not None:
        x = deferred.rows
    M, K = x.shape
    N = w.shape[0]
    if (x.dtype == torch.bfloat16 and USE_TCGEN05 and M <= FUSED_MAX_TOKENS):
        _want(x, "linear input", torch.bfloat16, contiguous=False)
        _want(w, "linear weight", torch.bfloat16, contiguous=False)
        for name, t in (("positions", positions), ("seq_of_token", seq_of_token), ("block table", block_table)):
            _want(t, name, torch.int32)
        _want(k_pages, "k pages", torch.bfloat16)
        _want(v_pages, "v pages", torch.bfloat16)
        if rotary > 0:
            _want(cos, "cos table", torch.float32)
            _want(sin, "sin table", torch.float32)
        if bias is not None:
            _want(bias, "linear bias", torch.float32)
        num_pages, page_kv, page_size, page_hd = k_pages.shape
        if page_kv != kv_heads or page_hd != head_dim or v_pages.shape != k_pages.shape or w.shape[1] != K:
            raise KernelError("linear_qkv_rope_store: shapes do not fit")
        lib = core()
        need = max(lib.tge_gemm_tcgen05_scratch_floats(M, N, K), M * N)
        scratch = scratch_floats(need)
        qkv = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        rc = lib.tge_gemm_tcgen05_qkv_rope(x.data_ptr(), _rows_2d(x, "linear input"), w.data_ptr(),
                                           _rows_2d(w, "linear weight"), _ptr(bias), qkv.data_ptr(), N, M, N, K,
                                           _ptr(cos), _ptr(sin), 0 if cos is None else cos.shape[0], rotary,
                                           positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                           block_table.shape[1], k_pages.data_ptr(), v_pages.data_ptr(), num_pages,
                                           page_size, heads, kv_heads, head_dim, scratch.data_ptr(), scratch.numel(),
                                           status_word().data_ptr(),
                                           *(_NO_FACTOR if deferred is None else deferred.factor_args()), _stream())
        if _check(rc, lib) != UNSUPPORTED:
            return qkv
    qkv = linear(x if deferred is None else deferred, w, bias, GEMM_STORE)
    rope_kv_store(qkv, cos, sin, rotary, positions, seq_of_token, block_table, k_pages, v_pages, heads, kv_heads,
                  head_dim)
    return qkv


def attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
              q_start: torch.Tensor, start_pos: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
              num_seqs: int, max_q_len: int, max_ctx_len: int, heads: int, kv_heads: int, head_dim: int,
              scale: float, window: int = 0, split_tokens: int = 0, out: Optional[torch.Tensor] = None,
              force_simt: bool = False, typical_ctx_len: int = 0, decode_prefix: int = 0,
              sink: Optional[torch.Tensor] = None, pool: int = 0, pooled_k: Optional[torch.Tensor] = None,
              pooled_v: Optional[torch.Tensor] = None, pool_table: Optional[torch.Tensor] = None,
              values_in_keys: int = 0, dist_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Paged causal attention of a flat batch of portions.

    q: [T, >= heads*head_dim] (dense rows, any row stride) holding rotated queries;
    pages [num_pages, kv_heads, page_size, head_dim] already hold the keys and values of
    every position up to each portion's last token.  Returns [T, heads*value_dim].  The values may have
    a size of their own: v pages [num_pages, kv_heads, page_size, value_dim].  ``sink`` (float32 [heads]):
    a learned score per head that joins the softmax's denominator once, unscaled, with no key or value.
    ``split_tokens`` > 0 cuts the keys into runs of that many positions (a multiple of 64)
    that are attended in parallel and merged; 0 picks a value from the batch shape.
    ``decode_prefix``: how many sequences at the head of the batch are known to bring one token each
    while others bring more (0: unknown); the tensor-core path then serves them with its decode kernel.
    ``pool`` > 0 (with a window): beside the last ``window`` tokens a query sees one pooled key and value for
    every block of ``pool`` positions that lies wholly before them, in the same softmax; ``pooled_k`` /
    ``pooled_v`` are pages shaped like the keys' and values', entry b of a request where position b would be, found
    through ``pool_table``.  Served by the CUDA-core kernel.
    ``values_in_keys`` > 0: a position's value is the first that many numbers of its key entry (a latent cache whose
    entries serve as keys whole and as values in part); ``v_pages`` is then not used and may be None.
    ``dist_bias`` (float32 [heads, span]): a learned bias by distance, added unscaled to the scaled score of the key
    that lies n positions back, entry min(n, span - 1) of the head's row; every attention kernel adds it where it
    scales its scores.
    """
    v_pitch = 0
    if values_in_keys:
        if not 0 < values_in_keys <= head_dim or pool:
            raise KernelError(f"attention: values of {values_in_keys} inside keys of {head_dim} (and no pooled blocks)")
        v_pages, v_pitch = k_pages[..., :values_in_keys], head_dim
    _want(q, "queries", _FLOAT, contiguous=False)
    q_stride = _rows_2d(q, "queries")
    tokens = q.shape[0]
    _want(k_pages, "k pages", q.dtype)
    _want(v_pages, "v pages", q.dtype, contiguous=not values_in_keys)
    for name, t in (("block table", block_table), ("q_start", q_start), ("start_pos", start_pos),
                    ("positions", positions), ("seq_of_token", seq_of_token)):
        _want(t, name, torch.int32)
    num_pages, page_kv, page_size, page_hd = k_pages.shape
    if (page_kv != kv_heads or page_hd != head_dim or v_pages.dim() != 4
            or tuple(v_pages.shape[:3]) != tuple(k_pages.shape[:3])):
        raise KernelError(f"pages must be [pages, {kv_heads}, page_size, {head_dim}] and the like for the values, "
                          f"got {tuple(k_pages.shape)} and {tuple(v_pages.shape)}")
    value_dim = v_pages.shape[3]
    if sink is not None:
        _want(sink, "attention sinks", torch.float32)
        if sink.numel() != heads:
            raise KernelError(f"attention: {sink.numel()} sinks for {heads} heads")
    max_pages = block_table.shape[1]
    if out is None:
        out = torch.empty((tokens, heads * value_dim), dtype=q.dtype, device=q.device)
    _want(out, "attention output", q.dtype, contiguous=False)
    out_stride = _rows_2d(out, "attention output")
    # the tensor-core kernels read and write pairs of bfloat16: rows that start on odd elements (an inner buffer
    # whose neighbour has an odd width, say) go to the CUDA-core kernel
    pairs_ok = (q_stride % 2 == 0 and out_stride % 2 == 0 and q.data_ptr() % 4 == 0 and out.data_ptr() % 4 == 0)
    pool_pages = pool_width = 0
    if pool:
        if window <= 0 or pooled_k is None or pooled_v is None or pool_table is None:
            raise KernelError("attention: pooled blocks need a window, their pages and their table")
        _want(pooled_k, "pooled k pages", q.dtype)
        _want(pooled_v, "pooled v pages", q.dtype)
        _want(pool_table, "pooled block table", torch.int32)
        if (tuple(pooled_k.shape[1:]) != (kv_heads, page_size, head_dim)
                or tuple(pooled_v.shape[1:]) != (kv_heads, page_size, value_dim) or pooled_k.shape[0] != pooled_v.shape[0]):
            raise KernelError(f"pooled pages must be shaped like the keys' and values', got {tuple(pooled_k.shape)} "
                              f"and {tuple(pooled_v.shape)}")
        pool_pages, pool_width = pooled_k.shape[0], pool_table.shape[1]
    dist_span = 0
    if dist_bias is not None:
        _want(dist_bias, "bias by distance", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[0] != heads or pool:
            raise KernelError(f"attention: a bias by distance is [heads, span] (and goes without pooled blocks), got "
                              f"{tuple(dist_bias.shape)}")
        dist_span = dist_bias.shape[1]
    use_mma = (q.dtype == torch.bfloat16 and USE_MMA_ATTENTION and not force_simt and pairs_ok
               and mma_attention_supports(head_dim, heads, kv_heads, page_size, value_dim)
               and not (v_pitch and value_dim == head_dim))
    if use_mma:
        lib = attention_lib(head_dim, value_dim)
        prefix = decode_prefix if decode_prefix >= MIN_DECODE_PREFIX and max_q_len > 1 and not pool else 0
        prefix_split = split_tokens
        if pool:
            # The window's tokens go through the tensor-core kernels with their keys cut into at least two runs, so
            # that they leave unnormalised states in the scratch memory; one more kernel walks the few pooled entries
            # a query sees, merges the runs' states into that and writes the row.
            if split_tokens == 0:
                split_tokens = choose_attention_split(tokens, num_seqs, max_q_len, typical_ctx_len or max_ctx_len, heads,
                                                      kv_heads, bound=max_ctx_len)
            if split_tokens == 0 or split_tokens >= max_ctx_len:
                # one run would be normalised at once: cut in two (a bound of two tiles at least; a run beyond a
                # request's keys holds nothing and is never read)
                max_ctx_len = max(max_ctx_len, 128)
                split_tokens = 64 * -(-max_ctx_len // 128)
        if split_tokens == 0:
            split_tokens = choose_attention_split(tokens, num_seqs, max_q_len, typical_ctx_len or max_ctx_len,
                                                  heads, kv_heads, bound=max_ctx_len)
            # the single tokens at the head of a mixed step are a decode batch of their own: a few of them deep in
            # long contexts want their keys cut although the portions beside them do not
            prefix_split = choose_attention_split(prefix, prefix, 1, max_ctx_len, heads, kv_heads,
                                                  bound=max_ctx_len) if prefix else 0
        count = lambda split: 1 if split == 0 or max_ctx_len <= split else -(-max_ctx_len // split)
        splits = max(count(split_tokens), count(prefix_split) if prefix else 1)
        need = lib.tge_attention_mma_scratch_floats(tokens, heads, splits)
        scratch = scratch_floats(need) if need > 0 else None
        _check(lib.tge_attention_mma(q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(),
                                     block_table.data_ptr(), max_pages, num_pages, page_size, q_start.data_ptr(),
                                     start_pos.data_ptr(), positions.data_ptr(), num_seqs, tokens, max_q_len,
                                     max_ctx_len, out.data_ptr(), out_stride, heads, kv_heads, float(scale), window,
                                     split_tokens, _ptr(scratch), status_word().data_ptr(), prefix, prefix_split,
                                     _ptr(sink), int(bool(pool)), v_pitch, _ptr(dist_bias), dist_span, _stream()), lib)
        if pool:
            core_lib = core()
            states = scratch.data_ptr()
            _check(core_lib.tge_attention_pooled_merge(q.data_ptr(), q_stride, pooled_k.data_ptr(), pooled_v.data_ptr(),
                                                       pool_table.data_ptr(), pool_width, pool_pages, page_size,
                                                       positions.data_ptr(), seq_of_token.data_ptr(), states,
                                                       states + 4 * splits * tokens * heads * value_dim, splits, split_tokens,
                                                       out.data_ptr(), out_stride, tokens, heads, kv_heads, head_dim,
                                                       value_dim, float(scale), window, int(pool), _ptr(sink), 1,
                                                       status_word().data_ptr(), _stream()), core_lib)
        return out
    lib = core()
    _check(lib.tge_attention_simt(q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(),
                                  block_table.data_ptr(), max_pages, num_pages, page_size, positions.data_ptr(),
                                  seq_of_token.data_ptr(), out.data_ptr(), out_stride, tokens, heads, kv_heads,
                                  head_dim, value_dim, _ptr(sink), float(scale), window, int(q.dtype == torch.bfloat16),
                                  int(pool), _ptr(pooled_k), _ptr(pooled_v), _ptr(pool_table), pool_width, pool_pages,
                                  v_pitch, _ptr(dist_bias), dist_span, status_word().data_ptr(), _stream()), lib)
    return out


def to_run_dtype(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 rows ``x`` in the format the products read (``x`` itself when that is float32)."""
    _want(x, "rows", torch.float32)
    if dtype == torch.float32:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    lib = core()
    _check(lib.tge_to_run_dtype(x.data_ptr(), out.data_ptr(), 1, x.numel(), _stream()), lib)
    return out


def scale_add_norm(x: torch.Tensor, y: torch.Tensor, alpha: float, weight: torch.Tensor, eps: float,
                   dtype: torch.dtype) -> torch.Tensor:
    """The stream of a layer that normalises after the sum: x <- rms(alpha x + y) * weight, in place on the float32
    rows ``x`` (``y`` float32, dense rows).  Returns the new rows in ``dtype`` for the next product (``x`` itself
    when that is float32)."""
    _want(x, "stream", torch.float32)
    _want(y, "addend", torch.float32, contiguous=False)
    _want(weight, "norm weight", torch.float32)
    rows, hidden = x.shape
    if tuple(y.shape) != (rows, hidden) or weight.numel() != hidden:
        raise KernelError(f"scale_add_norm: stream {tuple(x.shape)}, addend {tuple(y.shape)}, weight {weight.numel()}")
    copy = None if dtype == torch.float32 else torch.empty((rows, hidden), dtype=dtype, device=x.device)
    lib = core()
    _check(lib.tge_scale_add_norm(x.data_ptr(), y.data_ptr(), _rows_2d(y, "addend"), weight.data_ptr(), _ptr(copy),
                                  int(copy is not None), rows, hidden, float(alpha), float(eps), _stream()), lib)
    return x if copy is None else copy


def decay_scan(rows: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, dim: int, vdim: int,
               decay: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, q_start: torch.Tensor,
               positions: torch.Tensor, num_seqs: int, activation: bool = False, cos: Optional[torch.Tensor] = None,
               sin: Optional[torch.Tensor] = None, rotary: int = 0, k_scale: float = 1.0,
               max_q_len: int = 0) -> torch.Tensor:
    """Linear attention with a fixed decay per head over a flat batch of portions, its state carried per request.

    ``rows`` [T, ...] (run dtype, dense rows) holds the projections: q at column ``q_off`` and k at ``k_off``
    (heads x dim each), v at ``v_off`` (heads x vdim).  q, k and v pass through SiLU first if ``activation``; q and
    k are rotated over their first ``rotary`` elements (tables float32 [positions, rotary/2]); k is multiplied by
    ``k_scale``.  Per head S <- decay S + k v^T and o = S^T q, token by token in float32; ``state`` is float32
    [slots, heads, dim, vdim], read and written in the row ``slots[s]`` of each portion.  Returns o, float32
    [T, heads*vdim].  ``max_q_len``: the longest portion (0: unknown, taken as long); steps with portions of 16 tokens
    or more go chunk by chunk (three small products per 32 tokens), the others token by token."""
    _want(rows, "projections", _FLOAT, contiguous=False)
    ld = _rows_2d(rows, "projections")
    tokens = rows.shape[0]
    _want(decay, "decay", torch.float32)
    _want(state, "state", torch.float32)
    for name, t in (("slots", slots), ("q_start", q_start), ("positions", positions)):
        _want(t, name, torch.int32)
    if decay.numel() != heads or state.dim() != 4 or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"decay_scan: state must be [slots, {heads}, {dim}, {vdim}], got {tuple(state.shape)}; "
                          f"decay has {decay.numel()} elements")
    if max(q_off, k_off) + heads * dim > rows.shape[1] or v_off + heads * vdim > rows.shape[1]:
        raise KernelError("decay_scan: the projections' rows are too short for the given offsets")
    table_positions = 0
    if rotary > 0:
        _want(cos, "cos table", torch.float32)
        _want(sin, "sin table", torch.float32)
        if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != rotary // 2:
            raise KernelError(f"rotary tables must be [positions, {rotary // 2}], got {tuple(cos.shape)}")
        table_positions = cos.shape[0]
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=rows.device)
    longest = int(max_q_len) if max_q_len > 0 else tokens
    # the chunked kernels read q and k as the recurrence takes them from a buffer that one kernel fills per step
    prepared = (torch.empty((tokens, heads, 2, dim), dtype=torch.float32, device=rows.device)
                if longest >= 16 and dim <= 256 else None)
    # one long portion is shared out over many blocks in segments of 256 tokens: a state per segment in between
    carry = (torch.empty((tokens // 256 + num_seqs, heads, dim, vdim), dtype=torch.float32, device=rows.device)
             if prepared is not None and longest >= 512 and dim <= 128 and dim % 4 == 0 else None)
    lib = core()
    _check(lib.tge_decay_scan(rows.data_ptr(), int(rows.dtype == torch.bfloat16), ld, q_off, k_off, v_off, heads, dim,
                              vdim, int(activation), _ptr(cos) if rotary else None, _ptr(sin) if rotary else None,
                              table_positions, rotary, float(k_scale), decay.data_ptr(), state.data_ptr(),
                              slots.data_ptr(), q_start.data_ptr(), positions.data_ptr(), out.data_ptr(), num_seqs, tokens,
                              longest, _ptr(prepared), _ptr(carry), status_word().data_ptr(), _stream()), lib)
    return out


def gated_norm(o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], groups: int, eps: float,
               sigmoid: bool, out: Optional[torch.Tensor] = None, gate_first: bool = False,
               out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """out = o / rms(o) * weight * act(gate), the root mean square taken over each of ``groups`` equal runs of a
    row (one per head, or 1: all heads together).  ``o`` float32 [T, n]; ``gate`` run dtype [T, n] (dense rows, any
    row stride; it may be float32 while the rows go on in bfloat16: ``out_dtype``); ``weight`` float32 [n] or None; act is SiLU, or the logistic function with ``sigmoid``.  With
    ``gate_first`` the SiLU gate comes before the norm: out = y / rms(y) * weight, y = o * silu(gate)."""
    _want(o, "readout", torch.float32)
    _want(gate, "gate", _FLOAT, contiguous=False)
    tokens, width = o.shape
    if tuple(gate.shape) != (tokens, width) or width % groups:
        raise KernelError(f"gated_norm: readout {tuple(o.shape)}, gate {tuple(gate.shape)}, {groups} groups")
    if weight is not None:
        _want(weight, "norm weight", torch.float32)
        if weight.numel() != width:
            raise KernelError(f"gated_norm: weight has {weight.numel()} elements for rows of {width}")
    if out is None:
        out = torch.empty((tokens, width), dtype=out_dtype or gate.dtype, device=o.device)
    _want(out, "gated_norm output", _FLOAT, contiguous=False)       # a float32 gate may go with bfloat16 rows
    lib = core()
    _check(lib.tge_gated_norm(o.data_ptr(), gate.data_ptr(), int(gate.dtype == torch.bfloat16), _rows_2d(gate, "gate"),
                              _ptr(weight), out.data_ptr(), _rows_2d(out, "gated_norm output"), tokens, groups,
                              width // groups, float(eps), 2 if gate_first else int(sigmoid),
                              int(out.dtype == torch.bfloat16), _stream()), lib)
    return out


def conv_norm_rope_store(raw: torch.Tensor, conv_w: Optional[torch.Tensor], taps: int, conv_state: Optional[torch.Tensor],
                         slots: torch.Tensor, q_start: torch.Tensor, num_seqs: int, q_norm: Optional[torch.Tensor],
                         k_norm: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                         sin: Optional[torch.Tensor], rotary: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                         block_table: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
                         v_pages: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """What lies between the q/k/v product and the attention when the projections pass through a short causal
    convolution over time: y_t = sum_j w[:, j] u_(t - taps + 1 + j) on every channel (``conv_w`` float32 [channels,
    taps]; inputs from before the portion come from ``conv_state`` float32 [slots, taps-1, channels], which is then
    brought up to date), an RMS norm of each q and k head (weights float32 [dim], None: none), the rotation of their
    first ``rotary`` elements, and the store of k and v into their pages (None: nothing is stored).  ``raw`` [T, q | k
    | v] in the run dtype.  Returns the queries [T, heads*dim].  ``taps`` 0: no convolution."""
    _want(raw, "projections", _FLOAT, contiguous=False)
    ld = _rows_2d(raw, "projections")
    tokens = raw.shape[0]
    channels = (heads + kv_heads) * dim + kv_heads * vdim
    if raw.shape[1] < channels:
        raise KernelError(f"conv_norm_rope_store: rows of {raw.shape[1]} for {channels} channels")
    if taps:
        _want(conv_w, "convolution weights", torch.float32)
        if tuple(conv_w.shape) != (channels, taps):
            raise KernelError(f"convolution weights must be [{channels}, {taps}], got {tuple(conv_w.shape)}")
        if taps > 1:
            _want(conv_state, "convolution state", torch.float32)
            if conv_state.dim() != 3 or tuple(conv_state.shape[1:]) != (taps - 1, channels):
                raise KernelError(f"convolution state must be [slots, {taps - 1}, {channels}], got {tuple(conv_state.shape)}")
    for name, t in (("slots", slots), ("q_start", q_start), ("positions", positions), ("seq_of_token", seq_of_token)):
        _want(t, name, torch.int32)
    for name, t in (("q norm weight", q_norm), ("k norm weight", k_norm)):
        if t is not None:
            _want(t, name, torch.float32)
            if t.numel() != dim:
                raise KernelError(f"{name} has {t.numel()} elements for heads of {dim}")
    table_positions = 0
    if rotary > 0:
        _want(cos, "cos table", torch.float32)
        _want(sin, "sin table", torch.float32)
        if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != rotary // 2:
            raise KernelError(f"rotary tables must be [positions, {rotary // 2}], got {tuple(cos.shape)}")
        table_positions = cos.shape[0]
    store = k_pages is not None
    num_pages = page_size = max_pages = 0
    if store:
        _want(k_pages, "k pages", raw.dtype)
        _want(v_pages, "v pages", raw.dtype)
        _want(block_table, "block table", torch.int32)
        num_pages, _, page_size, _ = k_pages.shape
        if (tuple(k_pages.shape) != (num_pages, kv_heads, page_size, dim)
                or tuple(v_pages.shape) != (num_pages, kv_heads, page_size, vdim)):
            raise KernelError(f"pages must be [pages, {kv_heads}, page_size, {dim} | {vdim}], got "
                              f"{tuple(k_pages.shape)} and {tuple(v_pages.shape)}")
        max_pages = block_table.shape[1]
    q_out = torch.empty((tokens, heads * dim), dtype=raw.dtype, device=raw.device)
    lib = core()
    _check(lib.tge_conv_norm_rope_store(raw.data_ptr(), int(raw.dtype == torch.bfloat16), ld, _ptr(conv_w) if taps else None,
                                        int(taps), _ptr(conv_state) if taps > 1 else None, slots.data_ptr(),
                                        q_start.data_ptr(), _ptr(q_norm), _ptr(k_norm), float(eps),
                                        _ptr(cos) if rotary else None, _ptr(sin) if rotary else None, table_positions,
                                        rotary, positions.data_ptr(), seq_of_token.data_ptr(), _ptr(block_table), max_pages,
                                        _ptr(k_pages), _ptr(v_pages), num_pages, page_size, q_out.data_ptr(), heads * dim,
                                        tokens, num_seqs, heads, kv_heads, dim, vdim, int(store),
                                        status_word().data_ptr(), _stream()), lib)
    return q_out


def pool_kv(k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor, pooled_k: torch.Tensor,
            pooled_v: torch.Tensor, pool_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
            pool: int) -> None:
    """For every token of the step that is the last of a block of ``pool`` positions: the mean of the block's keys
    and of its values as the pages hold them, written as entry (position + 1) / pool - 1 of the request's pooled
    pages.  Pages [pages, kv_heads, page_size, dim | vdim]; both tables int32 [S, width]."""
    _want(k_pages, "k pages", _FLOAT)
    _want(v_pages, "v pages", k_pages.dtype)
    _want(pooled_k, "pooled k pages", k_pages.dtype)
    _want(pooled_v, "pooled v pages", k_pages.dtype)
    for name, t in (("block table", block_table), ("pooled block table", pool_table), ("positions", positions),
                    ("seq_of_token", seq_of_token)):
        _want(t, name, torch.int32)
    num_pages, kv_heads, page_size, dim = k_pages.shape
    vdim = v_pages.shape[3]
    if tuple(pooled_k.shape[1:]) != (kv_heads, page_size, dim) or tuple(pooled_v.shape[1:]) != (kv_heads, page_size, vdim):
        raise KernelError("pool_kv: pooled pages must be shaped like the keys' and values'")
    lib = core()
    _check(lib.tge_pool_kv(k_pages.data_ptr(), v_pages.data_ptr(), int(k_pages.dtype == torch.bfloat16),
                           block_table.data_ptr(), block_table.shape[1], num_pages, pooled_k.data_ptr(),
                           pooled_v.data_ptr(), pool_table.data_ptr(), pool_table.shape[1], pooled_k.shape[0], page_size,
                           positions.data_ptr(), seq_of_token.data_ptr(), positions.numel(), kv_heads, dim, vdim, int(pool),
                           status_word().data_ptr(), _stream()), lib)


# Fewer leading single-token sequences than this ride along in the prefill kernel: each fills one query tile,
# which costs less than another launch.
MIN_DECODE_PREFIX = 8


def choose_attention_split(tokens: int, num_seqs: int, max_q_len: int, max_ctx_len: int, heads: int,
                           kv_heads: int, bound: int = 0) -> int:
    """Keys per split for the tensor-core attention: enough blocks to fill the GPU, no more.

    The choice depends on the step's shape only through launch geometry; a row's value
    differs between choices by rounding alone.
    """
    if max_ctx_len <= 256:
        return 0
    group = heads // kv_heads
    if max_q_len <= 1 and group <= 16:
        blocks = num_seqs * kv_heads                      # the decode kernel: one block per (request, kv head)
    elif max_q_len > 1:
        # Portions of prompts.  Cutting their keys pays only where a block's keys are many and the rows to merge
        # few: a short portion deep in a long context.  A block takes 64 rows or more; a prompt of 320 tokens cut
        # in two took 18 us per layer for the attention and 34 us for merging its 8,960 rows of partial states.
        if max_ctx_len < 2048 or tokens * 4 > max_ctx_len:
            return 0
        blocks = -(-tokens // max(64 // group, 1)) * kv_heads
    else:
        blocks = num_seqs * kv_heads
    sms = core().tge_device_sm_count()
    most = -(-max_ctx_len // 128)                             # no split below 128 keys

    def keys_per_split(splits: int) -> int:
        return max(128, -(-(-(-max_ctx_len // splits)) // 64) * 64)

    if max_q_len > 1:
        # Two blocks fit on each SM (148 on a B200) and all blocks should run at once: a few more than that and
        # the last ones run alone.
        want_splits = min(2 * sms // blocks, most)
        return keys_per_split(want_splits) if want_splits > 1 else 0
    # Single tokens.  About one block per SM is best: every split more is a state more to write and to merge, and
    # the merging kernel holds sixteen states in registers (A/B in one process, ms per step of the 7B shape, 296
    # blocks against 148: batch 16 at context 2,048 3.33 / 3.22; batch 8 at 4,096 3.30 / 3.13; batch 4 at 4,096
    # 3.23 / 3.04; batch 4 at 30,000 4.05 / 3.89; batch 1 at 32,000 3.71 / 3.38).  Two exceptions, both measured:
    # splits of no more than 256 keys, sixteen at most over the whole bound, are better taken twice as many
    # (batch 8 at 2,048: 3.03 / 3.07); and requests that alone make half the SMs' worth of blocks or more are
    # still cut in two once their keys are many (batch 32 at 4,096: 4.29 / 4.57).
    want_splits = min(sms // blocks, most)
    twice = min(2 * sms // blocks, most)
    if twice > want_splits and keys_per_split(twice) <= 256 and -(-max(bound, max_ctx_len) // keys_per_split(twice)) <= 16:
        want_splits = twice
    if want_splits <= 1 and 2 * blocks <= 2 * sms and max_ctx_len >= 4096:
        want_splits = 2
    return keys_per_split(want_splits) if want_splits > 1 else 0


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits: arg-max where temperature <= 0, else a draw."""
    _want(logits, "logits", torch.float32, contiguous=False)
    stride = _rows_2d(logits, "logits")
    rows, vocab = logits.shape
    _want(temperature, "temperature", torch.float32)
    _want(uniform, "uniform draws", torch.float32)
    if temperature.numel() != rows or uniform.numel() != rows:
        raise KernelError("sample: one temperature and one uniform draw per row")
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _want(out, "sampled ids", torch.int32)
    lib = core()
    _check(lib.tge_sample(logits.data_ptr(), stride, temperature.data_ptr(), uniform.data_ptr(), out.data_ptr(), rows,
                          vocab, _stream()), lib)
    return out


def apply_penalty(logits: torch.Tensor, history: torch.Tensor, history_start: torch.Tensor,
                  penalty: torch.Tensor) -> torch.Tensor:
    """A copy of ``logits`` (float32 [R, V]) with the repetition penalty applied.

    ``history`` (int32) is every row's window of recent tokens, one after another;
    ``history_start`` (int32 [R + 1]) its offsets; ``penalty`` float32 [R], 1.0 = off.
    """
    _want(logits, "logits", torch.float32, contiguous=False)
    stride = _rows_2d(logits, "logits")
    rows, vocab = logits.shape
    for name, t, dtype in (("history", history, torch.int32), ("history offsets", history_start, torch.int32),
                           ("penalty", penalty, torch.float32)):
        _want(t, name, dtype)
    out = logits.clone()
    lib = core()
    _check(lib.tge_apply_penalty(logits.data_ptr(), out.data_ptr(), stride, history.data_ptr(),
                                 history_start.data_ptr(), penalty.data_ptr(), rows, vocab, _stream()), lib)
    return out


def sample_cuts(scores: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                min_p: torch.Tensor, uniform: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row with the top-k / min-p / top-p cuts (0 / 0.0 / 1.0 switch a cut off).  Given ``out``
    (int32 [rows], already holding ids), rows with every cut switched off are left as they are."""
    _want(scores, "scores", torch.float32, contiguous=False)
    stride = _rows_2d(scores, "scores")
    rows, vocab = scores.shape
    for name, t, dtype in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                           ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                           ("uniform draws", uniform, torch.float32)):
        _want(t, name, dtype)
        if t.numel() != rows:
            raise KernelError(f"sample_cuts: one {name} per row")
    lib = core()
    padded = lib.tge_sample_cuts_padded(vocab)
    sort_prob = torch.empty((rows, padded), dtype=torch.float32, device=scores.device)
    sort_index = torch.empty((rows, padded), dtype=torch.int32, device=scores.device)
    skip_uncut = out is not None
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=scores.device)
    _want(out, "sampled ids", torch.int32)
    if out.numel() != rows:
        raise KernelError("sample_cuts: one id per row")
    _check(lib.tge_sample_cuts(scores.data_ptr(), stride, temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                               min_p.data_ptr(), uniform.data_ptr(), sort_prob.data_ptr(), sort_index.data_ptr(),
                               out.data_ptr(), rows, vocab, int(skip_uncut), _stream()), lib)
    return out


# ----------------------------------------------------------------------------
# norms in groups, token shift
# ----------------------------------------------------------------------------
def group_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, out_dtype: torch.dtype,
               rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               weight2: Optional[torch.Tensor] = None):
    """RMS norm in ``groups`` equal consecutive parts of every float32 row (each part over its own root mean
    square), times ``weight``; rows optionally gathered by ``rows``.  ``out_dtype`` float32 or bfloat16; ``out`` may
    be ``x`` itself (float32, no gather): the stream normalised in place.  With ``weight2`` the same normalised rows
    are also written times that weight, and the result is the pair of outputs."""
    _want(x, "norm input", torch.float32)
    _want(weight, "norm weight", torch.float32)
    src_rows, width = x.shape
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {width}")
    out_rows = src_rows if rows is None else rows.numel()
    if rows is not None:
        _want(rows, "norm row index", torch.int32)
    if out is None:
        out = torch.empty((out_rows, width), dtype=out_dtype, device=x.device)
    _want(out, "norm output", _FLOAT)
    if tuple(out.shape) != (out_rows, width) or (out.data_ptr() == x.data_ptr() and (rows is not None or out.dtype != x.dtype)):
        raise KernelError("group_norm: the output must be [rows, width], and may be the input only ungathered in float32")
    out2 = None
    if weight2 is not None:
        _want(weight2, "second norm weight", torch.float32)
        if weight2.numel() != width or out.data_ptr() == x.data_ptr():
            raise KernelError("group_norm: a second weight of the row's width, and not in place")
        out2 = torch.empty_like(out)
    lib = core()
    _check(lib.tge_group_norm(x.data_ptr(), weight.data_ptr(), _ptr(rows), out.data_ptr(), int(out.dtype == torch.bfloat16),
                              out_rows, src_rows, width, int(groups), float(eps), _ptr(weight2), _ptr(out2),
                              status_word().data_ptr(), _stream()), lib)
    return out if weight2 is None else (out, out2)


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, seq_of_token: torch.Tensor,
                q_start: torch.Tensor, start_pos: torch.Tensor, num_seqs: int, update: bool = True) -> torch.Tensor:
    """out_t = h_t + (h_(t-1) - h_t) * mu, the row before a portion's first token taken from the request's row of
    ``state`` (float32 [slots, width]; zeros at position 0); with ``update`` every portion's last row of ``h`` then
    replaces its request's row of ``state``."""
    _want(h, "rows", _FLOAT)
    _want(mu, "shift weight", torch.float32)
    _want(state, "shift state", torch.float32)
    for name, t in (("slots", slots), ("seq_of_token", seq_of_token), ("q_start", q_start), ("start_pos", start_pos)):
        _want(t, name, torch.int32)
    tokens, width = h.shape
    if mu.numel() != width or state.dim() != 2 or state.shape[1] != width:
        raise KernelError(f"token_shift: weight of {mu.numel()} and state {tuple(state.shape)} for rows of {width}")
    out = torch.empty_like(h)
    lib = core()
    _check(lib.tge_token_shift(h.data_ptr(), int(h.dtype == torch.bfloat16), mu.data_ptr(), state.data_ptr(), slots.data_ptr(),
                               state.shape[0], seq_of_token.data_ptr(), q_start.data_ptr(), start_pos.data_ptr(), out.data_ptr(),
                               tokens, int(num_seqs), width, int(update), status_word().data_ptr(), _stream()), lib)
    return out


# ----------------------------------------------------------------------------
# attention over a latent cache
# ----------------------------------------------------------------------------
def latent_prepare(raw: torch.Tensor, q_rank: int, kv_rank: int, rot: int, gate_n: int, has_kv: bool,
                   q_weight: torch.Tensor, kv_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                   sin: Optional[torch.Tensor], rot_dims: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                   block_table: Optional[torch.Tensor], pages: Optional[torch.Tensor], out_dtype: torch.dtype):
    """From the float32 rows ``raw`` = [query latent | kv latent | shared key part | gate logits] (the middle two only
    with ``has_kv``): the RMS-normed query latent (run dtype [T, q_rank]) and the logistic gate (float32 [T, gate_n]);
    with ``pages`` ([num_pages, 1, page_size, kv_rank + rot]) the RMS-normed kv latent and the shared key part, its
    first ``rot_dims`` numbers rotated in neighbouring pairs by the float32 tables ``cos`` / ``sin`` [positions,
    rot_dims / 2], are written into each token's entry."""
    _want(raw, "latent rows", torch.float32, contiguous=False)
    ld = _rows_2d(raw, "latent rows")
    tokens = raw.shape[0]
    _want(q_weight, "query latent norm weight", torch.float32)
    if q_weight.numel() != q_rank:
        raise KernelError(f"latent_prepare: a norm weight of {q_weight.numel()} for a query latent of {q_rank}")
    max_pages = num_pages = page_size = max_positions = 0
    if has_kv:
        _want(kv_weight, "kv latent norm weight", torch.float32)
        if kv_weight.numel() != kv_rank:
            raise KernelError(f"latent_prepare: a norm weight of {kv_weight.numel()} for a kv latent of {kv_rank}")
    if has_kv and pages is not None:
        _want(pages, "latent pages", out_dtype)
        _want(block_table, "block table", torch.int32)
        if pages.dim() != 4 or pages.shape[1] != 1 or pages.shape[3] != kv_rank + rot:
            raise KernelError(f"latent_prepare: pages must be [pages, 1, page_size, {kv_rank + rot}], got {tuple(pages.shape)}")
        num_pages, page_size, max_pages = pages.shape[0], pages.shape[2], block_table.shape[1]
        max_positions = 2 ** 31 - 1
        if rot_dims:
            _want(cos, "cos table", torch.float32)
            _want(sin, "sin table", torch.float32)
            if cos.shape != sin.shape or cos.shape[1] != rot_dims // 2:
                raise KernelError(f"latent_prepare: tables {tuple(cos.shape)} for {rot_dims} rotated numbers")
            max_positions = cos.shape[0]
    _want(positions, "positions", torch.int32)
    _want(seq_of_token, "seq_of_token", torch.int32)
    q_latent = torch.empty((tokens, q_rank), dtype=out_dtype, device=raw.device)
    gate = torch.empty((tokens, gate_n), dtype=torch.float32, device=raw.device)
    lib = core()
    _check(lib.tge_latent_prepare(raw.data_ptr(), ld, q_rank, kv_rank, rot, gate_n, int(has_kv), q_weight.data_ptr(),
                                  _ptr(kv_weight), float(eps), _ptr(cos), _ptr(sin), rot_dims, max_positions,
                                  positions.data_ptr(), seq_of_token.data_ptr(), _ptr(block_table), max_pages, num_pages,
                                  page_size, _ptr(pages) if has_kv else None, q_latent.data_ptr(), gate.data_ptr(),
                                  int(out_dtype == torch.bfloat16), tokens, status_word().data_ptr(), _stream()), lib)
    return q_latent, gate


def head_linear(x: torch.Tensor, x_head: int, w: torch.Tensor, out: torch.Tensor, out_head: int,
                gate: Optional[torch.Tensor] = None, gate_mode: int = 0) -> torch.Tensor:
    """A product per head: out[t, n * out_head + j] = g * sum_k x[t, n * x_head + k] * w[n, j, k] for j < w.shape[1],
    k < w.shape[2].  ``x`` and ``out`` are 2-D with dense rows (views are fine; a head's run may be narrower than its
    stride).  ``gate`` float32 [T, heads] (``gate_mode`` 1) or [T, heads * outputs] (2) multiplies the result."""
    _want(x, "head_linear input", _FLOAT, contiguous=False)
    _want(w, "head_linear weight", x.dtype)
    _want(out, "head_linear output", x.dtype, contiguous=False)
    heads, n_out, k_in = w.shape
    tokens = x.shape[0]
    ldx, ldo = _rows_2d(x, "head_linear input"), _rows_2d(out, "head_linear output")
    if (out.shape[0] != tokens or (heads - 1) * x_head + k_in > x.shape[1] or (heads - 1) * out_head + n_out > out.shape[1]
            or x_head < k_in or out_head < n_out):
        raise KernelError(f"head_linear: {heads} heads of {k_in} -> {n_out} do not fit rows of {x.shape[1]} and {out.shape[1]}")
    gate_row = 0
    if gate_mode:
        _want(gate, "head_linear gate", torch.float32)
        gate_row = gate.shape[1]
        if gate.shape[0] != tokens or gate_row != (heads if gate_mode == 1 else heads * n_out):
            raise KernelError(f"head_linear: gate {tuple(gate.shape)} for mode {gate_mode}")
    lib = core()
    _check(lib.tge_head_linear(x.data_ptr(), ldx, int(x_head), w.data_ptr(), out.data_ptr(), ldo, int(out_head),
                               _ptr(gate) if gate_mode else None, int(gate_mode), gate_row, tokens, heads, n_out, k_in,
                               int(x.dtype == torch.bfloat16), _stream()), lib)
    return out


def rotate_interleaved(src: torch.Tensor, src_head: int, dst: torch.Tensor, dst_head: int, heads: int, width: int,
                       cos: torch.Tensor, sin: torch.Tensor, rot_dims: int, positions: torch.Tensor, first: int = 0) -> torch.Tensor:
    """dst[t, n * dst_head + e] = src[t, n * src_head + e] for e < width, with the ``rot_dims`` numbers of every
    run from ``first`` on rotated in neighbouring pairs: (u, v) at position p -> (u cos a - v sin a, v cos a + u sin a),
    a = p * f_i, from float32 tables [positions, rot_dims / 2].  Two buffers (or disjoint runs)."""
    _want(src, "rotation input", _FLOAT, contiguous=False)
    _want(dst, "rotation output", src.dtype, contiguous=False)
    _want(positions, "positions", torch.int32)
    lds, ldd = _rows_2d(src, "rotation input"), _rows_2d(dst, "rotation output")
    tokens = src.shape[0]
    if rot_dims:
        _want(cos, "cos table", torch.float32)
        _want(sin, "sin table", torch.float32)
        if cos.shape != sin.shape or cos.shape[1] != rot_dims // 2:
            raise KernelError(f"rotate_interleaved: tables {tuple(cos.shape)} for {rot_dims} rotated numbers")
    if (heads - 1) * src_head + width > src.shape[1] or (heads - 1) * dst_head + width > dst.shape[1] or dst.shape[0] != tokens:
        raise KernelError("rotate_interleaved: the runs do not fit the rows")
    lib = core()
    _check(lib.tge_rotate_interleaved(src.data_ptr(), lds, int(src_head), dst.data_ptr(), ldd, int(dst_head), _ptr(cos) if rot_dims else None,
                                      _ptr(sin) if rot_dims else None, int(rot_dims), cos.shape[0] if rot_dims else 2 ** 31 - 1,
                                      positions.data_ptr(), tokens, int(heads), int(width), int(first),
                                      int(src.dtype == torch.bfloat16), status_word().data_ptr(), _stream()), lib)
    return dst


def latent_gather(pages: torch.Tensor, table: torch.Tensor, page_seq: torch.Tensor, page_idx: torch.Tensor, ctx_len: torch.Tensor,
                  kv_rank: int, heads: int, latents: torch.Tensor, keys: torch.Tensor) -> None:
    """For attention with every head's own keys over a latent cache: fills the step's own pages.  ``pages`` [pool, 1,
    page, kv_rank + rot] found through ``table`` [S, max_pages]; own page p is request ``page_seq[p]``'s
    ``page_idx[p]``-th; ``ctx_len`` [S] positions held.  latents [>= own pages * page, kv_rank] gets every position's
    latent (zeros beyond what is held), keys [>= own pages, heads, page, per] the shared key part in the last rot
    numbers of every head's row."""
    _want(pages, "latent pages", _FLOAT)
    _want(latents, "latent rows", pages.dtype)
    _want(keys, "key pages", pages.dtype)
    for name, t in (("block table", table), ("page owners", page_seq), ("page indices", page_idx), ("context lengths", ctx_len)):
        _want(t, name, torch.int32)
    num_pages, one, page_size, entry = pages.shape
    own = page_seq.numel()
    per = keys.shape[3]
    if (one != 1 or keys.shape[0] < own or tuple(keys.shape[1:3]) != (heads, page_size) or latents.shape[1] != kv_rank
            or latents.shape[0] < own * page_size or per < entry - kv_rank or page_idx.numel() != own):
        raise KernelError("latent_gather: shapes do not agree")
    lib = core()
    _check(lib.tge_latent_gather(pages.data_ptr(), table.data_ptr(), table.shape[1], num_pages, page_seq.data_ptr(),
                                 page_idx.data_ptr(), ctx_len.data_ptr(), own, page_size, int(kv_rank), entry - int(kv_rank),
                                 int(heads), per, latents.data_ptr(), keys.data_ptr(), int(pages.dtype == torch.bfloat16),
                                 status_word().data_ptr(), _stream()), lib)


def latent_scatter(expanded: torch.Tensor, own_pages: int, dim: int, keys: torch.Tensor, values: torch.Tensor) -> None:
    """expanded [own pages * page, heads * dim + heads * vdim] (per position every head's plain key part, then every
    head's value) into keys [>= own pages, heads, page, per] (the first dim numbers of a row) and values [>= own
    pages, heads, page, vdim]."""
    _want(expanded, "expanded rows", _FLOAT, contiguous=False)
    _want(keys, "key pages", expanded.dtype)
    _want(values, "value pages", expanded.dtype)
    _, heads, page_size, per = keys.shape
    vdim = values.shape[3]
    if (expanded.shape[0] < own_pages * page_size or expanded.shape[1] != heads * (dim + vdim) or keys.shape[0] < own_pages
            or tuple(values.shape[:3]) != tuple(keys.shape[:3]) or per < dim):
        raise KernelError("latent_scatter: shapes do not agree")
    lib = core()
    _check(lib.tge_latent_scatter(expanded.data_ptr(), _rows_2d(expanded, "expanded rows"), int(own_pages), page_size, heads,
                                  int(dim), per, vdim, keys.data_ptr(), values.data_ptr(), int(expanded.dtype == torch.bfloat16),
                                  _stream()), lib)


def gate_rows(x: torch.Tensor, gate: torch.Tensor, heads: int, mode: int) -> torch.Tensor:
    """In place: x[t, n, j] *= gate[t, n] (mode 1, gate float32 [T, heads]) or gate[t, n, j] (mode 2, [T, heads * vdim])."""
    _want(x, "attended rows", _FLOAT, contiguous=False)
    _want(gate, "gate", torch.float32)
    tokens, width = x.shape
    if width % heads or gate.shape[0] != tokens or gate.shape[1] != (heads if mode == 1 else width):
        raise KernelError("gate_rows: shapes do not agree")
    lib = core()
    _check(lib.tge_gate_rows(x.data_ptr(), _rows_2d(x, "attended rows"), gate.data_ptr(), gate.shape[1], int(mode), tokens,
                             int(heads), width // heads, int(x.dtype == torch.bfloat16), _stream()), lib)
    return x


# ----------------------------------------------------------------------------
# routed feed-forward
# ----------------------------------------------------------------------------
ACT_RELU_SQUARED, ACT_XIELU = 0, 1


def router_topk(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, group_count: int = 1,
                group_keep: int = 1):
    """(ids int32 [T, top], weights float32 [T, top]) from float32 router logits [T, outputs]: scores = softmax over
    all outputs; the ``top`` outputs with the largest score + correction are chosen (the lowest index among equals),
    only inside the ``group_keep`` of ``group_count`` groups of neighbouring outputs whose best such value is largest;
    weights = the chosen outputs' scores over their sum (+ 1e-20)."""
    _want(logits, "router logits", torch.float32, contiguous=False)
    ld = _rows_2d(logits, "router logits")
    tokens, outputs = logits.shape
    if correction is not None:
        _want(correction, "router correction", torch.float32)
        if correction.numel() != outputs:
            raise KernelError(f"router_topk: a correction of {correction.numel()} for {outputs} outputs")
    ids = torch.empty((tokens, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=logits.device)
    lib = core()
    _check(lib.tge_router_topk(logits.data_ptr(), ld, _ptr(correction), tokens, outputs, int(top), int(group_count),
                               int(group_keep), ids.data_ptr(), weights.data_ptr(), _stream()), lib)
    return ids, weights


def activation(rows: torch.Tensor, kind: int, params: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place on run-dtype rows (a view with dense rows is fine).  ``ACT_RELU_SQUARED``: relu(z)^2.  ``ACT_XIELU``:
    z > 0: softplus(p) z^2 + z/2, else (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2, (p, q) = ``params`` float32 [2]."""
    _want(rows, "activation rows", _FLOAT, contiguous=False)
    ld = _rows_2d(rows, "activation rows")
    if kind == ACT_XIELU:
        _want(params, "activation parameters", torch.float32)
        if params.numel() != 2:
            raise KernelError("activation: two parameters")
    lib = core()
    _check(lib.tge_activation(rows.data_ptr(), ld, rows.shape[0], rows.shape[1], int(kind), _ptr(params),
                              int(rows.dtype == torch.bfloat16), _stream()), lib)
    return rows


def experts_direct(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                   x: torch.Tensor) -> None:
    """x[t] += sum_k weights[t, k] * (w_down[e] relu(w_up[e] h[t])^2 with e = ids[t, k], or h[t] itself when e is
    beyond the experts), every pair reading its expert's rows directly: for steps of few tokens.  w_up [experts, ff,
    width], w_down [width, experts, ff] (the experts' down matrices side by side), x float32 [T, width]."""
    _want(h, "expert input", _FLOAT, contiguous=False)
    _want(w_up, "expert up weights", h.dtype)
    _want(w_down, "expert down weights", h.dtype)
    _want(ids, "expert ids", torch.int32)
    _want(weights, "expert weights", torch.float32)
    _want(x, "stream", torch.float32)
    tokens, width = x.shape
    experts, ff = w_up.shape[0], w_up.shape[1]
    top = ids.shape[1]
    if w_up.shape[2] != width or tuple(w_down.shape) != (width, experts, ff) or h.shape[0] != tokens or h.shape[1] != width:
        raise KernelError("experts: shapes do not agree")
    inner = torch.empty((tokens * top, ff), dtype=h.dtype, device=h.device)
    lib = core()
    _check(lib.tge_experts_direct(h.data_ptr(), _rows_2d(h, "expert input"), w_up.data_ptr(), w_down.data_ptr(), ff,
                                  experts * ff, ids.data_ptr(), weights.data_ptr(), inner.data_ptr(), x.data_ptr(), tokens, top,
                                  experts, width, ff, int(h.dtype == torch.bfloat16), _stream()), lib)


def experts_dense_weigh(z: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, h: torch.Tensor, x: torch.Tensor,
                        experts: int) -> torch.Tensor:
    """In place on z [T, experts * ff] (every expert's up projection of every token): the rows of a token's chosen
    experts become weights[t, k] * relu(z)^2, all others zero; the share of choices beyond the experts (identity
    experts), weights[t, k] * h[t], is added into x (float32 [T, width]).  Returns z."""
    _want(z, "expert rows", _FLOAT)
    _want(h, "expert input", z.dtype, contiguous=False)
    _want(ids, "expert ids", torch.int32)
    _want(weights, "expert weights", torch.float32)
    _want(x, "stream", torch.float32)
    tokens, width = x.shape
    if z.shape[0] != tokens or z.shape[1] % experts or h.shape[0] != tokens or h.shape[1] != width or ids.shape[0] != tokens:
        raise KernelError("experts: shapes do not agree")
    lib = core()
    _check(lib.tge_experts_dense_weigh(z.data_ptr(), ids.data_ptr(), weights.data_ptr(), h.data_ptr(), _rows_2d(h, "expert input"),
                                       x.data_ptr(), tokens, ids.shape[1], int(experts), width, z.shape[1] // experts,
                                       int(z.dtype == torch.bfloat16), _stream()), lib)
    return z


def experts_group(h: torch.Tensor, ids: torch.Tensor, experts: int):
    """Groups the (token, choice) pairs by expert: (place int32 [T * top]: a pair's row among the grouped rows, -1 for
    choices beyond the experts; offsets int32 [experts + 1]; grouped [T * top, width]: copies of the pairs' input rows,
    expert e's at offsets[e] .. offsets[e + 1])."""
    _want(h, "expert input", _FLOAT, contiguous=False)
    _want(ids, "expert ids", torch.int32)
    tokens, width = h.shape
    top = ids.shape[1]
    place = torch.empty(tokens * top, dtype=torch.int32, device=h.device)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=h.device)
    grouped = torch.empty((tokens * top, width), dtype=h.dtype, device=h.device)
    lib = core()
    _check(lib.tge_experts_group(h.data_ptr(), _rows_2d(h, "expert input"), ids.data_ptr(), place.data_ptr(), offsets.data_ptr(),
                                 grouped.data_ptr(), tokens, top, int(experts), width, int(h.dtype == torch.bfloat16), _stream()), lib)
    return place, offsets, grouped


def experts_combine_add(outputs: torch.Tensor, place: torch.Tensor, weights: torch.Tensor, h: torch.Tensor,
                        x: torch.Tensor) -> None:
    """x[t] += sum_k weights[t, k] * (outputs[place[t, k]] or, where place is -1, h[t]); outputs float32 grouped rows."""
    _want(outputs, "expert outputs", torch.float32)
    _want(place, "expert places", torch.int32)
    _want(weights, "expert weights", torch.float32)
    _want(h, "expert input", _FLOAT, contiguous=False)
    _want(x, "stream", torch.float32)
    tokens, width = x.shape
    top = weights.shape[1]
    lib = core()
    _check(lib.tge_experts_combine_add(outputs.data_ptr(), place.data_ptr(), weights.data_ptr(), h.data_ptr(),
                                       _rows_2d(h, "expert input"), x.data_ptr(), tokens, top, width,
                                       int(h.dtype == torch.bfloat16), _stream()), lib)


# ----------------------------------------------------------------------------
# mixers with a matrix state that every token decays, corrects and reads; what surrounds them
# ----------------------------------------------------------------------------
GATED_DELTA, GATED_STATE_SPACE = 0, 1


def gated_prepare(raw: torch.Tensor, mode: int, groups: int, heads: int, dim: int, vdim: int, taps: int,
                  conv_w: torch.Tensor, conv_b: Optional[torch.Tensor], tails: Optional[torch.Tensor], slots: torch.Tensor,
                  q_start: torch.Tensor, seq_of_token: torch.Tensor, num_seqs: int, a_log: torch.Tensor,
                  dt_bias: torch.Tensor, unit_eps: float = 1e-6, q_scale: float = 1.0):
    """What the recurrence of :func:`gated_rule_scan` takes, from a mixer's input product ``raw`` (float32 [T, n]).

    ``GATED_DELTA``: raw = [q | k | v | gate | b | a] with q and k of ``groups`` heads x dim and v of heads x vdim;
    q, k and v pass a causal convolution over time per channel (``conv_w`` float32 [channels, taps], the last tap the
    current token's; ``tails`` float32 [slots, taps-1, channels] holds every request's last inputs and is brought up
    to date) and SiLU; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times ``q_scale``;
    decay = exp(-exp(a_log) softplus(a + dt_bias)), strength = sigmoid(b).
    ``GATED_STATE_SPACE``: raw = [z | x | B | C | dt] with x of heads x vdim and B, C of ``groups`` x dim; x, B and C
    pass the convolution (with ``conv_b``) and SiLU; q = C, k = B; dt <- softplus(dt + dt_bias), decay =
    exp(-exp(a_log) dt), strength = dt.
    Returns (qk float32 [T, groups, 2, dim], v float32 [T, heads * vdim], gates float32 [T, heads, 2])."""
    _want(raw, "projections", torch.float32, contiguous=False)
    ld = _rows_2d(raw, "projections")
    tokens = raw.shape[0]
    channels = 2 * groups * dim + heads * vdim
    _want(conv_w, "convolution taps", torch.float32)
    if tuple(conv_w.shape) != (channels, taps):
        raise KernelError(f"gated_prepare: taps must be [{channels}, {taps}], got {tuple(conv_w.shape)}")
    if conv_b is not None:
        _want(conv_b, "convolution bias", torch.float32)
        if conv_b.numel() != channels:
            raise KernelError(f"gated_prepare: the convolution's bias has {conv_b.numel()} elements for {channels} channels")
    if taps > 1:
        _want(tails, "convolution tails", torch.float32)
        if tails.dim() != 3 or tuple(tails.shape[1:]) != (taps - 1, channels):
            raise KernelError(f"gated_prepare: tails must be [slots, {taps - 1}, {channels}], got {tuple(tails.shape)}")
    for name, t in (("slots", slots), ("q_start", q_start), ("seq_of_token", seq_of_token)):
        _want(t, name, torch.int32)
    for name, t in (("a_log", a_log), ("dt_bias", dt_bias)):
        _want(t, name, torch.float32)
        if t.numel() != heads:
            raise KernelError(f"gated_prepare: {name} has {t.numel()} elements for {heads} heads")
    qk = torch.empty((tokens, groups, 2, dim), dtype=torch.float32, device=raw.device)
    v = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=raw.device)
    gates = torch.empty((tokens, heads, 2), dtype=torch.float32, device=raw.device)
    lib = core()
    _check(lib.tge_gated_prepare(raw.data_ptr(), ld, int(mode), groups, heads, dim, vdim, taps, conv_w.data_ptr(),
                                 _ptr(conv_b), _ptr(tails) if taps > 1 else None, slots.data_ptr(), q_start.data_ptr(),
                                 seq_of_token.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), float(unit_eps),
                                 float(q_scale), qk.data_ptr(), v.data_ptr(), gates.data_ptr(), tokens, num_seqs,
                                 _stream()), lib)
    return qk, v, gates


def gated_rule_scan(qk: torch.Tensor, v: torch.Tensor, gates: torch.Tensor, state: torch.Tensor, slots: torch.Tensor,
                    q_start: torch.Tensor, num_seqs: int, delta: bool, skip: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per head and request, token by token in float32: S <- a S; u = b (v - S^T k) with ``delta``, else u = b v;
    S <- S + k u^T; o = S^T q + skip v.  ``qk`` [T, groups, 2, dim] (q then k), ``v`` [T, heads * vdim], ``gates``
    [T, heads, 2] = (a, b), ``state`` float32 [slots, heads, dim, vdim] read and written in row ``slots[s]``; head h
    uses group h // (heads / groups); ``skip`` float32 [heads] or None.  Returns o float32 [T, heads * vdim]."""
    for name, t in (("q and k", qk), ("values", v), ("gates", gates), ("state", state)):
        _want(t, name, torch.float32)
    tokens, groups, _two, dim = qk.shape
    heads = gates.shape[1]
    vdim = v.shape[1] // heads
    if (tuple(v.shape) != (tokens, heads * vdim) or tuple(gates.shape) != (tokens, heads, 2) or state.dim() != 4
            or tuple(state.shape[1:]) != (heads, dim, vdim) or heads % groups):
        raise KernelError(f"gated_rule_scan: q/k {tuple(qk.shape)}, values {tuple(v.shape)}, gates {tuple(gates.shape)}, "
                          f"state {tuple(state.shape)}")
    if skip is not None:
        _want(skip, "skip weights", torch.float32)
        if skip.numel() != heads:
            raise KernelError(f"gated_rule_scan: {skip.numel()} skip weights for {heads} heads")
    _want(slots, "slots", torch.int32)
    _want(q_start, "q_start", torch.int32)
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=qk.device)
    lib = core()
    _check(lib.tge_gated_rule_scan(qk.data_ptr(), v.data_ptr(), gates.data_ptr(), _ptr(skip), int(delta), heads, groups, dim,
                                   vdim, state.data_ptr(), slots.data_ptr(), q_start.data_ptr(), out.data_ptr(), num_seqs,
                                   tokens, _stream()), lib)
    return out


def norm_scale_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, alpha: float = 1.0) -> None:
    """x (float32 [T, H]) += alpha * y / sqrt(mean(y^2) + eps) * weight, row by row; y float32 (dense rows)."""
    _want(x, "stream", torch.float32)
    _want(y, "addend", torch.float32, contiguous=False)
    _want(weight, "norm weight", torch.float32)
    if x.shape != y.shape or weight.numel() != x.shape[1]:
        raise KernelError(f"norm_scale_add: {tuple(x.shape)}, {tuple(y.shape)}, weight of {weight.numel()}")
    lib = core()
    _check(lib.tge_norm_scale_add(x.data_ptr(), y.data_ptr(), _rows_2d(y, "addend"), weight.data_ptr(), x.shape[0],
                                  x.shape[1], float(alpha), float(eps), _stream()), lib)


def qk_temp_store(qk: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                  temp_coef: float, temp_every: int, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  block_table: Optional[torch.Tensor], k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                  heads: int, kv_heads: int, head_dim: int) -> None:
    """After the q/k product of an attention whose values are its keys as projected: rows ``qk`` [T, q | k].  The
    values' pages get k as it arrives; q and k are then normalised per head (weights float32 [head_dim], None: not
    normalised), q is multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (``temp_every`` 0: not) and
    rewritten in place, and k goes to its pages.  Pages None: nothing is stored."""
    _want(qk, "q and k", _FLOAT, contiguous=False)
    stride = _rows_2d(qk, "q and k")
    for name, t in (("q norm weight", q_weight), ("k norm weight", k_weight)):
        if t is not None:
            _want(t, name, torch.float32)
            if t.numel() != head_dim:
                raise KernelError(f"{name} has {t.numel()} elements for heads of {head_dim}")
    _want(positions, "positions", torch.int32)
    _want(seq_of_token, "seq_of_token", torch.int32)
    store = k_pages is not None
    num_pages = page_size = max_pages = 0
    if store:
        _want(k_pages, "k pages", qk.dtype)
        _want(v_pages, "v pages", qk.dtype)
        _want(block_table, "block table", torch.int32)
        num_pages, _, page_size, _ = k_pages.shape
        if tuple(k_pages.shape) != (num_pages, kv_heads, page_size, head_dim) or v_pages.shape != k_pages.shape:
            raise KernelError(f"pages must be [pages, {kv_heads}, page_size, {head_dim}], got {tuple(k_pages.shape)} and "
                              f"{tuple(v_pages.shape)}")
        max_pages = block_table.shape[1]
    lib = core()
    _check(lib.tge_qk_temp_store(qk.data_ptr(), int(qk.dtype == torch.bfloat16), stride, _ptr(q_weight), _ptr(k_weight),
                                 float(eps), float(temp_coef), int(temp_every), positions.data_ptr(), seq_of_token.data_ptr(),
                                 _ptr(block_table), max_pages, _ptr(k_pages), _ptr(v_pages), num_pages, page_size,
                                 qk.shape[0], heads, kv_heads, head_dim, int(store), status_word().data_ptr(), _stream()), lib)


def gated_clamp_act(rows: torch.Tensor, limit: float, alpha: float, offset: float, out_dtype: torch.dtype,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``rows`` float32 [T, 2 n] with (g_i, u_i) side by side -> [T, n]: min(g, L) sigmoid(alpha min(g, L))
    (clamp(u, -L, L) + offset)."""
    _want(rows, "gate and up rows", torch.float32, contiguous=False)
    tokens, both = rows.shape
    if both % 2:
        raise KernelError("gated_clamp_act: rows hold pairs")
    if out is None:
        out = torch.empty((tokens, both // 2), dtype=out_dtype, device=rows.device)
    _want(out, "activated rows", _FLOAT, contiguous=False)
    lib = core()
    _check(lib.tge_gated_clamp_act(rows.data_ptr(), _rows_2d(rows, "gate and up rows"), out.data_ptr(),
                                   _rows_2d(out, "activated rows"), int(out.dtype == torch.bfloat16), tokens, both // 2,
                                   float(limit), float(alpha), float(offset), _stream()), lib)
    return out


def concat_rows(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """[a | b] of two float32 [T, H] tensors, in ``out_dtype``."""
    _want(a, "rows", torch.float32)
    _want(b, "rows", torch.float32)
    if a.shape != b.shape:
        raise KernelError("concat_rows: shapes differ")
    out = torch.empty((a.shape[0], 2 * a.shape[1]), dtype=out_dtype, device=a.device)
    lib = core()
    _check(lib.tge_concat_rows(a.data_ptr(), b.data_ptr(), out.data_ptr(), int(out_dtype == torch.bfloat16), a.shape[0],
                               a.shape[1], _stream()), lib)
    return out
