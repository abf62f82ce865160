"""ctypes signatures of the native library and small marshalling helpers."""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p
from typing import Any, Optional

import torch

from .. import _native

_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

_SIGNATURES = {
    "fsb_gemm_bf16": [c_void_p] * 6 + [c_int] * 13 + [c_void_p, c_void_p],
    "fsb_gemm_bf16_streamed_a": [c_void_p] * 4 + [c_int] * 7 + [c_void_p, c_uint] + [c_int] * 4 + [c_longlong, c_void_p, c_void_p],
    "fsb_gemm_bf16_streamed_b": [c_void_p] * 4 + [c_int] * 6 + [c_void_p, c_uint, c_longlong, c_int, c_longlong, c_void_p, c_void_p],
    "fsb_adam_chunk_size": [],
    "fsb_multi_tensor_adam": [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int] + [c_float] * 8 + [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "fsb_multi_tensor_sumsq": [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p],
    "fsb_multi_tensor_scale": [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p],
    "fsb_norm_fwd": [c_void_p] * 6 + [c_longlong, c_int, c_float, c_int, c_void_p],
    "fsb_norm_bwd_num_strips": [c_longlong],
    "fsb_norm_bwd": [c_void_p] * 9 + [c_longlong, c_int, c_int, c_void_p],
    "fsb_colsum_num_strips": [c_longlong],
    "fsb_colsum": [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p],
    "fsb_ce_fwd": [c_void_p] * 5 + [c_longlong, c_int, c_longlong, c_longlong, c_longlong, c_void_p],
    "fsb_ce_bwd": [c_void_p] * 4 + [c_int, c_float, c_void_p, c_longlong, c_int, c_longlong, c_longlong, c_longlong, c_void_p],
    "fsb_embedding_fwd": [c_void_p] * 4 + [c_longlong, c_int, c_int, c_longlong, c_longlong, c_float, c_void_p],
    "fsb_embedding_bwd": [c_void_p] * 4 + [c_longlong, c_int, c_int, c_longlong, c_longlong, c_float, c_void_p],
    "fsb_cast": [c_void_p, c_int, c_void_p, c_int, c_longlong, c_float, c_void_p],
    "fsb_accum_bf16_into_f32": [c_void_p, c_void_p, c_longlong, c_float, c_int, c_void_p],
    "fsb_gelu": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    "fsb_swiglu_fwd": [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    "fsb_swiglu_bwd": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    "fsb_add_bf16": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p],
    "fsb_rope": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "fsb_dropout": [c_void_p, c_void_p, c_longlong, c_float, c_ulonglong, c_ulonglong, c_void_p],
    "fsb_delay": [c_ulonglong, c_void_p],
    "fsb_softmax": [c_void_p, c_void_p, c_longlong, c_int, c_int, c_float, c_int, c_int, c_void_p],
}

_bound: dict = {}
_launch_count = 0


def fn(name: str) -> Any:
    """Bound native function with argtypes set (cached)."""
    f = _bound.get(name)
    if f is None:
        f = getattr(_native.lib(), name)
        if name in _SIGNATURES:
            f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _bound[name] = f
    return f


def call(name: str, *args: Any, launches: int = 1) -> None:
    """Invoke a native entry point and raise on a non-zero return code."""
    global _launch_count
    code = fn(name)(*args)
    if code != 0:
        raise RuntimeError(f"{name} failed with code {code}")
    _launch_count += launches


def launch_count() -> int:
    """Number of kernels of this library launched so far by this process."""
    return _launch_count


def add_launches(n: int) -> None:
    global _launch_count
    _launch_count += n


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: Any = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    return _DTYPE_CODE[dt]


def use_native(*tensors: Any) -> bool:
    return _native.use_native(*tensors)


def status_ptr(device: Any) -> int:
    return _native.status_word(device).data_ptr()
