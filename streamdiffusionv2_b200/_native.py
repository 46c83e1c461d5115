"""ctypes binding of libsdv2.so (see include/sdv2.h).  There is no fallback: if the library is
missing or a call fails, an exception is raised."""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsdv2.so")

MAX_ROWS = 64
DTYPE_BF16, DTYPE_F32 = 0, 1
ERR_TIMEOUT = -5
ERR_INVALID_ARG = -1


class View(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_row", C.c_int64), ("stride_tok", C.c_int64),
                ("stride_head", C.c_int64)]


class NativeError(RuntimeError):
    def __init__(self, code: int, what: str, msg: str):
        super().__init__(f"{what}: {msg} (code {code})")
        self.code = code


_lib = None

_SIGNATURES = {
    "sdv2_abi_version": (C.c_int, []),
    "sdv2_strerror": (C.c_char_p, [C.c_int]),
    "sdv2_last_cuda_error": (C.c_int, []),
    "sdv2_rope_kv_append": (C.c_int, [C.POINTER(View)] * 6 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                                               C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                               C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                                               C.c_void_p, C.c_void_p,
                                                               C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                                               C.c_int, C.c_void_p, C.c_void_p]),
    "sdv2_rope_kv_append_indirect": (C.c_int, [C.POINTER(View)] * 6 + [C.c_int, C.c_int, C.c_int, C.c_int,
                                                                        C.c_int64, C.c_void_p, C.c_int, C.c_int,
                                                                        C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                                                        C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "sdv2_norm_rope_kv_append": (C.c_int, [C.POINTER(View)] * 6 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                                                    C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                                    C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                                                    C.c_void_p, C.c_void_p, C.c_void_p,
                                                                    C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                                                    C.c_void_p, C.c_void_p, C.c_float,
                                                                    C.c_void_p, C.c_void_p]),
    "sdv2_frame_means": (C.c_int, [C.POINTER(View)] * 4 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                                            C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "sdv2_frame_means_scratch_bytes": (C.c_size_t, [C.c_int] * 4),
    "sdv2_ring_plan_adaptive": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_int,
                                          C.c_int64, C.c_int64, C.POINTER(C.c_int64), C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p]),
    "sdv2_attn_kvcache": (C.c_int, [C.POINTER(View)] * 4 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                                             C.POINTER(C.c_int32), C.c_float, C.c_void_p,
                                                             C.c_size_t, C.c_void_p]),
    "sdv2_attn_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "sdv2_cross_attn": (C.c_int, [C.POINTER(View)] * 4 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                           C.c_float, C.c_void_p, C.c_size_t, C.c_void_p]),
    "sdv2_attn_kvcache_simt": (C.c_int, [C.POINTER(View)] * 4 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                                                  C.POINTER(C.c_int32), C.c_float, C.c_int,
                                                                  C.c_void_p]),
    "sdv2_attn_kvcache_static": (C.c_int, [C.POINTER(View)] * 4 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64,
                                                                    C.POINTER(C.c_int32), C.c_float,
                                                                    C.POINTER(C.c_void_p), C.c_void_p]),
    "sdv2_rmsnorm": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int,
                               C.c_float, C.c_void_p]),
    "sdv2_ln_modulate": (C.c_int, [C.c_void_p] * 3 + [C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                      C.c_float, C.c_void_p]),
    "sdv2_gate_residual": (C.c_int, [C.c_void_p] * 3 + [C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                        C.c_void_p]),
    "sdv2_layernorm_affine": (C.c_int, [C.c_void_p] * 4 + [C.c_int64, C.c_int, C.c_float, C.c_void_p]),
    "sdv2_gelu_tanh": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "sdv2_residual_layernorm": (C.c_int, [C.c_void_p] * 3 + [C.c_int64, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                                             C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                                             C.c_float, C.c_void_p]),
    "sdv2_read_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.c_void_p]),
    "sdv2_selftest_umma": (C.c_int, [C.c_void_p] * 4 + [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sdv2_selftest_wait_timeout": (C.c_int, [C.c_void_p, C.c_longlong, C.c_void_p]),
    "sdv2_attn_partial_slots": (C.c_int, [C.c_int] * 5),
}


def exported_symbols():
    """Names declared in include/sdv2.h that the binding expects the library to export."""
    return sorted(_SIGNATURES)


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m streamdiffusionv2_b200.build` "
                "(there is no fallback path)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        if l.sdv2_abi_version() != 1:
            raise RuntimeError("libsdv2.so ABI version mismatch; rebuild it")
        _lib = l
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        l = lib()
        msg = l.sdv2_strerror(code).decode()
        if code == -4:
            msg += f" [cuda error {l.sdv2_last_cuda_error()}]"
        raise NativeError(code, what, msg)


def view(t: torch.Tensor) -> View:
    """[rows, tokens, heads, head_dim] tensor -> View (head_dim must be contiguous)."""
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError("expected a [rows, tokens, heads, head_dim] tensor with contiguous head_dim")
    if not t.is_cuda:
        raise ValueError("expected a CUDA tensor (there is no CPU path)")
    # a size-1 row dimension may carry any stride; give it a legal one
    stride_row = t.stride(0) if t.shape[0] > 1 else t.shape[1] * t.stride(1)
    return View(t.data_ptr(), stride_row, t.stride(1), t.stride(2))


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return DTYPE_BF16
    if dt == torch.float32:
        return DTYPE_F32
    raise ValueError(f"unsupported dtype {dt}")


def i64_array(vals: Sequence[int]):
    return (C.c_int64 * len(vals))(*[int(v) for v in vals])


def i32_array(vals: Sequence[int]):
    return (C.c_int32 * len(vals))(*[int(v) for v in vals])


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
