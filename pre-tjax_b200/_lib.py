"""ctypes binding of libptj_b200.so (the C ABI declared in include/ptj_b200.h).

There is no CPU or PyTorch fallback: if the library is missing, or an entry point returns a non-zero status, a
RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_uint8, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libptj_b200.so"

PTJ_F32, PTJ_BF16 = 0, 1
EPI_NONE, EPI_GELU, EPI_GELU_BWD, EPI_DROPOUT_RESID, EPI_ACCUM = 0, 1, 2, 3, 4


class DropoutArgs(ctypes.Structure):
    _fields_ = [("p", c_float), ("train", c_int), ("seed", c_uint64), ("stream_id", c_uint32)]


class GemmProblem(ctypes.Structure):
    _fields_ = [("a", c_void_p), ("b", c_void_p), ("c", c_void_p), ("M", c_int64), ("N", c_int64), ("lda", c_int64),
                ("ldb", c_int64), ("ldc", c_int64), ("out_dtype", c_int), ("epilogue", c_int), ("split_k", c_int),
                ("workspace", c_void_p),
                ("workspace_floats", c_size_t)]


class AttnShape(ctypes.Structure):
    _fields_ = [
        ("batch", c_int64), ("heads", c_int64), ("seq", c_int64), ("d_head", c_int64),
        ("q_strides", c_int64 * 3), ("k_strides", c_int64 * 3), ("v_strides", c_int64 * 3), ("o_strides", c_int64 * 3),
    ]


_P = c_void_p
_SIGNATURES = {
    "ptj_version": (c_int, []),
    "ptj_status_string": (c_char_p, [c_int]),
    "ptj_device_check": (c_int, []),
    "ptj_launch_count": (c_int64, []),
    "ptj_last_kernel_fault": (c_int, [_P, POINTER(ctypes.c_uint)]),
    "ptj_layernorm_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int, _P]),
    "ptj_layernorm_bwd_scratch_floats": (c_size_t, [c_int64, c_int64]),
    "ptj_layernorm_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_size_t, c_int64, c_int64, c_int, _P]),
    "ptj_layernorm_bwd_dropout": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_size_t, c_int64, c_int64, c_float, c_int,
                                          c_uint64, c_uint32, c_int, _P]),
    "ptj_layernorm_bwd_noalloc_max_dim": (c_size_t, []),
    "ptj_layernorm_bwd_noalloc": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, _P]),
    "ptj_gelu_fwd": (c_int, [_P, _P, c_int64, c_int, _P]),
    "ptj_gelu_bwd": (c_int, [_P, _P, _P, c_int64, c_int, _P]),
    "ptj_gelu_bwd_colsum": (c_int, [_P, _P, _P, _P, _P, c_size_t, c_int64, c_int64, c_int64, c_int, _P]),
    "ptj_dropout": (c_int, [_P, _P, _P, c_int64, c_float, c_int, c_uint64, c_uint32, c_int, _P]),
    "ptj_log_softmax_fwd": (c_int, [_P, _P, c_int64, c_int64, c_int64, c_int64, c_int, _P]),
    "ptj_log_softmax_bwd": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, _P]),
    "ptj_cross_entropy": (c_int, [_P, _P, _P, _P, _P, c_int, _P, c_int64, c_int64, c_int64, c_int, _P]),
    "ptj_argmax_rows": (c_int, [_P, _P, c_int64, c_int64, c_int64, c_int, _P]),
    "ptj_embed_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_uint64, c_uint32,
                              c_int, c_int, _P]),
    "ptj_embed_bwd": (c_int, [_P, _P, _P, _P, _P, c_int, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_uint64,
                              c_uint32, c_int, _P]),
    "ptj_colsum_scratch_floats": (c_size_t, [c_int64, c_int64]),
    "ptj_colsum": (c_int, [_P, _P, _P, c_size_t, c_int64, c_int64, c_int64, c_int, _P]),
    "ptj_gemm": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                         c_int, c_int, c_int, POINTER(DropoutArgs), c_int, _P, c_size_t, _P]),
    "ptj_gemm_tail_split_floats": (c_size_t, [c_int64, c_int64, c_int64]),
    "ptj_gemm_tail_split_rows": (c_int64, [c_int64, c_int64, c_int64]),
    "ptj_gemm_grouped2": (c_int, [POINTER(GemmProblem), POINTER(GemmProblem), c_int64, c_int, c_int, _P]),
    "ptj_attn_keep_bits_bytes": (c_size_t, [POINTER(AttnShape), c_int]),
    "ptj_attn_keep_bits": (c_int, [_P, POINTER(AttnShape), c_float, c_uint64, c_uint32, c_int, _P]),
    "ptj_attn_fwd": (c_int, [_P, _P, _P, _P, _P, _P, POINTER(AttnShape), c_float, c_int, c_uint64, c_uint32, _P, _P, c_int,
                             _P]),
    "ptj_attn_bwd_workspace_bytes": (c_size_t, [POINTER(AttnShape), c_int]),
    "ptj_attn_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, POINTER(AttnShape), POINTER(AttnShape), c_float,
                             c_int, c_uint64, c_uint32, _P, _P, _P, c_size_t, c_int, _P]),
    "ptj_sumsq_scratch_floats": (c_size_t, [c_int64]),
    "ptj_sumsq": (c_int, [_P, _P, _P, c_size_t, c_int64, _P]),
    "ptj_adamw": (c_int, [_P, _P, _P, _P, _P, c_int64, _P, _P, c_int, c_float, c_float, c_float, c_float, c_float,
                          c_int64, c_float, _P, c_float, _P]),
    "ptj_cast_f32_to_bf16": (c_int, [_P, _P, c_int64, _P]),
}

_lib = None


def exported_symbols() -> list[str]:
    """Names this binding expects the shared library to export."""
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the sm_100a kernels first (python pre-tjax_b200/build.py). "
                "There is no fallback implementation."
            )
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().ptj_status_string(status).decode()
        raise RuntimeError(f"{what} failed with status {status}: {msg}")


def launch_count() -> int:
    return int(lib().ptj_launch_count())
