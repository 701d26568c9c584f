"""ctypes binding of libkandle_cuda.so (the C ABI declared in include/kandle_cuda.h).

This is the Python twin of the N-API / FFI stub a Kandle `backend-cuda` package would carry: it
only loads the library, declares argument types and turns non-zero status codes into exceptions.
There is no fallback: if the library has not been built the import of this module fails.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

KD_MAX_DIMS = 8

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libkandle_cuda.so")


class KandleCudaError(RuntimeError):
    """Raised for every non-zero kd_status (the reference throws a JS Error at the same points)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[kd_status {status}] {message}")
        self.status = status


class kd_tensor(ctypes.Structure):
    _fields_ = [
        ("storage", ctypes.c_uint64),
        ("offset", ctypes.c_int64),
        ("dtype", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("shape", ctypes.c_int64 * KD_MAX_DIMS),
        ("strides", ctypes.c_int64 * KD_MAX_DIMS),
    ]


class kd_matmul_cfg(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
        ("transpose_a", ctypes.c_int32), ("transpose_b", ctypes.c_int32),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("has_c", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


# logical dtype name <-> kd_dtype code, element size, numpy type used on the host side
DTYPES = {
    "float32": (0, 4, np.float32),
    "float16": (1, 2, np.float16),
    "bfloat16": (2, 2, np.uint16),  # numpy has no bfloat16: raw bits on the host
    "int32": (3, 4, np.int32),
    "int64": (4, 8, np.int64),
    "uint8": (5, 1, np.uint8),
    "bool": (6, 1, np.bool_),
}
DTYPE_NAMES = {v[0]: k for k, v in DTYPES.items()}

POINTWISE_OPS = {
    "add": 0, "mul": 1, "mul_scalar": 2, "neg": 3, "cos": 4, "sin": 5, "silu": 6, "gelu": 7, "abs": 8,
    "div": 9, "maximum": 10, "tanh": 11, "sigmoid": 12, "sub": 13,
}


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even conversion of float32 to bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    out = (rounded >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(a)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_to_bf16(a: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bfloat16, still stored as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(a)).reshape(np.shape(a))


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python kandle_b200/build.py` (needs nvcc). "
        "kandle_b200 has no CPU fallback.")

_lib = ctypes.CDLL(LIB_PATH)

_T = ctypes.POINTER(kd_tensor)
_u64 = ctypes.c_uint64
_SIGNATURES = {
    "kd_init": [ctypes.c_int, ctypes.c_uint],
    "kd_shutdown": [],
    "kd_synchronize": [],
    "kd_device_count": [ctypes.POINTER(ctypes.c_int)],
    "kd_last_error": [ctypes.c_char_p, ctypes.c_size_t],
    "kd_stream": [ctypes.POINTER(ctypes.c_void_p)],
    "kd_selftest_wait_timeout": [ctypes.c_uint32],
    "kd_launch_count": [ctypes.POINTER(_u64), ctypes.c_int],
    "kd_storage_alloc": [_u64, ctypes.c_int, ctypes.POINTER(_u64)],
    "kd_storage_retain": [_u64],
    "kd_storage_release": [_u64],
    "kd_storage_bytes": [_u64, ctypes.POINTER(_u64)],
    "kd_storage_device_ptr": [_u64, ctypes.POINTER(ctypes.c_void_p)],
    "kd_upload": [_u64, _u64, ctypes.c_void_p, _u64],
    "kd_download": [_u64, _u64, ctypes.c_void_p, _u64],
    "kd_upload_async": [_u64, _u64, ctypes.c_void_p, _u64],
    "kd_download_async": [_u64, _u64, ctypes.c_void_p, _u64],
    "kd_host_alloc_pinned": [_u64, ctypes.POINTER(ctypes.c_void_p)],
    "kd_host_free_pinned": [ctypes.c_void_p],
    "kd_memory_stats": [ctypes.POINTER(_u64), ctypes.POINTER(_u64), ctypes.POINTER(_u64)],
    "kd_empty_cache": [],
    "kd_workspace_bytes": [ctypes.POINTER(_u64)],
    "kd_debug_fill_scratch": [ctypes.c_int],
    "kd_flash_attention": [_T, _T, _T, _T, ctypes.c_float, ctypes.c_int],
    "kd_matmul": [ctypes.POINTER(kd_matmul_cfg), _T, _T, _T, _T],
    "kd_rms_norm": [_T, _T, ctypes.c_float, _T],
    "kd_layer_norm": [_T, _T, _T, ctypes.c_float, _T],
    "kd_softmax": [_T, _T],
    "kd_index_select": [_T, _T, ctypes.c_int, _T],
    "kd_pointwise": [ctypes.c_int, _T, _T, ctypes.c_float, _T],
    "kd_copy": [_T, _T],
    "kd_fill": [_T, ctypes.c_double],
    "kd_arange": [_T, ctypes.c_double, ctypes.c_double],
    "kd_argmax": [_T, _T],
    "kd_randn": [_T, _u64, ctypes.c_uint32, ctypes.c_float, ctypes.c_float, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64],
    "kd_conv1d": [_T, _T, _T, ctypes.c_int, ctypes.c_int, _T],
    "kd_event_create": [ctypes.POINTER(_u64)],
    "kd_event_record": [_u64],
    "kd_event_elapsed_ms": [_u64, _u64, ctypes.POINTER(ctypes.c_float)],
    "kd_event_destroy": [_u64],
    "kd_linear_bf16": [_T, _T, _T, ctypes.c_int, _T],
    "kd_conv1d_tokens_bf16": [_T, _T, _T, _T, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _T],
    "kd_linear_bf16_bias": [_T, _T, _T, _T, ctypes.c_int, _T],
    "kd_linear_bf16_skinny": [_T, _T, ctypes.c_int, _T],
    "kd_linear_bf16_skinny_splits": [ctypes.c_int64, ctypes.c_int64, ctypes.POINTER(ctypes.c_int)],
    "kd_rope_table": [_T, _T, ctypes.c_int, ctypes.c_int, _T, _T],
    "kd_qkv_norm_rope_cachewrite": [_T, _T, _T, ctypes.c_float, _T, _T, _T, _T, _T, ctypes.c_int, _T],
    "kd_qkv_norm_rope_cachewrite_paged": [_T, _T, _T, ctypes.c_float, _T, _T, _T, _T, _T, _T, ctypes.c_int, _T],
    "kd_kv_pages_write": [_T, _T, _T, _T, _T, ctypes.c_int],
    "kd_qkv_linear_norm_rope_cachewrite": [_T, _T, _T, _T, ctypes.c_float, _T, _T, _T, _T, ctypes.c_int, _T],
    "kd_swiglu": [_T, _T],
    "kd_add_rmsnorm": [_T, _T, _T, ctypes.c_float, _T, _T],
    "kd_increment_i32": [_T, ctypes.c_int],
    "kd_stft_frames": [_T, _T, ctypes.c_int, ctypes.c_int, ctypes.c_int, _T],
    "kd_power_spectrum": [_T, _T],
    "kd_whisper_log_mel_norm": [_T, _T],
    "kd_sample": [_T, ctypes.c_double, ctypes.c_int, ctypes.c_double, ctypes.c_int, _T, _T, _T],
    "kd_decode_layer_chain": [_T, _T, _T, _T, _T, _T, _T, ctypes.c_float, _T, _T, _T, _T, _T, _T],
    "kd_decode_layer_fused": [_T, _T, _T, _T, _T, _T, _T, ctypes.c_float, _T, _T, _T, _T, _T, _T, _T, _T, _T, _T, _T, _T],
    "kd_decode_layer_fused_tp": [_T, _T, _T, _T, _T, _T, _T, ctypes.c_float, _T, _T, _T, _T, _T, _T, _T, _T, _T, _T, _T, _T],
    "kd_debug_decode_layer_plan": [ctypes.c_int] * 9 + [ctypes.POINTER(ctypes.c_int), ctypes.c_int],
    "kd_debug_decode_layer_trace": [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int],
    "kd_decode_layer_chain_splits": [ctypes.c_int64, ctypes.c_int64, ctypes.POINTER(ctypes.c_int)],
    "kd_set_pdl": [ctypes.c_int],
    "kd_graph_begin": [],
    "kd_graph_end": [ctypes.POINTER(_u64)],
    "kd_graph_launch": [_u64],
    "kd_graph_destroy": [_u64],
    "kd_comm_unique_id": [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t],
    "kd_comm_init": [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t],
    "kd_comm_info": [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
    "kd_allreduce_sum": [_T],
    "kd_comm_check": [],
    "kd_comm_destroy": [],
    "kd_p2p_prepare": [ctypes.c_char_p, ctypes.c_size_t],
    "kd_p2p_connect": [ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t],
    "kd_p2p_emulate": [ctypes.c_int],
    "kd_p2p_info": [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)],
    "kd_p2p_disconnect": [],
    "kd_allreduce_add_rmsnorm": [_T, _T, _T, ctypes.c_float, _T, _T],
    "kd_p2p_selftest_dropped_flag": [_T, _T, _T, ctypes.c_int, ctypes.c_uint32],
    "kd_p2p_selftest_silent_peers": [ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32],
    "kd_attention_decode": [_T, _T, _T, _T, ctypes.c_int, ctypes.c_float, ctypes.c_int, _T],
    "kd_attention_decode_noalloc": [_T, _T, _T, _T, ctypes.c_int, ctypes.c_float, ctypes.c_int, _T],
    "kd_attention_decode_paged": [_T, _T, _T, _T, _T, ctypes.c_int, ctypes.c_float, ctypes.c_int, _T],
}


EXTRA_SIGNATURES: dict = {}


def declare(name: str, argtypes: list) -> None:
    fn = getattr(_lib, name)
    fn.argtypes = argtypes
    fn.restype = ctypes.c_int


for _name, _args in _SIGNATURES.items():
    declare(_name, _args)


def last_error() -> str:
    buf = ctypes.create_string_buffer(1024)
    _lib.kd_last_error(buf, 1024)
    return buf.value.decode("utf-8", "replace")


def call(name: str, *args) -> None:
    """Calls a kd_* entry point and raises KandleCudaError on a non-zero status."""
    st = getattr(_lib, name)(*args)
    if st != 0:
        raise KandleCudaError(st, f"{name}: {last_error()}")


def raw():
    return _lib
