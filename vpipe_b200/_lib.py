"""ctypes loader for libvpq.so (the C ABI in include/vpq.h)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "libvpq.so")
_lib = None

VPQ_OK = 0
UNIQUE_ID_BYTES = 128

# every symbol include/vpq.h declares: (name, restype, argtypes)
_vp, _i64, _i, _f = C.c_void_p, C.c_int64, C.c_int, C.c_float
SYMBOLS = [
    ("vpq_version", _i, []),
    ("vpq_status_string", C.c_char_p, [_i]),
    ("vpq_last_error", C.c_char_p, []),
    ("vpq_weight_bytes", C.c_size_t, [_i, _i, _i]),
    ("vpq_scale_bytes", C.c_size_t, [_i, _i, _i]),
    ("vpq_affine_quant_w4_g64", _i, [_vp, _i, _vp, _vp, _vp, _i64, _i64, _f, _vp]),
    ("vpq_narrow_f32_bf16", _i, [_vp, _vp, _i64, _vp]),
    ("vpq_scales_f16_to_bf16", _i, [_vp, _vp, _i64, _vp]),
    ("vpq_affine_dequant_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    ("vpq_affine_qmv_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_quant", _i, [_vp, _i, _vp, _vp, _vp, _i64, _i64, _i, _i, C.c_float, _vp]),
    ("vpq_affine_dequant_bf16", _i, [_vp, _vp, _vp, _vp, _i64, _i64, _i, _i, _vp]),
    ("vpq_affine_requant_w8_to_w4_g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    ("vpq_affine_qmm_swiglu_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmm_swiglu_bf16_rs", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _i64, _i64, _vp]),
    ("vpq_qmm_grouped_tile_rows", _i, []),
    ("vpq_affine_qmm_grouped_w4g64_bf16", _i,
     [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp]),
    ("vpq_affine_qmm_grouped_swiglu_w4g64_bf16", _i,
     [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _vp]),
    ("vpq_affine_qmm_grouped_geglu_w4g64_bf16", _i,
     [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _vp]),
    ("vpq_affine_qmm_grouped_w8g64_bf16", _i,
     [_i, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _vp, _vp]),
    ("vpq_affine_qmm_geglu_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmm_swiglu_w8g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmm_geglu_w8g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_geglu_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_gelu_mul_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    ("vpq_affine_qmm_qkv_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmm_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _i, _i, _vp]),
    ("vpq_affine_qmm_w8g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_w4g32_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_w8g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_batch_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_w4g64_bf16_add", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    ("vpq_affine_qmv_swiglu_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_qkv_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmv_w4g64_bf16_batch", _i, [_vp, _i, _vp]),
    ("vpq_affine_qmv_w8g64_bf16_fused", _i, [_vp, _vp]),
    ("vpq_affine_qmv_w8g32_bf16_fused", _i, [_vp, _vp]),
    ("vpq_affine_moe_gate_w8g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    ("vpq_affine_qmv_batch_w4g64_bf16_fused", _i, [_vp, _vp]),
    ("vpq_affine_qmv_w4g32_bf16_fused", _i, [_vp, _vp]),
    ("vpq_affine_qmv_w4g32_q40_bf16_fused", _i, [_vp, _vp]),
    ("vpq_affine_qmv_w4g64_bf16_set_noalloc", _i, [_vp, _i, _vp]),
    ("vpq_qmv_plan_bytes", C.c_size_t, [_vp, _i]),
    ("vpq_qmv_plan_create", _i, [_vp, _i, _vp, C.c_size_t, _vp, C.POINTER(_vp)]),
    ("vpq_qmv_plan_run", _i, [_vp, _vp]),
    ("vpq_qmv_plan_destroy", _i, [_vp]),
    ("vpq_affine_qmm_w4g64_bf16", _i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_device_status", _i, [_vp, C.POINTER(C.c_uint32)]),
    ("vpq_wait_probe", _i, [C.c_uint32, C.c_uint32, _vp]),
    ("vpq_peer_barrier_probe", _i, [_vp, _i, _i, C.c_uint32, _vp]),
    ("vpq_function_lookup", _vp, [C.c_char_p, C.c_char_p]),
    ("vpq_function_name", C.c_char_p, [_vp]),
    ("vpq_dispatch", _i, [_vp, _vp, _vp]),
    ("vpq_comm_unique_id", _i, [_vp]),
    ("vpq_comm_create", _i, [_vp, _i, _i, C.POINTER(_vp)]),
    ("vpq_comm_destroy", _i, [_vp]),
    ("vpq_comm_rank", _i, [_vp]),
    ("vpq_comm_world", _i, [_vp]),
    ("vpq_comm_alloc_symmetric", _i, [_vp, C.c_size_t, C.POINTER(_vp)]),
    ("vpq_comm_free_symmetric", _i, [_vp, _vp]),
    ("vpq_affine_qmm_w4g64_bf16_nsplit_fused", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    ("vpq_affine_qmm_w4g64_bf16_nsplit", _i,
     [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _vp]),
]


class DispatchArgs(C.Structure):
    """struct vpq_dispatch_args"""
    _fields_ = [("buffers", C.c_void_p * 12), ("K", C.c_int64), ("N", C.c_int64),
                ("M", C.c_int64), ("clip", C.c_float), ("q_rows", C.c_int64),
                ("k_rows", C.c_int64), ("v_rows", C.c_int64), ("out_stride", C.c_int64),
                ("out_off", C.c_int64), ("experts", C.c_int64), ("rows", C.c_int64),
                ("top_k", C.c_int64), ("eps", C.c_float)]


class LinearDesc(C.Structure):
    """struct vpq_linear_desc"""
    _fields_ = [("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
                ("x", C.c_void_p), ("y", C.c_void_p), ("K", C.c_int64), ("N", C.c_int64),
                ("M", C.c_int64), ("epilogue", C.c_int32), ("depends", C.c_int32),
                ("aux", C.c_void_p), ("y3", C.c_void_p), ("q_rows", C.c_int64),
                ("k_rows", C.c_int64), ("norm_w", C.c_void_p), ("expert", C.c_void_p),
                ("experts", C.c_int64), ("x_div", C.c_int32), ("eps", C.c_float),
                ("row_map", C.c_void_p), ("row_gather", C.c_int32), ("expert_div", C.c_int32)]


class VpqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"vpq status {status} ({status_string(status)}): {message}")
        self.status = status


def lib_path() -> str:
    return _PATH


def lib():
    """Loads libvpq.so; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            raise RuntimeError(
                f"{_PATH} is missing: build it with `python -m vpipe_b200.build`. "
                "vpipe_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(_PATH)
        for name, res, args in SYMBOLS:
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().vpq_status_string(int(status)).decode()


def check(status: int) -> None:
    if status != VPQ_OK:
        raise VpqError(status, lib().vpq_last_error().decode())
