"""CPU oracle for the 4-bit affine quantized linear -- TEST INFRASTRUCTURE ONLY.

numpy/ctypes front end to ``libvpq_oracle.so`` (the C restatement, see
``vpq_oracle.h`` for the reference file:line each function follows) and, when
it has been built, to ``_ref/libvpq_ref.so`` (the reference's own quantize /
dequantize shader source compiled as C++).

Only the tests, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this package, and only as
the checker or the timed CPU baseline. The shipped library never does.

16-bit float arrays are ``np.uint16`` bit patterns throughout.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libvpq_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libvpq_ref.so")

_lib = None
_ref = None


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference-source pin when the reference
    checkout is present) with oracle/Makefile."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE, "-s", "all"], check=True)
    else:
        # cheap: lets make decide whether the reference pin needs (re)building
        subprocess.run(["make", "-C", _HERE, "-s", "all"], check=False,
                       stdout=subprocess.DEVNULL)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        L.vpq_o_quant_w4_g64.restype = C.c_int
        L.vpq_o_quant_w4_g64.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int, C.c_int, C.c_float]
        L.vpq_o_quant.restype = C.c_int
        L.vpq_o_quant.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        L.vpq_o_dequant_bf16.restype = C.c_int
        L.vpq_o_dequant_bf16.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
        for name in ("vpq_o_dequant_w4g64_bf16", "vpq_o_dequant_w4g64_f32"):
            f = getattr(L, name)
            f.restype = None
            f.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_int]
        L.vpq_o_narrow_f32_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.vpq_o_narrow_f32_bf16.restype = None
        L.vpq_o_f16_to_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.vpq_o_f16_to_bf16.restype = None
        L.vpq_o_matmul_f32_seq.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3
        L.vpq_o_matmul_f32_seq.restype = None
        L.vpq_o_matmul_f64.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3
        L.vpq_o_matmul_f64.restype = None
        L.vpq_o_matmul_f32_fast.argtypes = [C.c_void_p] * 3 + [C.c_int] * 4
        L.vpq_o_matmul_f32_fast.restype = None
        L.vpq_o_qmv_kernel_order.argtypes = [C.c_void_p] * 5 + [C.c_int] * 3
        L.vpq_o_qmv_kernel_order.restype = None
        L.vpq_o_qmm_kernel_numerics.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4
        L.vpq_o_qmm_kernel_numerics.restype = None
        L.vpq_o_cpu_linear.argtypes = [C.c_void_p] * 6 + [C.c_int] * 4
        L.vpq_o_cpu_linear.restype = C.c_double
        L.vpq_o_max_threads.restype = C.c_int
        L.vpq_o_weight_bytes.restype = C.c_size_t
        L.vpq_o_weight_bytes.argtypes = [C.c_int] * 3
        L.vpq_o_scale_bytes.restype = C.c_size_t
        L.vpq_o_scale_bytes.argtypes = [C.c_int] * 3
        L.vpq_o_f32_to_f16.restype = C.c_uint16
        L.vpq_o_f32_to_f16.argtypes = [C.c_float]
        L.vpq_o_f16_to_f32.restype = C.c_float
        L.vpq_o_f16_to_f32.argtypes = [C.c_uint16]
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.exists(_REF_PATH)


def ref():
    """The reference's own shader source compiled as C++ (None if not built)."""
    global _ref
    if _ref is None and have_ref():
        R = C.CDLL(_REF_PATH)
        for sfx in ("f16", "bf16"):
            q = getattr(R, f"ref_affine_quant_w4_g64_{sfx}")
            q.restype = C.c_int
            q.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_int, C.c_float]
            d = getattr(R, f"ref_affine_dequant_w4g64_{sfx}")
            d.restype = C.c_int
            d.argtypes = [C.c_void_p] * 4 + [C.c_int, C.c_int]
            q = getattr(R, f"ref_affine_quant_{sfx}")
            q.restype = C.c_int
            q.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float]
            d = getattr(R, f"ref_affine_dequant_{sfx}")
            d.restype = C.c_int
            d.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4
            r = getattr(R, f"ref_affine_requant_w8_to_w4_g64_{sfx}")
            r.restype = C.c_int
            r.argtypes = [C.c_void_p] * 6 + [C.c_int] * 2
        _ref = R
    return _ref


# ------------------------------------------------------------------ helpers

def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def narrow_f32_bf16(w_f32: np.ndarray) -> np.ndarray:
    src = _c(w_f32, np.float32)
    out = np.empty(src.shape, np.uint16)
    lib().vpq_o_narrow_f32_bf16(_p(src), _p(out), src.size)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (_c(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f16_to_bf16(a: np.ndarray) -> np.ndarray:
    src = _c(a, np.uint16)
    out = np.empty(src.shape, np.uint16)
    lib().vpq_o_f16_to_bf16(_p(src), _p(out), src.size)
    return out


def quant_w4_g64(w_elt: np.ndarray, src_is_bf16: bool = True, clip: float = 1.0,
                 use_ref: bool = False):
    """[N,K] f16/bf16 bit patterns -> (codes u32 [N,K/8], scales f16, biases f16)."""
    w = _c(w_elt, np.uint16)
    N, K = w.shape
    codes = np.zeros((N, K // 8), np.uint32)
    s = np.zeros((N, K // 64), np.uint16)
    b = np.zeros((N, K // 64), np.uint16)
    if use_ref:
        fn = getattr(ref(), "ref_affine_quant_w4_g64_" + ("bf16" if src_is_bf16 else "f16"))
        rc = fn(_p(w), _p(codes), _p(s), _p(b), K, N, clip)
    else:
        rc = lib().vpq_o_quant_w4_g64(_p(w), int(src_is_bf16), _p(codes), _p(s), _p(b),
                                      K, N, clip)
    if rc != 0:
        raise ValueError("quant_w4_g64: bad arguments")
    return codes, s, b


def dequant_bf16(codes, s_bf16, b_bf16, use_ref: bool = False) -> np.ndarray:
    codes = _c(codes, np.uint32)
    N, Kw = codes.shape
    K = Kw * 8
    s = _c(s_bf16, np.uint16)
    b = _c(b_bf16, np.uint16)
    out = np.empty((N, K), np.uint16)
    if use_ref:
        ref().ref_affine_dequant_w4g64_bf16(_p(codes), _p(s), _p(b), _p(out), K, N)
    else:
        lib().vpq_o_dequant_w4g64_bf16(_p(codes), _p(s), _p(b), _p(out), K, N)
    return out


def quant(w_elt: np.ndarray, bits: int, group: int, src_is_bf16: bool = True, clip: float = 1.0,
          use_ref: bool = False):
    """Any (bits, group) of the reference's quantizer template (4|8, 64|32):
    [N,K] f16/bf16 bit patterns -> (codes u32 [N,K*bits/32], scales f16, biases f16 [N,K/group])."""
    w = _c(w_elt, np.uint16)
    N, K = w.shape
    codes = np.zeros((N, K * bits // 32), np.uint32)
    s = np.zeros((N, K // group), np.uint16)
    b = np.zeros((N, K // group), np.uint16)
    if use_ref:
        fn = getattr(ref(), "ref_affine_quant_" + ("bf16" if src_is_bf16 else "f16"))
        rc = fn(_p(w), _p(codes), _p(s), _p(b), K, N, bits, group, clip)
    else:
        rc = lib().vpq_o_quant(_p(w), int(src_is_bf16), _p(codes), _p(s), _p(b), K, N, bits, group, clip)
    if rc != 0:
        raise ValueError("quant: bad arguments")
    return codes, s, b


def dequant_bf16_any(codes, s_bf16, b_bf16, bits: int, group: int, use_ref: bool = False) -> np.ndarray:
    """Dequantizer for any (bits, group): affine_dequant_w4g64 / _w8g64 / _w8g32 / _w4g32
    (gpu-kernels/metal/quant/affine_dequant.metal:25-135,191-225)."""
    codes = _c(codes, np.uint32)
    N, Kw = codes.shape
    K = Kw * 32 // bits
    out = np.empty((N, K), np.uint16)
    args = (_p(codes), _p(_c(s_bf16, np.uint16)), _p(_c(b_bf16, np.uint16)), _p(out), K, N, bits, group)
    rc = ref().ref_affine_dequant_bf16(*args) if use_ref else lib().vpq_o_dequant_bf16(*args)
    if rc != 0:
        raise ValueError("dequant_bf16_any: bad arguments")
    return out


def requant_w8_to_w4_g64(codes8, s8_bf16, b8_bf16, use_ref: bool = False):
    """affine_requant_w8_to_w4_g64 (gpu-kernels/metal/quant/affine_dequant.metal:135-189), bf16 build:
    per group of 64, v = s8 * q8 + b8 in f32 (the product of an 8-bit significand and an 8-bit code is
    exact, so fused or not is the same value), scale = (max - min) / 15, inv = scale > 0 ? 1 / scale : 0,
    q4 = clamp(round((v - min) * inv), 0, 15) with round() halves away from zero; the stored scale and
    bias are scale and min narrowed to bf16. Returns (codes4 u32 [N, K/8], s4, b4 bf16 bits [N, K/64])."""
    codes8 = _c(codes8, np.uint32)
    N, Kw = codes8.shape
    K = Kw * 4
    G = K // 64
    if use_ref:
        w4 = np.zeros((N, K // 8), np.uint32)
        s4 = np.zeros((N, G), np.uint16)
        b4 = np.zeros((N, G), np.uint16)
        rc = ref().ref_affine_requant_w8_to_w4_g64_bf16(_p(codes8), _p(_c(s8_bf16, np.uint16)), _p(_c(b8_bf16, np.uint16)),
                                                        _p(w4), _p(s4), _p(b4), K, N)
        if rc != 0:
            raise ValueError("requant_w8_to_w4_g64: bad arguments")
        return w4, s4, b4
    q8 = ((codes8[:, :, None] >> (np.arange(4, dtype=np.uint32) * 8)) & np.uint32(0xFF)).reshape(N, G, 64).astype(np.float32)
    s = bf16_to_f32(s8_bf16).reshape(N, G, 1)
    b = bf16_to_f32(b8_bf16).reshape(N, G, 1)
    v = (s * q8 + b).astype(np.float32)           # s * q8 is exact in f32: one rounding, on the add
    mn = v.min(axis=2, keepdims=True)
    mx = v.max(axis=2, keepdims=True)
    scale = ((mx - mn).astype(np.float32) / np.float32(15.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(scale > 0, np.float32(1.0) / scale, np.float32(0.0)).astype(np.float32)
    t = ((v - mn).astype(np.float32) * inv).astype(np.float32)
    q4 = np.clip(np.floor(t.astype(np.float64) + 0.5), 0, 15).astype(np.uint32).reshape(N, K // 8, 8)
    w4 = np.zeros((N, K // 8), np.uint32)
    for i in range(8):
        w4 |= q4[:, :, i] << np.uint32(4 * i)
    return w4, narrow_f32_bf16(scale.reshape(N, G)), narrow_f32_bf16(mn.reshape(N, G))


def dequant_f16_ref(codes, s_f16, b_f16) -> np.ndarray:
    """Reference-source dequant in its f16 build (scales/biases/output f16)."""
    codes = _c(codes, np.uint32)
    N, Kw = codes.shape
    out = np.empty((N, Kw * 8), np.uint16)
    ref().ref_affine_dequant_w4g64_f16(_p(codes), _p(_c(s_f16, np.uint16)),
                                       _p(_c(b_f16, np.uint16)), _p(out), Kw * 8, N)
    return out


def dequant_f32(codes, s_bf16, b_bf16) -> np.ndarray:
    codes = _c(codes, np.uint32)
    N, Kw = codes.shape
    K = Kw * 8
    out = np.empty((N, K), np.float32)
    lib().vpq_o_dequant_w4g64_f32(_p(codes), _p(_c(s_bf16, np.uint16)),
                                  _p(_c(b_bf16, np.uint16)), _p(out), K, N)
    return out


def matmul_f32(x_bf16, deq, mode: str = "fast", threads: int = 0) -> np.ndarray:
    """fp32 dequantise-then-matmul reference: y[m,n] = sum_k x[m,k]*deq[n,k]."""
    x = _c(x_bf16, np.uint16)
    d = _c(deq, np.float32)
    M, K = x.shape
    N = d.shape[0]
    assert d.shape[1] == K
    if mode == "f64":
        y = np.empty((M, N), np.float64)
        lib().vpq_o_matmul_f64(_p(x), _p(d), _p(y), M, N, K)
        return y
    y = np.empty((M, N), np.float32)
    if mode == "seq":
        lib().vpq_o_matmul_f32_seq(_p(x), _p(d), _p(y), M, N, K)
    else:
        lib().vpq_o_matmul_f32_fast(_p(x), _p(d), _p(y), M, N, K, threads)
    return y


def linear_f32(codes, s_bf16, b_bf16, x_bf16, mode: str = "fast") -> np.ndarray:
    return matmul_f32(x_bf16, dequant_f32(codes, s_bf16, b_bf16), mode)


def rms_norm_bf16(x_bf16: np.ndarray, norm_w_bf16: np.ndarray, eps: float) -> np.ndarray:
    """RMSNorm prologue of the fused norm + q|k|v GEMV, per row of x: sum of squares in f32,
    `inv = rsqrt(total / K + eps)`, `tg_x[k] = T(float(x[k]) * inv * float(norm_w[k]))`
    (gpu-kernels/metal/quant/affine_qmv.metal:601-621). Returns bf16 bit patterns. The f32 sum is
    taken in double here and rounded once, so a kernel's summation order shows as at most one ulp
    of `inv`."""
    x = bf16_to_f32(np.ascontiguousarray(x_bf16, np.uint16))
    w = bf16_to_f32(np.ascontiguousarray(norm_w_bf16, np.uint16)).reshape(1, -1)
    x = x.reshape(-1, w.shape[1])
    total = (x.astype(np.float64) ** 2).sum(axis=1, keepdims=True).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt(total / np.float32(x.shape[1]) + np.float32(eps))).astype(np.float32)
    y = (x * inv).astype(np.float32) * w
    u = y.astype(np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def fused_add(y_f32: np.ndarray, residual_bf16: np.ndarray) -> np.ndarray:
    """Residual store of the fused GEMV: the sum is rounded to bf16, the add happens in bf16
    (`T v = static_cast<T>(result[row]); if (ADD) v += residual[row];`,
    gpu-kernels/metal/quant/affine_qmv.metal:268-270). Returns bf16 bits."""
    y = bf16_to_f32(narrow_f32_bf16(np.asarray(y_f32, np.float32)))
    return narrow_f32_bf16((y + bf16_to_f32(residual_bf16)).astype(np.float32))


def fused_swiglu(y_f32: np.ndarray) -> np.ndarray:
    """SwiGLU store over row-interleaved gate | up (column 2j = gate j, 2j+1 = up j of y[M, N]):
    `(g / (1 + exp(-g))) * u` in f32 from the unrounded sums, rounded once
    (gpu-kernels/metal/quant/affine_qmv.metal:881-887). Returns bf16 bits [M, N/2]."""
    y = np.asarray(y_f32, np.float32)
    g, u = y[:, 0::2], y[:, 1::2]
    one = np.float32(1.0)
    return narrow_f32_bf16(((g / (one + np.exp(-g))) * u).astype(np.float32))


def gelu_tanh_f32(x: np.ndarray) -> np.ndarray:
    """gelu_pytorch_tanh in f32: `0.5 x (1 + tanh(k0 (x + 0.044715 x^3)))`, k0 = sqrt(2 / pi)
    (gpu-kernels/metal/ops/llm_elementwise.metal:388-407)."""
    x = np.asarray(x, np.float32)
    k0, c = np.float32(0.7978845608028654), np.float32(0.044715)
    t = np.tanh((k0 * (x + c * x * x * x)).astype(np.float32)).astype(np.float32)
    return (np.float32(0.5) * x * (np.float32(1.0) + t)).astype(np.float32)


def fused_geglu(y_f32: np.ndarray) -> np.ndarray:
    """GeGLU store over row-interleaved gate | up: gelu_tanh(g) * u in f32 from the unrounded sums,
    rounded once (gpu-kernels/metal/quant/affine_qmv.metal:1421-1429,
    quant/affine_qmm_steel.metal:1535-1545). Returns bf16 bits [M, N/2]."""
    y = np.asarray(y_f32, np.float32)
    return narrow_f32_bf16((gelu_tanh_f32(y[:, 0::2]) * y[:, 1::2]).astype(np.float32))


def fused_gelu_mul(y_f32: np.ndarray, mul_bf16: np.ndarray) -> np.ndarray:
    """Per-layer-input gate store: gelu_tanh of the bf16-rounded sum, times `mul`, rounded once
    (gpu-kernels/metal/quant/affine_qmv.metal:271-282). Returns bf16 bits."""
    y = bf16_to_f32(narrow_f32_bf16(np.asarray(y_f32, np.float32)))
    return narrow_f32_bf16((gelu_tanh_f32(y) * bf16_to_f32(mul_bf16)).astype(np.float32))


def qmv_kernel_order(codes, s_bf16, b_bf16, x_bf16) -> np.ndarray:
    codes = _c(codes, np.uint32)
    x = _c(x_bf16, np.uint16)
    N, Kw = codes.shape
    M, K = x.shape
    y = np.empty((M, N), np.uint16)
    lib().vpq_o_qmv_kernel_order(_p(codes), _p(_c(s_bf16, np.uint16)),
                                 _p(_c(b_bf16, np.uint16)), _p(x), _p(y), K, N, M)
    return y


def qmm_kernel_numerics(codes, s_bf16, b_bf16, x_bf16, threads: int = 0) -> np.ndarray:
    codes = _c(codes, np.uint32)
    x = _c(x_bf16, np.uint16)
    N, Kw = codes.shape
    M, K = x.shape
    y = np.empty((M, N), np.uint16)
    lib().vpq_o_qmm_kernel_numerics(_p(codes), _p(_c(s_bf16, np.uint16)),
                                    _p(_c(b_bf16, np.uint16)), _p(x), _p(y), K, N, M,
                                    threads)
    return y


def cpu_linear_seconds(codes, s_bf16, b_bf16, x_bf16, threads: int = 0):
    """Timed CPU baseline: returns (seconds, y_bf16)."""
    codes = _c(codes, np.uint32)
    x = _c(x_bf16, np.uint16)
    N, Kw = codes.shape
    M, K = x.shape
    y = np.empty((M, N), np.uint16)
    scratch = np.empty((N, K), np.float32)
    t = lib().vpq_o_cpu_linear(_p(codes), _p(_c(s_bf16, np.uint16)),
                               _p(_c(b_bf16, np.uint16)), _p(x), _p(y), _p(scratch),
                               K, N, M, threads)
    return float(t), y


def max_threads() -> int:
    return int(lib().vpq_o_max_threads())


# ------------------------------------------------------------ error metrics

def err_metrics(got_f32: np.ndarray, ref_f32: np.ndarray) -> dict:
    """The reference tests' own error forms plus the RMS-floored max.

    rel_l2          tests/unit-tests/metal-compute-gemm-mma.cc:478-485
    max_rel_1e2     max |d| / (|ref| + 1e-2), tests/unit-tests/metal-lm/quant-gemv.cc:293-294
    max_rel_rms     max |d| / (|ref| + rms(ref)): relative error with the
                    denominator floored at the tensor's own scale
    """
    g = np.asarray(got_f32, np.float64).ravel()
    r = np.asarray(ref_f32, np.float64).ravel()
    d = np.abs(g - r)
    den = float(np.sqrt(np.sum(r * r)))
    rms = float(np.sqrt(np.mean(r * r))) if r.size else 0.0
    return {
        "rel_l2": float(np.sqrt(np.sum(d * d)) / den) if den > 0 else float(np.sqrt(np.sum(d * d))),
        "max_rel_1e2": float(np.max(d / (np.abs(r) + 1e-2))) if r.size else 0.0,
        "max_rel_rms": float(np.max(d / (np.abs(r) + max(rms, 1e-30)))) if r.size else 0.0,
        "max_abs": float(np.max(d)) if r.size else 0.0,
        "rms_ref": rms,
    }
