"""Torch-tensor front end to the C ABI (device pointers pass straight through).

16-bit float tensors may be torch.bfloat16 / torch.float16 or raw int16/uint16
bit patterns; packed weights are int32 / uint32 [N, K/8].
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check, lib


def _ptr(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise ValueError("vpipe_b200.ops: tensors must live on a CUDA device (no CPU path)")
    if not t.is_contiguous():
        raise ValueError("vpipe_b200.ops: tensors must be contiguous")
    return t.data_ptr()


def _stream(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def quantize(w: torch.Tensor, clip: float = 1.0, stream=None, bits: int = 4, group: int = 64):
    """Dense [N,K] f16/bf16 -> (codes int32 [N,K*bits/32], scales f16, biases f16 [N,K/group])."""
    if w.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("quantize: w must be float16 or bfloat16")
    N, K = w.shape
    dev = w.device
    with torch.cuda.device(dev):
        codes = torch.empty((N, max(K * bits // 32, 1)), dtype=torch.int32, device=dev)
        s = torch.empty((N, max(K // group, 1)), dtype=torch.float16, device=dev)
        b = torch.empty_like(s)
        if (bits, group) == (4, 64):
            check(lib().vpq_affine_quant_w4_g64(_ptr(w), int(w.dtype == torch.bfloat16), _ptr(codes),
                                                _ptr(s), _ptr(b), K, N, clip, _stream(stream)))
        else:
            check(lib().vpq_affine_quant(_ptr(w), int(w.dtype == torch.bfloat16), _ptr(codes), _ptr(s), _ptr(b),
                                         K, N, bits, group, clip, _stream(stream)))
    return codes, s, b


def dequantize_any(codes, scales, biases, bits: int, group: int, out=None, stream=None) -> torch.Tensor:
    """Any of the format twins (bits 4 | 8, group 64 | 32) -> dense bf16 [N, K]."""
    N, Kw = codes.shape
    K = Kw * 32 // bits
    if out is None:
        out = torch.empty((N, K), dtype=torch.bfloat16, device=codes.device)
    with torch.cuda.device(codes.device):
        check(lib().vpq_affine_dequant_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(out), K, N, bits, group,
                                            _stream(stream)))
    return out


def requant_w8_to_w4(codes8, scales8, biases8, stream=None):
    """8-bit group-64 weights -> (codes int32 [N, K/8], scales bf16, biases bf16 [N, K/64]) at 4 bits
    (vpq_affine_requant_w8_to_w4_g64_bf16)."""
    N, Kw = codes8.shape
    K = Kw * 4
    dev = codes8.device
    codes4 = torch.empty((N, K // 8), dtype=torch.int32, device=dev)
    s4 = torch.empty((N, K // 64), dtype=torch.bfloat16, device=dev)
    b4 = torch.empty((N, K // 64), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        check(lib().vpq_affine_requant_w8_to_w4_g64_bf16(_ptr(codes8), _ptr(scales8), _ptr(biases8), _ptr(codes4),
                                                         _ptr(s4), _ptr(b4), K, N, _stream(stream)))
    return codes4, s4, b4


def narrow_f32_bf16(w: torch.Tensor, stream=None) -> torch.Tensor:
    out = torch.empty(w.shape, dtype=torch.bfloat16, device=w.device)
    with torch.cuda.device(w.device):
        check(lib().vpq_narrow_f32_bf16(_ptr(w), _ptr(out), w.numel(), _stream(stream)))
    return out


def scales_to_bf16(s_f16: torch.Tensor, stream=None) -> torch.Tensor:
    out = torch.empty(s_f16.shape, dtype=torch.bfloat16, device=s_f16.device)
    with torch.cuda.device(s_f16.device):
        check(lib().vpq_scales_f16_to_bf16(_ptr(s_f16), _ptr(out), s_f16.numel(), _stream(stream)))
    return out


def dequantize(codes, scales, biases, out=None, stream=None) -> torch.Tensor:
    N, Kw = codes.shape
    K = Kw * 8
    if out is None:
        out = torch.empty((N, K), dtype=torch.bfloat16, device=codes.device)
    with torch.cuda.device(codes.device):
        check(lib().vpq_affine_dequant_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(out),
                                                  K, N, _stream(stream)))
    return out


def qmv(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmv_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x),
                                              _ptr(out), K, N, M, _stream(stream)))
    return out


def qmv_g32(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    """GEMV over 4-bit group-32 weights, scales / biases [N, K/32] (vpq_affine_qmv_w4g32_bf16)."""
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmv_w4g32_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out),
                                              K, N, M, _stream(stream)))
    return out


def qmv_w8(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    """GEMV over 8-bit group-64 weights, codes int32 [N, K/4] (vpq_affine_qmv_w8g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * 4
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmv_w8g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out),
                                              K, N, M, _stream(stream)))
    return out


def moe_gate_w8(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    """out[m] = sigmoid(dequant(w[1, K]) . x[m]) for one 8-bit row (vpq_affine_moe_gate_w8g64_bf16)."""
    K = codes.numel() * 4
    M = x.numel() // K
    if out is None:
        out = torch.empty((M,), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_moe_gate_w8g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out), K, M,
                                                   _stream(stream)))
    return out


def qmv_w8_fused(codes, scales, biases, x, y, store, stream=None, kind="w8"):
    """A GEMV with a fused store through one descriptor; `store` as in qmv_set, `y` the (first) output
    tensor. kind "w8": 8-bit weights (vpq_affine_qmv_w8g64_bf16_fused); "batch": w4 g64 rows sharing one
    weight stream (vpq_affine_qmv_batch_w4g64_bf16_fused); "g32": w4 g32 (vpq_affine_qmv_w4g32_bf16_fused);
    "q40": w4 g32 scale-only, `biases` may be None (vpq_affine_qmv_w4g32_q40_bf16_fused); "w8g32": 8-bit weights
    in groups of 32 (vpq_affine_qmv_w8g32_bf16_fused)."""
    N, Kw = codes.shape
    K = Kw * (4 if kind in ("w8", "w8g32") else 8)
    d = _lib.LinearDesc()
    d.w, d.scales, d.x, d.y = _ptr(codes), _ptr(scales), _ptr(x), _ptr(y)
    d.biases = _ptr(biases) if biases is not None else None
    d.K, d.N, d.M = K, N, x.numel() // K
    d.epilogue = EPILOGUES[store["epilogue"]]
    if store.get("aux") is not None:
        d.aux = _ptr(store["aux"])
    if store.get("y3") is not None:
        d.y3 = _ptr(store["y3"])
    d.q_rows, d.k_rows = store.get("q_rows", 0), store.get("k_rows", 0)
    fn = {"w8": lib().vpq_affine_qmv_w8g64_bf16_fused, "w8g32": lib().vpq_affine_qmv_w8g32_bf16_fused,
          "batch": lib().vpq_affine_qmv_batch_w4g64_bf16_fused,
          "g32": lib().vpq_affine_qmv_w4g32_bf16_fused, "q40": lib().vpq_affine_qmv_w4g32_q40_bf16_fused}[kind]
    with torch.cuda.device(x.device):
        check(fn(C.byref(d), _stream(stream)))
    return y


def qmv_batch_rows(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    """x [M, K] with small M: the rows share one stream of the weights (vpq_affine_qmv_batch_w4g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmv_batch_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out),
                                                    K, N, M, _stream(stream)))
    return out


def qmv_add(codes, scales, biases, x, residual, out=None, stream=None) -> torch.Tensor:
    """y = bf16(bf16(x W^T) + residual) (vpq_affine_qmv_w4g64_bf16_add)."""
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmv_w4g64_bf16_add(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out),
                                                  K, N, M, _ptr(residual), _stream(stream)))
    return out


def qmv_swiglu(codes, scales, biases, x, out=None, stream=None, act="swiglu") -> torch.Tensor:
    """Rows of W interleaved gate / up: y[M, N/2] = silu(gate) * up (vpq_affine_qmv_swiglu_w4g64_bf16),
    or gelu_tanh(gate) * up with act="geglu" (vpq_affine_qmv_geglu_w4g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    fn = {"swiglu": lib().vpq_affine_qmv_swiglu_w4g64_bf16, "geglu": lib().vpq_affine_qmv_geglu_w4g64_bf16}[act]
    with torch.cuda.device(x.device):
        check(fn(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out), K, N, M, _stream(stream)))
    return out


def qmv_geglu(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    return qmv_swiglu(codes, scales, biases, x, out, stream, act="geglu")


def qmv_gelu_mul(codes, scales, biases, x, mul, out=None, stream=None) -> torch.Tensor:
    """y = bf16(gelu_tanh(bf16(x W^T)) * mul) (vpq_affine_qmv_gelu_mul_w4g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmv_gelu_mul_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x),
                                                       _ptr(out), K, N, M, _ptr(mul), _stream(stream)))
    return out


def qmv_qkv(codes, scales, biases, x, q_rows, k_rows, v_rows, stream=None):
    """W = q | k | v row-concatenated; returns (q, k, v) (vpq_affine_qmv_qkv_w4g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    assert q_rows + k_rows + v_rows == N
    outs = [torch.empty((M, r), dtype=torch.bfloat16, device=x.device) for r in (q_rows, k_rows, v_rows)]
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmv_qkv_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x),
                                                  _ptr(outs[0]), _ptr(outs[1]) if k_rows else None,
                                                  _ptr(outs[2]) if v_rows else None, K, q_rows, k_rows, v_rows,
                                                  M, _stream(stream)))
    return tuple(outs)


EPILOGUES = {"none": 0, "add": 1, "swiglu": 2, "qkv": 3, "geglu": 4, "gelu_mul": 5, "silu_mul": 6}


def qmv_set(problems):
    """Builds the host descriptor array for qmv_batch / QmvPlan from (codes, scales, biases, x, y)
    tuples; an optional sixth element is a dict describing a fused store and the other options:
    {"epilogue": "add", "aux": residual} | {"epilogue": "swiglu"} | {"epilogue": "geglu"} |
    {"epilogue": "gelu_mul", "aux": mul} | {"epilogue": "silu_mul", "aux": mul} |
    {"epilogue": "qkv", "aux": k_out, "y3": v_out, "q_rows": .., "k_rows": ..};
    "norm_w": weights [K] and "eps" (RMSNorm of x while it is staged); "depends": True (plans: this
    GEMV reads what earlier entries write); "expert": int32 device tensor [M] with "x_div" (codes is
    then [E, N, K/8]: row m uses slab expert[m] and reads x row m // x_div); "M": rows, when x holds
    fewer rows than the descriptor has (expert gather)."""
    arr = (_lib.LinearDesc * len(problems))()
    for d, prob in zip(arr, problems):
        codes, scales, biases, x, y = prob[:5]
        e = prob[5] if len(prob) > 5 and prob[5] else {}
        N, Kw = codes.shape[-2], codes.shape[-1]
        d.w, d.scales, d.biases, d.x, d.y = _ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(y)
        d.K, d.N, d.M = Kw * 8, N, e.get("M", x.numel() // (Kw * 8))
        d.epilogue = EPILOGUES[e.get("epilogue", "none")]
        if e.get("aux") is not None:
            d.aux = _ptr(e["aux"])
        if e.get("y3") is not None:
            d.y3 = _ptr(e["y3"])
        d.q_rows, d.k_rows = e.get("q_rows", 0), e.get("k_rows", 0)
        d.depends = 1 if e.get("depends") else 0
        if e.get("norm_w") is not None:
            d.norm_w = _ptr(e["norm_w"])
            d.eps = float(e.get("eps", 1e-6))
        if e.get("expert") is not None:
            d.expert = _ptr(e["expert"])
            d.experts = codes.shape[0]
            d.x_div = int(e.get("x_div", 1))
            d.expert_div = int(e.get("expert_div", 1))
        if e.get("row_map") is not None:      # sorted slots: live iff row_map[m] >= 0; "row_gather": x row = row_map[m]
            d.row_map = _ptr(e["row_map"])
            d.row_gather = 1 if e.get("row_gather") else 0
    return arr


def qmv_batch(descs, stream=None) -> None:
    check(lib().vpq_affine_qmv_w4g64_bf16_batch(descs, len(descs), _stream(stream)))


def qmv_set_noalloc(descs, stream=None) -> None:
    """One launch for a set of at most 64 independent GEMV rows, with no device allocation and no
    workspace (vpq_affine_qmv_w4g64_bf16_set_noalloc). Calls must not overlap on the GPU."""
    check(lib().vpq_affine_qmv_w4g64_bf16_set_noalloc(descs, len(descs), _stream(stream)))


class QmvPlan:
    """A list of independent GEMVs run as one launch (vpq_qmv_plan_*). Holds the device workspace."""

    def __init__(self, problems, stream=None, workspace=None):
        self.descs = qmv_set(problems)
        self._keep = problems            # the plan captures pointers: keep the tensors alive
        dev = problems[0][0].device
        n = lib().vpq_qmv_plan_bytes(self.descs, len(self.descs))
        if workspace is not None and workspace.numel() < n:
            raise ValueError(f"QmvPlan: workspace of {workspace.numel()} bytes, {n} needed")
        self.workspace = workspace if workspace is not None else torch.empty(n, dtype=torch.uint8, device=dev)
        self.handle = C.c_void_p()
        with torch.cuda.device(dev):
            check(lib().vpq_qmv_plan_create(self.descs, len(self.descs), self.workspace.data_ptr(), self.workspace.numel(),
                                            _stream(stream), C.byref(self.handle)))

    def run(self, stream=None) -> None:
        check(lib().vpq_qmv_plan_run(self.handle, _stream(stream)))

    def close(self) -> None:
        if self.handle:
            lib().vpq_qmv_plan_destroy(self.handle)
            self.handle = None


def qmm(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmm_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x),
                                              _ptr(out), K, N, M, _stream(stream)))
    return out


def qmm_qkv(codes, scales, biases, x, q_rows, k_rows, v_rows, outs=None, stream=None):
    """W = q | k | v row-concatenated, one GEMM, three outputs (vpq_affine_qmm_qkv_w4g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * 8
    M = x.numel() // K
    assert q_rows + k_rows + v_rows == N
    if outs is None:
        outs = [torch.empty((M, r), dtype=torch.bfloat16, device=x.device) for r in (q_rows, k_rows, v_rows)]
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmm_qkv_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(outs[0]),
                                                  _ptr(outs[1]), _ptr(outs[2]), K, q_rows, k_rows, v_rows, M,
                                                  _stream(stream)))
    return tuple(outs)


def qmm_any(codes, scales, biases, x, bits: int, group: int, act: str = "none", out=None, stream=None) -> torch.Tensor:
    """GEMM over any format twin (vpq_affine_qmm_bf16): bits 4 | 8, group 64 | 32, act "none" | "geglu"."""
    N, Kw = codes.shape
    K = Kw * (32 // bits)
    M = x.numel() // K
    a = {"none": 0, "geglu": 2}[act]
    if out is None:
        out = torch.empty((M, N // 2 if a else N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmm_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out), K, N, M, bits,
                                        group, a, _stream(stream)))
    return out


def qmm_w8(codes, scales, biases, x, out=None, stream=None) -> torch.Tensor:
    """GEMM over 8-bit group-64 weights, codes int32 [N, K/4] (vpq_affine_qmm_w8g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * 4
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmm_w8g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out),
                                              K, N, M, _stream(stream)))
    return out


def qmm_swiglu(codes, scales, biases, x, out=None, stream=None, act="swiglu", bits=4) -> torch.Tensor:
    """Rows of W interleaved gate / up: y[M, N/2] = act(gate) * up, act silu ("swiglu") or gelu_tanh
    ("geglu"), over 4- or 8-bit weights (vpq_affine_qmm_{swiglu,geglu}_w{4,8}g64_bf16)."""
    N, Kw = codes.shape
    K = Kw * (32 // bits)
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    fn = getattr(lib(), f"vpq_affine_qmm_{act}_w{bits}g64_bf16")
    with torch.cuda.device(x.device):
        check(fn(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out), K, N, M, _stream(stream)))
    return out


def qmm_swiglu_into(codes, scales, biases, x, out, out_off, bits=4, stream=None) -> torch.Tensor:
    """silu(gate) * up written into columns [out_off, out_off + N/2) of the row-major `out` [M, stride]
    (vpq_affine_qmm_swiglu_bf16_rs)."""
    N, Kw = codes.shape
    K = Kw * (32 // bits)
    M = x.numel() // K
    with torch.cuda.device(x.device):
        check(lib().vpq_affine_qmm_swiglu_bf16_rs(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out), K, N,
                                                  M, bits, out.shape[-1], out_off, _stream(stream)))
    return out


def qmm_grouped_tile_rows() -> int:
    return int(lib().vpq_qmm_grouped_tile_rows())


def qmm_grouped_gated(codes, scales, biases, x, tile2e, srow=None, act="swiglu", out=None, stream=None, bits=4):
    """Gate|up GEMM of a mixture of experts over sorted, padded rows: codes [E, N, K*bits/32]; x the hidden
    [T, K] with srow [M] (gathered), or already sorted [M, K] with srow None. Returns y [M, N/2] in
    sorted order (vpq_affine_qmm_grouped_{swiglu,geglu}_w4g64_bf16; bits=8: vpq_affine_qmm_grouped_w8g64_bf16)."""
    E, N, Kw = codes.shape
    K = Kw * 32 // bits
    M = int(srow.numel()) if srow is not None else x.numel() // K
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    scratch = torch.empty((M, K), dtype=torch.bfloat16, device=x.device) if srow is not None else None
    args = (_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x), _ptr(out), K, N, M, _ptr(tile2e),
            _ptr(srow) if srow is not None else None, E, x.numel() // K,
            _ptr(scratch) if scratch is not None else None, _stream(stream))
    with torch.cuda.device(x.device):
        if bits == 8:
            check(lib().vpq_affine_qmm_grouped_w8g64_bf16({"swiglu": 1, "geglu": 2}[act], *args))
        else:
            check(getattr(lib(), f"vpq_affine_qmm_grouped_{act}_w4g64_bf16")(*args))
    return out


def qmm_grouped_down(codes, scales, biases, x_sorted, tile2e, sdst=None, y_rows=0, out=None, stream=None, bits=4):
    """Down GEMM of a mixture of experts: x_sorted [M, K]; row m of the product lands in row sdst[m]
    of y [y_rows, N] (vpq_affine_qmm_grouped_w4g64_bf16; bits=8: vpq_affine_qmm_grouped_w8g64_bf16). Rows of y
    no slot points at are not written."""
    E, N, Kw = codes.shape
    K = Kw * 32 // bits
    M = x_sorted.numel() // K
    rows = y_rows if sdst is not None else M
    if out is None:
        out = torch.zeros((rows, N), dtype=torch.bfloat16, device=x_sorted.device)
    with torch.cuda.device(x_sorted.device):
        if bits == 8:
            check(lib().vpq_affine_qmm_grouped_w8g64_bf16(0, _ptr(codes), _ptr(scales), _ptr(biases), _ptr(x_sorted),
                                                          _ptr(out), K, N, M, _ptr(tile2e),
                                                          _ptr(sdst) if sdst is not None else None, E, rows, None,
                                                          _stream(stream)))
        else:
            check(lib().vpq_affine_qmm_grouped_w4g64_bf16(_ptr(codes), _ptr(scales), _ptr(biases), _ptr(x_sorted),
                                                          _ptr(out), K, N, M, _ptr(tile2e),
                                                          _ptr(sdst) if sdst is not None else None, E, rows,
                                                          _stream(stream)))
    return out


def device_status(stream=None) -> int:
    """Raises VpqError(TIMEOUT) if a bounded device-side wait gave up; else 0."""
    detail = C.c_uint32(0)
    check(lib().vpq_device_status(_stream(stream), C.byref(detail)))
    return int(detail.value)


def function(library: str, entry: str):
    """The reference's load_library(name).function(entry); None if unknown."""
    return lib().vpq_function_lookup(library.encode(), entry.encode())


def dispatch(fn, buffers, K=0, N=0, M=0, clip=1.0, q_rows=0, k_rows=0, v_rows=0, out_stride=0, out_off=0,
             experts=0, rows=0, top_k=0, eps=0.0, stream=None) -> None:
    """One dispatch with the reference's slot numbering (see include/vpq.h). `buffers` is a list
    indexed by slot, or a dict {slot: tensor}."""
    a = _lib.DispatchArgs()
    items = buffers.items() if isinstance(buffers, dict) else enumerate(buffers)
    for i, t in items:
        a.buffers[i] = _ptr(t) if t is not None else None
    a.K, a.N, a.M, a.clip = K, N, M, clip
    a.q_rows, a.k_rows, a.v_rows = q_rows, k_rows, v_rows
    a.out_stride, a.out_off, a.experts, a.rows = out_stride, out_off, experts, rows
    a.top_k, a.eps = top_k, eps
    check(lib().vpq_dispatch(fn, C.byref(a), _stream(stream)))
