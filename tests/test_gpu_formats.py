"""GPU parity of the format twins (w8g64, w8g32, w4g32) of the quantizer and dequantizer: bit-exact
against the oracle and against fixtures the reference's own shader source produced
(gpu-kernels/metal/quant/affine_dequant.metal:60-135, 243-306), through the C ABI."""
import os

import numpy as np
import pytest
import torch

from vpipe_b200 import synth

from test_gpu_parity import bits16, bits32, dev, to_dev

pytestmark = pytest.mark.gpu

TWINS = ["twin_w8g64_bf16_n12_k256", "twin_w8g32_bf16_n12_k160", "twin_w4g32_bf16_n12_k160",
         "twin_w8g64_f16_n12_k128"]


@pytest.mark.parametrize("name", TWINS)
def test_twin_quantizer_and_dequantizer_on_reference_fixtures(vpq, golden_dir, name):
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    bits, group = int(g["bits"]), int(g["group"])
    w = to_dev(g["w_bits"], torch.bfloat16 if int(g["src_is_bf16"]) else torch.float16)
    codes, s, b = vpq.ops.quantize(w, clip=float(g["clip"]), bits=bits, group=group)
    assert np.array_equal(bits32(codes), g["codes"])
    assert np.array_equal(bits16(s), g["scales_f16"])
    assert np.array_equal(bits16(b), g["biases_f16"])
    if "deq_bf16" in g:
        got = vpq.ops.dequantize_any(to_dev(g["codes"]), to_dev(g["scales_bf16"], torch.bfloat16),
                                     to_dev(g["biases_bf16"], torch.bfloat16), bits, group)
        assert np.array_equal(bits16(got), g["deq_bf16"])


@pytest.mark.parametrize("bits,group", [(8, 64), (8, 32), (4, 32), (4, 64)])
@pytest.mark.parametrize("N,K,bf16,clip", [(33, 1024, True, 1.0), (7, 4096, True, 0.9), (130, 320, False, 1.0)])
def test_twin_quantize_then_dequantize_bit_exact_vs_oracle(vpq, oracle_mod, bits, group, N, K, bf16, clip):
    w = synth.weight_f32(N, K, synth.seed_for("twin", bits, group, N, K))
    wb = synth.f32_to_bf16_bits(w) if bf16 else w.astype(np.float16).view(np.uint16)
    wb[0, :group] = 0x8000 if bf16 else 0x8000        # a group of -0
    wb[1, :group] = wb[1, 0]                          # a constant group: scale 0
    want = oracle_mod.quant(wb, bits, group, bf16, clip)
    got = vpq.ops.quantize(to_dev(wb, torch.bfloat16 if bf16 else torch.float16), clip=clip, bits=bits, group=group)
    assert np.array_equal(bits32(got[0]), want[0])
    assert np.array_equal(bits16(got[1]), want[1])
    assert np.array_equal(bits16(got[2]), want[2])
    sb, bb = oracle_mod.f16_to_bf16(want[1]), oracle_mod.f16_to_bf16(want[2])
    deq = vpq.ops.dequantize_any(got[0], to_dev(sb, torch.bfloat16), to_dev(bb, torch.bfloat16), bits, group)
    assert np.array_equal(bits16(deq), oracle_mod.dequant_bf16_any(want[0], sb, bb, bits, group))


def test_twins_by_reference_names_and_dense_route(vpq, oracle_mod):
    """A w8 layer through the route the reference takes for formats without a fused kernel:
    dequantise once, multiply densely (affine_dequant.metal:100-106)."""
    ops = vpq.ops
    N, K, M = 96, 512, 8
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 8800))
    w = to_dev(wb, torch.bfloat16)
    codes = torch.empty((N, K // 4), dtype=torch.int32, device=dev())
    s = torch.empty((N, K // 64), dtype=torch.float16, device=dev())
    b = torch.empty_like(s)
    ops.dispatch(ops.function("affine_dequant_bf16", "affine_quant_w8_g64"), [w, codes, s, b], K=K, N=N, clip=1.0)
    want = oracle_mod.quant(wb, 8, 64)
    assert np.array_equal(bits32(codes), want[0]) and np.array_equal(bits16(s), want[1])
    sb, bb = ops.scales_to_bf16(s), ops.scales_to_bf16(b)
    deq = torch.empty((N, K), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_dequant_bf16", "affine_dequant_w8g64"), [codes, sb, bb, deq], K=K, N=N)
    assert np.array_equal(bits16(deq), oracle_mod.dequant_bf16_any(want[0], bits16(sb), bits16(bb), 8, 64))
    x = to_dev(synth.activations_bf16(M, K, 8801), torch.bfloat16)
    y = (x.float() @ deq.float().T)
    ref = x.float() @ w.float().T
    assert float((y - ref).norm() / ref.norm()) < 0.03      # w8 round-trip bound of the reference's tests
    # unknown width / group: refused, not guessed
    with pytest.raises(vpq.VpqError):
        ops.quantize(w, bits=2, group=64)


def _w8_reference(oracle_mod, codes, s_bf16, b_bf16, x_bits, mode="fast"):
    """fp32 dequantise-then-matmul oracle for w8 g64: deq = s * byte + b in f32 (affine_dequant.metal:88-92
    without the final rounding), then the oracle's matmul."""
    N, Kw = codes.shape
    q = codes.view(np.uint8).reshape(N, Kw * 4).astype(np.float32)
    s = np.repeat(synth.bf16_bits_to_f32(s_bf16), 64, axis=1)
    b = np.repeat(synth.bf16_bits_to_f32(b_bf16), 64, axis=1)
    return oracle_mod.matmul_f32(x_bits, (s * q + b).astype(np.float32), mode)


@pytest.mark.parametrize("K,N,M", [(4096, 4096, 1), (12288, 512, 1), (1024, 1024, 2), (3840, 40, 1), (64, 8, 1),
                                   (320, 33, 2), (1152, 8193, 1)])
def test_qmv_w8g64_matches_fp32_oracle(vpq, oracle_mod, K, N, M):
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, synth.seed_for("w8", K, N)))
    codes, s16, b16 = oracle_mod.quant(wb, 8, 64)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, synth.seed_for("w8x", K, N))
    y = vpq.ops.qmv_w8(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    assert y.shape == (M, N)
    assert vpq.ops.device_status() == 0
    e = oracle_mod.err_metrics(y.float().cpu().numpy(), _w8_reference(oracle_mod, codes, s, b, x))
    assert e["rel_l2"] < 1e-2 and e["max_rel_rms"] < 1e-2 and e["max_rel_1e2"] < 1e-2, e


def test_qmv_w8g64_f32_accuracy_and_name(vpq, oracle_mod):
    """Random bytes with large biases (cancellation): the result is the bf16 rounding of the f64
    reference up to one ulp nearly everywhere; and the entry is reachable by the reference's name."""
    N, K = 256, 2048
    rng = np.random.default_rng(9)
    codes = rng.integers(0, 2**32, (N, K // 4), dtype=np.uint32)
    s = synth.f32_to_bf16_bits((rng.random((N, K // 64)) * 0.001 + 0.0003).astype(np.float32))
    b = synth.f32_to_bf16_bits((rng.random((N, K // 64)) * 0.2 - 0.1).astype(np.float32))
    x = synth.activations_bf16(1, K, 91)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = vpq.ops.qmv_w8(*d)
    ref = _w8_reference(oracle_mod, codes, s, b, x, "f64")
    want = synth.f32_to_bf16_bits(ref.astype(np.float32))
    ulps = np.abs(bits16(y).astype(np.int64) - want.astype(np.int64))
    assert (ulps <= 1).mean() > 0.999
    y2 = torch.empty_like(y)
    vpq.ops.dispatch(vpq.ops.function("affine_qmv_bf16", "affine_qmv_w8g64"), list(d) + [y2], K=K, N=N)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("M,K,N", [(256, 512, 512), (130, 320, 95), (33, 128, 33), (2048, 4096, 1024), (512, 2560, 256)])
def test_qmm_w8g64(vpq, oracle_mod, M, K, N):
    """affine_qmm_steel_w8g64 (affine_qmm_steel.metal:1595-1675): against the fp32 oracle within the
    reference's GEMM bound, and against a dense f32 product of the bit-exact dequantised W."""
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, synth.seed_for("qmm8", M, K, N)))
    codes, s16, b16 = oracle_mod.quant(wb, 8, 64)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, synth.seed_for("qmm8x", M, K, N))
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = vpq.ops.qmm_w8(*d)
    assert y.shape == (M, N)
    assert vpq.ops.device_status() == 0
    e = oracle_mod.err_metrics(y.float().cpu().numpy(), _w8_reference(oracle_mod, codes, s, b, x))
    assert e["rel_l2"] < 3e-3 and e["max_rel_rms"] < 1e-2, e
    wd = vpq.ops.dequantize_any(d[0], d[1], d[2], 8, 64)
    assert np.array_equal(bits16(wd), oracle_mod.dequant_bf16_any(codes, s, b, 8, 64))
    ref = d[3].float() @ wd.float().t()
    assert float((y.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
    assert float((y.float() - ref).norm() / ref.norm()) < 3e-3


def test_qmm_w8g64_large_scales_take_the_exact_route(vpq, oracle_mod):
    """Scales at or above 2^-5 (and zero scales) cannot use the scaled-subnormal multiply: same result."""
    M, K, N = 256, 256, 128
    rng = np.random.default_rng(12)
    codes = rng.integers(0, 2**32, (N, K // 4), dtype=np.uint32)
    s = synth.f32_to_bf16_bits((rng.random((N, K // 64)) * 0.2).astype(np.float32))   # many above 2^-5
    s[0, :] = 0                                                                    # zero scale
    b = synth.f32_to_bf16_bits((rng.random((N, K // 64)) * 2 - 1).astype(np.float32))
    x = synth.activations_bf16(M, K, 13)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = vpq.ops.qmm_w8(*d)
    wd = vpq.ops.dequantize_any(d[0], d[1], d[2], 8, 64)
    ref = d[3].float() @ wd.float().t()
    assert float((y.float() - ref).norm() / ref.norm()) < 3e-3
    y2 = torch.empty_like(y)
    vpq.ops.dispatch(vpq.ops.function("affine_qmm_steel_bf16", "affine_qmm_steel_w8g64"), list(d) + [y2], K=K, N=N, M=M)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("bits", [4, 8])
def test_gemm_tile_dequant_is_bit_identical_to_the_dequantizer(vpq, oracle_mod, bits):
    """x = identity: y[m, n] = W_deq[n, m] with nothing to round, so the GEMM output IS the tile the
    kernel dequantised. Includes zero scales, scales >= 2^-5 (the plain route) and extreme pairs."""
    K, N = 256, 320
    rng = np.random.default_rng(20 + bits)
    codes = rng.integers(0, 2**32, (N, K * bits // 32), dtype=np.uint32)
    s = synth.f32_to_bf16_bits((rng.random((N, K // 64)) * (0.02 if bits == 4 else 0.002) + 0.0001).astype(np.float32))
    b = synth.f32_to_bf16_bits((rng.random((N, K // 64)) * 0.4 - 0.2).astype(np.float32))
    s[0, :], s[1, :], s[2, 0], s[3, 0] = 0, 0x3E00, 0x0080, 0x3D00      # zero, 0.125, smallest normal, 2^-5
    b[2, 0], b[4, 0] = 0x3F80, 0x8000
    x = synth.f32_to_bf16_bits(np.eye(K, dtype=np.float32))
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = (vpq.ops.qmm if bits == 4 else vpq.ops.qmm_w8)(*d)
    want = oracle_mod.dequant_bf16_any(codes, s, b, bits, 64)
    assert np.array_equal(bits16(y), want.T)


def _g32_reference(oracle_mod, codes, s_bf16, b_bf16, x_bits, mode="fast"):
    """fp32 dequantise-then-matmul oracle for w4 g32: deq = s * nibble + b in f32, group 32."""
    N, Kw = codes.shape
    K = Kw * 8
    q = np.zeros((N, K), np.float32)
    for i in range(8):
        q[:, i::8] = ((codes >> np.uint32(4 * i)) & np.uint32(0xF)).astype(np.float32)
    s = np.repeat(synth.bf16_bits_to_f32(s_bf16), 32, axis=1)
    b = np.repeat(synth.bf16_bits_to_f32(b_bf16), 32, axis=1)
    return oracle_mod.matmul_f32(x_bits, (s * q + b).astype(np.float32), mode)


@pytest.mark.parametrize("K,N,M", [(4096, 4096, 1), (4096, 1024, 2), (8192, 512, 3), (12288, 256, 2), (3840, 40, 1),
                                   (32, 8, 1), (96, 33, 2), (1152, 4099, 1)])
def test_qmv_w4g32_matches_fp32_oracle(vpq, oracle_mod, K, N, M):
    """affine_qmv_w4g32 (affine_qmv.metal:303-320): the quantizer's group-32 output through the GEMV,
    against the fp32 dequantise-then-matmul oracle and the bit-exact group-32 dequantizer."""
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, synth.seed_for("g32", K, N)))
    codes, s16, b16 = oracle_mod.quant(wb, 4, 32)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, synth.seed_for("g32x", K, N))
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = vpq.ops.qmv_g32(*d)
    assert y.shape == (M, N)
    assert vpq.ops.device_status() == 0
    e = oracle_mod.err_metrics(y.float().cpu().numpy(), _g32_reference(oracle_mod, codes, s, b, x))
    assert e["rel_l2"] < 1e-2 and e["max_rel_rms"] < 1e-2 and e["max_rel_1e2"] < 1e-2, e


def test_qmv_w4g32_f32_accuracy_and_name(vpq, oracle_mod):
    N, K = 256, 2048
    rng = np.random.default_rng(31)
    codes = rng.integers(0, 2**32, (N, K // 8), dtype=np.uint32)
    s = synth.f32_to_bf16_bits((rng.random((N, K // 32)) * 0.015 + 0.005).astype(np.float32))
    b = synth.f32_to_bf16_bits((rng.random((N, K // 32)) * 0.2 - 0.1).astype(np.float32))
    x = synth.activations_bf16(2, K, 32)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = vpq.ops.qmv_g32(*d)
    ref = _g32_reference(oracle_mod, codes, s, b, x, "f64")
    want = synth.f32_to_bf16_bits(ref.astype(np.float32))
    ulps = np.abs(bits16(y).astype(np.int64) - want.astype(np.int64))
    assert (ulps <= 1).mean() > 0.999
    y2 = torch.empty_like(y)
    vpq.ops.dispatch(vpq.ops.function("affine_qmv_bf16", "affine_qmv_w4g32"), list(d) + [y2], K=K, N=N, M=2)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("bits,act,M,K,N", [(4, "none", 300, 1024, 520), (4, "none", 2048, 4096, 1024),
                                            (8, "none", 512, 2048, 768), (4, "geglu", 260, 1024, 512)])
def test_qmm_group32_twins(vpq, oracle_mod, bits, act, M, K, N):
    """affine_qmm_steel_w4g32 / affine_qmm_steel_w8g32 / affine_qmm_geglu_w4g32
    (affine_qmm_steel.metal:618-639,1573-1593,1677-1697): the GEMM with two scales per 64-wide k block.
    Against a dense f32 product of the bit-exact dequantised W (rounded to bf16 as the kernel does)."""
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, synth.seed_for("g32", bits, M, K, N)))
    codes, s16, b16 = oracle_mod.quant(wb, bits, 32)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, synth.seed_for("g32x", bits, M, K, N))
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = vpq.ops.qmm_any(d[0], d[1], d[2], d[3], bits, 32, act)
    assert vpq.ops.device_status() == 0
    wd = vpq.ops.dequantize_any(d[0], d[1], d[2], bits, 32)
    assert np.array_equal(bits16(wd), oracle_mod.dequant_bf16_any(codes, s, b, bits, 32))
    ref = d[3].float() @ wd.float().t()
    if act == "geglu":
        ref = torch.from_numpy(synth.bf16_bits_to_f32(oracle_mod.fused_geglu(ref.cpu().numpy()))).to(ref.device)
        assert y.shape == (M, N // 2)
    assert float((y.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())
    assert float((y.float() - ref).norm() / ref.norm()) < 3e-3
    # by the reference's name
    name = {(4, "none"): "affine_qmm_steel_w4g32", (8, "none"): "affine_qmm_steel_w8g32",
            (4, "geglu"): "affine_qmm_geglu_w4g32"}[(bits, act)]
    y2 = torch.zeros_like(y)
    vpq.ops.dispatch(vpq.ops.function("affine_qmm_steel_bf16", name), [d[0], d[1], d[2], d[3], y2], K=K, N=N, M=M)
    assert torch.equal(y, y2)


def test_requant_w8_to_w4_bit_exact(vpq, oracle_mod, golden_dir):
    """affine_requant_w8_to_w4_g64 (affine_dequant.metal:135-189): the reference-built fixture, then
    larger random weights against the oracle; codes, scales and biases bit for bit; also by name."""
    g = dict(np.load(os.path.join(golden_dir, "requant_w8g64_bf16_n10_k320.npz")))
    cases = [(g["codes8"], g["scales8_bf16"], g["biases8_bf16"], (g["codes4"], g["scales4_bf16"], g["biases4_bf16"]))]
    for seed, (N, K) in enumerate([(257, 4096), (33, 64), (1000, 1024)]):
        rng = np.random.default_rng(700 + seed)
        w = (rng.standard_normal((N, K)) * 0.03).astype(np.float32)
        w[0, :64] = -0.5
        codes8, s, b = oracle_mod.quant(synth.f32_to_bf16_bits(w), 8, 64)
        s8, b8 = oracle_mod.f16_to_bf16(s), oracle_mod.f16_to_bf16(b)
        if seed == 1:
            s8[2, 0] ^= 0x8000          # a negative scale: min and max swap roles
        cases.append((codes8, s8, b8, oracle_mod.requant_w8_to_w4_g64(codes8, s8, b8)))
    for codes8, s8, b8, want in cases:
        d = (to_dev(codes8), to_dev(s8, torch.bfloat16), to_dev(b8, torch.bfloat16))
        c4, s4, b4 = vpq.ops.requant_w8_to_w4(*d)
        assert np.array_equal(c4.cpu().numpy().view(np.uint32), want[0])
        assert np.array_equal(bits16(s4), want[1])
        assert np.array_equal(bits16(b4), want[2])
        N, K = codes8.shape[0], codes8.shape[1] * 4
        c4b, s4b, b4b = torch.zeros_like(c4), torch.zeros_like(s4), torch.zeros_like(b4)
        vpq.ops.dispatch(vpq.ops.function("affine_dequant_bf16", "affine_requant_w8_to_w4_g64"),
                         [d[0], d[1], d[2], c4b, s4b, b4b], K=K, N=N)
        assert torch.equal(c4b, c4) and torch.equal(s4b, s4) and torch.equal(b4b, b4)


def test_dequant_w4g32_and_geglu_w8_by_name(vpq, oracle_mod, golden_dir):
    """affine_dequant_w4g32 (affine_dequant.metal:191-225) on the reference-built fixture; and
    affine_qmv_geglu_w8g64 by name against the descriptor call."""
    g = dict(np.load(os.path.join(golden_dir, "twin_w4g32_bf16_n12_k160.npz")))
    d = (to_dev(g["codes"]), to_dev(g["scales_bf16"], torch.bfloat16), to_dev(g["biases_bf16"], torch.bfloat16))
    N, K = g["codes"].shape[0], g["codes"].shape[1] * 8
    out = torch.zeros((N, K), dtype=torch.bfloat16, device=dev())
    vpq.ops.dispatch(vpq.ops.function("affine_dequant_bf16", "affine_dequant_w4g32"), [d[0], d[1], d[2], out], K=K, N=N)
    assert np.array_equal(bits16(out), g["deq_bf16"])
    K, N, M = 1024, 96, 2
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 7301))
    codes, s16, b16 = oracle_mod.quant(wb, 8, 64)
    x = synth.activations_bf16(M, K, 7302)
    d = (to_dev(codes), to_dev(oracle_mod.f16_to_bf16(s16), torch.bfloat16),
         to_dev(oracle_mod.f16_to_bf16(b16), torch.bfloat16), to_dev(x, torch.bfloat16))
    want = vpq.ops.qmv_w8_fused(*d, torch.zeros((M, N // 2), dtype=torch.bfloat16, device=dev()), {"epilogue": "geglu"})
    got = torch.zeros_like(want)
    vpq.ops.dispatch(vpq.ops.function("affine_qmv_bf16", "affine_qmv_geglu_w8g64"), {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: got},
                     K=K, N=N, M=M)
    assert torch.equal(got, want) and float(got.float().abs().max()) > 0


def _w8g32_reference(oracle_mod, codes, s_bf16, b_bf16, x_bits, mode="f64"):
    N, Kw = codes.shape
    q = codes.view(np.uint8).reshape(N, Kw * 4).astype(np.float32)
    s = np.repeat(synth.bf16_bits_to_f32(s_bf16), 32, axis=1)
    b = np.repeat(synth.bf16_bits_to_f32(b_bf16), 32, axis=1)
    return oracle_mod.matmul_f32(x_bits, (s * q + b).astype(np.float32), mode)


@pytest.mark.parametrize("K,N,M", [(4096, 4096, 1), (12288, 512, 1), (1024, 1024, 2), (2080, 40, 1), (32, 8, 1),
                                   (352, 33, 2), (1280, 4099, 1)])
def test_qmv_w8g32_matches_fp32_oracle(vpq, oracle_mod, K, N, M):
    """affine_qmv_w8g32 (affine_qmv.metal:3050-3066): the quantizer's 8-bit group-32 output through the
    GEMV, against the fp32 dequantise-then-matmul oracle; K values with and without whole 256-k spans
    (scale rows as TMA boxes or as plain loads), ragged N; by the reference's name; a fused store."""
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, synth.seed_for("w8g32", K, N)))
    codes, s16, b16 = oracle_mod.quant(wb, 8, 32)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, synth.seed_for("w8g32x", K, N))
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    vpq.ops.qmv_w8_fused(*d, y, {"epilogue": "none"}, kind="w8g32")
    assert not torch.isnan(y.float()).any()
    e = oracle_mod.err_metrics(y.float().cpu().numpy(), _w8g32_reference(oracle_mod, codes, s, b, x).astype(np.float32))
    assert e["rel_l2"] < 1e-2 and e["max_rel_rms"] < 1e-2, e
    y2 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    vpq.ops.dispatch(vpq.ops.function("affine_qmv_bf16", "affine_qmv_w8g32"), list(d) + [y2], K=K, N=N, M=M)
    assert torch.equal(y2, y)
    aux = to_dev(synth.activations_bf16(M, N, 7400 + N), torch.bfloat16)
    y3 = vpq.ops.qmv_w8_fused(*d, torch.zeros_like(y), {"epilogue": "add", "aux": aux}, kind="w8g32")
    assert torch.equal(y3, (y.float() + aux.float()).to(torch.bfloat16))
