"""GPU parity tests: every call goes through the C ABI (libvpq.so) and is
checked against the CPU oracle on the same seeded inputs.

Bars: quantize / convert / dequantize are bit-exact. QMV / QMM outputs (bf16
out, f32 accumulate) are compared with the fp32 dequantise-then-matmul
reference; the tolerance is 1e-2 on
    rel_l2       = |d|_2 / |ref|_2                      (reference QMM tests)
    max_rel_rms  = max |d| / (|ref| + rms(ref))         (max relative error with the
                                                         denominator floored at the tensor scale)
and, for QMV, also on the reference's own form max |d| / (|ref| + 1e-2).
"""
import os

import numpy as np
import pytest
import torch

from vpipe_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 1e-2


def dev():
    return torch.device("cuda", 0)


def to_dev(a: np.ndarray, dtype=None):
    """numpy bit patterns -> device tensor (uint16 travels as int16 and is re-viewed)."""
    if a.dtype == np.uint16:
        t = torch.from_numpy(a.view(np.int16)).to(dev())
        return t.view(dtype) if dtype is not None else t
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(dev())
    return torch.from_numpy(a).to(dev())


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def bits32(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int32).cpu().numpy().view(np.uint32)


def f32(t: torch.Tensor) -> np.ndarray:
    return t.float().cpu().numpy()


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(vpq):
    assert torch.cuda.is_available(), "the -m gpu tests need a CUDA device"
    assert torch.cuda.get_device_capability(0)[0] == 10, "the kernels are sm_100a only"
    torch.cuda.set_device(0)
    yield
    torch.cuda.synchronize()
    assert vpq.ops.device_status() == 0


# ------------------------------------------------------------------ quantizer

@pytest.mark.parametrize("name", ["quant_bf16_n24_k256", "quant_bf16_n8_k4096", "quant_f16_n16_k192",
                                  "quant_bf16_clip09_n16_k128"])
def test_quantizer_bit_exact_on_reference_fixtures(vpq, golden_dir, name):
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    dt = torch.bfloat16 if int(g["src_is_bf16"]) else torch.float16
    codes, s, b = vpq.ops.quantize(to_dev(g["w_bits"], dt), float(g["clip"]))
    assert np.array_equal(bits32(codes), g["codes"])
    assert np.array_equal(bits16(s), g["scales_f16"])
    assert np.array_equal(bits16(b), g["biases_f16"])


@pytest.mark.parametrize("N,K,bf16,clip", [(512, 4096, True, 1.0), (1000, 704, False, 1.0),
                                           (3, 64, True, 1.0), (257, 1024, True, 0.85),
                                           (1, 12288, True, 1.0)])
def test_quantizer_bit_exact_vs_oracle(vpq, oracle_mod, N, K, bf16, clip):
    w = synth.weight_f32(N, K, synth.seed_for("q", N, K))
    bits = synth.f32_to_bf16_bits(w) if bf16 else w.astype(np.float16).view(np.uint16)
    bits[0, :64] = 0x8000 if N > 1 else bits[0, :64]   # a group of -0
    want = oracle_mod.quant_w4_g64(bits, bf16, clip)
    got = vpq.ops.quantize(to_dev(bits, torch.bfloat16 if bf16 else torch.float16), clip)
    assert np.array_equal(bits32(got[0]), want[0])
    assert np.array_equal(bits16(got[1]), want[1])
    assert np.array_equal(bits16(got[2]), want[2])


def test_narrow_and_scale_conversion_bit_exact(vpq, oracle_mod):
    f = (np.random.default_rng(3).standard_normal(1 << 20) *
         10.0 ** np.random.default_rng(4).integers(-8, 8, 1 << 20)).astype(np.float32)
    got = vpq.ops.narrow_f32_bf16(torch.from_numpy(f).to(dev()))
    assert np.array_equal(bits16(got), oracle_mod.narrow_f32_bf16(f))
    # lengths that are no multiple of the kernel's 8-value step, and a source that is not 16-byte aligned
    fd = torch.from_numpy(f).to(dev())
    for n, off in ((1, 0), (7, 0), (8, 0), (4099, 0), (4099, 1), (65537, 3)):
        got = vpq.ops.narrow_f32_bf16(fd[off:off + n])
        assert np.array_equal(bits16(got), oracle_mod.narrow_f32_bf16(f[off:off + n])), (n, off)
    h = np.arange(65536, dtype=np.uint16)
    h = h[np.isfinite(h.view(np.float16))]
    got = vpq.ops.scales_to_bf16(to_dev(h, torch.float16))
    assert np.array_equal(bits16(got), oracle_mod.f16_to_bf16(h))


# ---------------------------------------------------------------- dequantizer

def test_dequant_bit_exact_on_reference_fixtures(vpq, golden_dir):
    for name in ["dequant_bf16_n33_k320", "quant_bf16_n24_k256", "quant_bf16_n8_k4096"]:
        g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
        got = vpq.ops.dequantize(to_dev(g["codes"]), to_dev(g["scales_bf16"], torch.bfloat16),
                                 to_dev(g["biases_bf16"], torch.bfloat16))
        assert np.array_equal(bits16(got), g["deq_bf16"]), name


@pytest.mark.parametrize("N,K", [(1024, 4096), (1, 64), (77, 832), (4096, 1024)])
def test_dequant_bit_exact_vs_oracle(vpq, oracle_mod, N, K):
    codes, s, b = synth.random_qweight(N, K, synth.seed_for("d", N, K))
    got = vpq.ops.dequantize(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16))
    assert np.array_equal(bits16(got), oracle_mod.dequant_bf16(codes, s, b))


def test_quantize_load_dequant_pipeline_equals_oracle(vpq, oracle_mod):
    """write -> read -> dequant byte-identical (tests/unit-tests/model-quantize-roundtrip.cc:84-164)."""
    N, K = 256, 2048
    bits = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 77))
    codes, s16, b16 = vpq.ops.quantize(to_dev(bits, torch.bfloat16))
    s, b = vpq.ops.scales_to_bf16(s16), vpq.ops.scales_to_bf16(b16)
    deq = vpq.ops.dequantize(codes, s, b)
    oc, os_, ob = oracle_mod.quant_w4_g64(bits, True)
    want = oracle_mod.dequant_bf16(oc, oracle_mod.f16_to_bf16(os_), oracle_mod.f16_to_bf16(ob))
    assert np.array_equal(bits16(deq), want)
    src = synth.bf16_bits_to_f32(bits)
    rel = np.linalg.norm(synth.bf16_bits_to_f32(want) - src) / np.linalg.norm(src)
    assert rel < 0.20


# ------------------------------------------------------------------------ QMV

def quantized_linear(oracle_mod, N, K, seed):
    """N(0,0.02) weights through the reference recipe: bf16 -> w4g64 -> F16 -> bf16."""
    bits = synth.f32_to_bf16_bits(synth.weight_f32(N, K, seed))
    codes, s, b = oracle_mod.quant_w4_g64(bits, True)
    return codes, oracle_mod.f16_to_bf16(s), oracle_mod.f16_to_bf16(b)


def check_linear(oracle_mod, y, codes, s, b, x, also_1e2=False, rows=None):
    deq = oracle_mod.dequant_f32(codes, s, b)
    xs = x if rows is None else x[rows]
    ref = oracle_mod.matmul_f32(xs, deq, "fast")
    got = f32(y) if rows is None else f32(y)[rows]
    e = oracle_mod.err_metrics(got, ref)
    assert e["rel_l2"] < TOL, e
    assert e["max_rel_rms"] < TOL, e
    if also_1e2:
        assert e["max_rel_1e2"] < TOL, e
    return e


QMV_SHAPES = [("C1", 4096, 4096, 1), ("C2.k", 4096, 1024, 1), ("C2.gate", 4096, 12288, 1),
              ("C2.down", 12288, 4096, 1), ("tail-k", 3840, 16, 1), ("one-group", 64, 8, 1),
              ("ragged-n", 320, 33, 1), ("n1", 1024, 1, 1), ("n7-m3", 2048, 7, 3),
              ("odd-steps", 5120, 2050, 2), ("n8193", 1088, 8193, 1)]


@pytest.mark.parametrize("tag,K,N,M", QMV_SHAPES)
def test_qmv_matches_fp32_oracle(vpq, oracle_mod, tag, K, N, M):
    codes, s, b = quantized_linear(oracle_mod, N, K, synth.seed_for("qmv-w", tag))
    x = synth.activations_bf16(M, K, synth.seed_for("qmv-x", tag))
    y = vpq.ops.qmv(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16),
                    to_dev(x, torch.bfloat16))
    assert y.shape == (M, N)
    check_linear(oracle_mod, y, codes, s, b, x, also_1e2=True)


def test_qmv_reference_test_distribution_and_f32_accuracy(vpq, oracle_mod):
    """Random nibbles with large biases (strong cancellation between s*sum(xq) and b*sum(x)):
    before the bf16 store the kernel must carry f32 noise only, so the result equals the
    bf16 rounding of the f64 reference up to one ulp nearly everywhere."""
    N, K = 512, 4096
    codes, s, b = synth.random_qweight(N, K, 41)
    x = synth.activations_bf16(1, K, 42)
    y = vpq.ops.qmv(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16),
                    to_dev(x, torch.bfloat16))
    ref = oracle_mod.linear_f32(codes, s, b, x, "f64")
    want = synth.f32_to_bf16_bits(ref.astype(np.float32))
    ulps = np.abs(bits16(y).astype(np.int64) - want.astype(np.int64))
    assert (ulps <= 1).mean() > 0.999
    assert oracle_mod.err_metrics(f32(y), ref)["max_rel_1e2"] < TOL


def test_qmv_does_not_touch_memory_past_its_buffers(vpq, oracle_mod):
    """Exact-size buffers between canaries (tests/unit-tests/metal-lm/quant-gemv.cc:215-222)."""
    K, N = 1088, 35
    codes, s, b = quantized_linear(oracle_mod, N, K, 51)
    x = synth.activations_bf16(1, K, 52)
    pad = 256
    ybuf = torch.full((pad + N + pad,), -7.0, dtype=torch.bfloat16, device=dev())
    y = ybuf[pad:pad + N].view(1, N)   # 512-byte offset keeps it 16-byte aligned
    vpq.ops.qmv(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16),
                to_dev(x, torch.bfloat16), out=y)
    assert torch.all(ybuf[:pad] == -7.0) and torch.all(ybuf[pad + N:] == -7.0)
    check_linear(oracle_mod, y, codes, s, b, x)


# ------------------------------------------------------------------------ QMM

# the reference's own QMM test shapes (tests/unit-tests/metal-compute-gemm-mma.cc:312-498)
QMM_REF_SHAPES = [(64, 64, 64), (96, 128, 128), (130, 320, 256), (512, 256, 2560),
                  (33, 33, 128), (64, 95, 192), (96, 161, 256)]


@pytest.mark.parametrize("M,N,K", QMM_REF_SHAPES)
def test_qmm_reference_test_shapes(vpq, oracle_mod, M, N, K):
    codes, s, b = synth.random_qweight(N, K, 999 + N + K)
    x = synth.activations_bf16(M, K, 555 + M + N + K)
    y = vpq.ops.qmm(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16),
                    to_dev(x, torch.bfloat16))
    assert vpq.ops.device_status() == 0
    e = check_linear(oracle_mod, y, codes, s, b, x)
    assert e["rel_l2"] < 3e-2          # the reference's bound
    # against the reference kernels' own numerics (W rounded to bf16 first) the
    # only difference left is the f32 summation order
    want = synth.bf16_bits_to_f32(oracle_mod.qmm_kernel_numerics(codes, s, b, x))
    assert oracle_mod.err_metrics(f32(y), want)["rel_l2"] < 2e-3


@pytest.mark.parametrize("tag,M,K,N", [("C3.q", 2048, 4096, 4096), ("C3.k", 2048, 4096, 1024),
                                       ("C3.down", 2048, 12288, 4096),
                                       ("shard-1728", 384, 5120, 1728), ("m-tail", 1000, 1024, 520)])
def test_qmm_matches_fp32_oracle(vpq, oracle_mod, tag, M, K, N):
    codes, s, b = quantized_linear(oracle_mod, N, K, synth.seed_for("qmm-w", tag))
    x = synth.activations_bf16(M, K, synth.seed_for("qmm-x", tag))
    y = vpq.ops.qmm(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16),
                    to_dev(x, torch.bfloat16))
    assert vpq.ops.device_status() == 0
    rows = None if M <= 512 else np.unique(np.concatenate(
        [np.arange(0, M, 61), [0, 127, 128, M - 129, M - 1]]))
    check_linear(oracle_mod, y, codes, s, b, x, rows=rows)


def _device_linear(vpq, N, K, M, seed):
    g = torch.Generator(device=dev()).manual_seed(seed)
    w = (torch.randn((N, K), generator=g, device=dev(), dtype=torch.float32) * 0.02).to(torch.bfloat16)
    codes, s16, b16 = vpq.ops.quantize(w)
    s, b = vpq.ops.scales_to_bf16(s16), vpq.ops.scales_to_bf16(b16)
    x = torch.randn((M, K), generator=g, device=dev(), dtype=torch.float32).to(torch.bfloat16)
    return codes, s, b, x


@pytest.mark.parametrize("tag,M,K,N", [("C3.gate", 2048, 4096, 12288), ("C4.mlp_down", 4096, 16384, 4096),
                                       ("C5.out-slab", 16384, 5120, 5120)])
def test_qmm_full_size_against_dequant_then_dense(vpq, oracle_mod, tag, M, K, N):
    """Full-size property: the fused kernel equals dequantise-once followed by a dense
    f32-accumulate matmul of the same bf16 operands (the reference's own comparator,
    tests/unit-tests/metal-compute-gemm-mma.cc:1995-2131), plus oracle parity on sampled rows."""
    codes, s, b, x = _device_linear(vpq, N, K, M, synth.seed_for("full", tag))
    y = vpq.ops.qmm(codes, s, b, x)
    assert vpq.ops.device_status() == 0
    wd = vpq.ops.dequantize(codes, s, b)
    num = 0.0
    den = 0.0
    for m0 in range(0, M, 4096):
        ref = x[m0:m0 + 4096].float() @ wd.float().t()
        d = y[m0:m0 + 4096].float() - ref
        num += float((d * d).sum())
        den += float((ref * ref).sum())
        assert float(d.abs().max()) <= TOL * float(ref.abs().max())
    assert (num / den) ** 0.5 < 3e-3
    rows = np.arange(0, M, max(M // 24, 1))
    check_linear(oracle_mod, y, bits32(codes), bits16(s), bits16(b), bits16(x), rows=rows)


# Every projection of the prefill / DiT configurations that is not covered above, at full size:
# C3 v / gate / up (M = 2048), C4 qkv / proj / mlp_up (M = 4096), and the four C5 shapes at the full
# M = 65280 (y up to 2.0 GB: row offsets near 2^31 bytes, the overflow class the reference guards
# against in tests/unit-tests/minimax-h3-blocks.cc:1792-1812). The oracle runs on sampled rows that
# include the first and last rows of the output and of interior row tiles.
FULL_SHAPES = [("C3.v", 2048, 4096, 1024), ("C3.gate", 2048, 4096, 12288), ("C3.up", 2048, 4096, 12288),
               ("C4.qkv", 4096, 4096, 12288), ("C4.proj", 4096, 4096, 4096), ("C4.mlp_up", 4096, 4096, 16384),
               ("C5.qkv", 65280, 5120, 15360), ("C5.out", 65280, 5120, 5120),
               ("C5.ffn_up", 65280, 5120, 13824), ("C5.ffn_down", 65280, 13824, 5120)]


@pytest.mark.parametrize("tag,M,K,N", FULL_SHAPES)
def test_qmm_full_configs_on_sampled_rows(vpq, oracle_mod, tag, M, K, N):
    codes, s, b, x = _device_linear(vpq, N, K, M, synth.seed_for("cfg", tag))
    y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    vpq.ops.qmm(codes, s, b, x, out=y)
    assert vpq.ops.device_status() == 0
    rng = np.random.Generator(np.random.Philox(key=synth.seed_for("rows", tag)))
    n_rows = 96 if M > 8192 else 64
    rows = np.unique(np.concatenate([rng.integers(0, M, n_rows), [0, 1, 127, 128, 255, 256, M // 2, M - 257,
                                                                  M - 256, M - 129, M - 128, M - 2, M - 1]]))
    idx = torch.from_numpy(rows).to(dev())
    ys = y.index_select(0, idx)
    xs = bits16(x.index_select(0, idx))
    deq = oracle_mod.dequant_f32(bits32(codes), bits16(s), bits16(b))
    ref = oracle_mod.matmul_f32(xs, deq, "fast")
    e = oracle_mod.err_metrics(f32(ys), ref)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, (tag, e)
    # every element was written (none of the NaN fill left), checked on the device
    assert int(torch.isnan(y).sum()) == 0


@pytest.mark.parametrize("M,K,q_rows,k_rows,v_rows", [(2048, 4096, 4096, 1024, 1024), (300, 1024, 256, 128, 72)])
def test_qmm_qkv_in_one_gemm_equals_three(vpq, oracle_mod, M, K, q_rows, k_rows, v_rows):
    """q | k | v as one GEMM over the row-concatenated weight: each output carries exactly the bytes of
    the plain GEMM on that projection's row slice, and the whole matches the fp32 oracle."""
    N = q_rows + k_rows + v_rows
    codes, s, b, x = _device_linear(vpq, N, K, M, synth.seed_for("qkvmm", M, K))
    q, k, v = vpq.ops.qmm_qkv(codes, s, b, x, q_rows, k_rows, v_rows)
    assert vpq.ops.device_status() == 0
    lo = 0
    for out, rows in ((q, q_rows), (k, k_rows), (v, v_rows)):
        want = vpq.ops.qmm(codes[lo:lo + rows].contiguous(), s[lo:lo + rows].contiguous(),
                           b[lo:lo + rows].contiguous(), x)
        assert torch.equal(out, want)
        lo += rows
    rows_s = np.arange(0, M, max(M // 16, 1))
    check_linear(oracle_mod, torch.cat([q, k, v], dim=1), bits32(codes), bits16(s), bits16(b), bits16(x), rows=rows_s)


def test_dispatch_by_reference_names(vpq, oracle_mod):
    """load_library(...).function(...) + slot-numbered dispatch gives the same bytes as the direct calls."""
    N, K, M = 256, 1024, 160
    codes, s, b = quantized_linear(oracle_mod, N, K, 61)
    x = synth.activations_bf16(M, K, 62)
    dc, ds, db, dx = to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16)
    ops = vpq.ops
    y1 = torch.empty((M, N), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm128"),
                 [dc, ds, db, dx, y1], K=K, N=N, M=M)
    assert torch.equal(y1, ops.qmm(dc, ds, db, dx))
    y2 = torch.empty((1, N), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_w4g64"), [dc, ds, db, dx[:1], y2], K=K, N=N, M=1)
    assert torch.equal(y2, ops.qmv(dc, ds, db, dx[:1]))
    wd = torch.empty((N, K), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_dequant_bf16", "affine_dequant_w4g64"), [dc, ds, db, wd], K=K, N=N)
    assert np.array_equal(bits16(wd), oracle_mod.dequant_bf16(codes, s, b))
    wsrc = to_dev(synth.f32_to_bf16_bits(synth.weight_f32(N, K, 63)), torch.bfloat16)
    c2 = torch.empty((N, K // 8), dtype=torch.int32, device=dev())
    s2 = torch.empty((N, K // 64), dtype=torch.float16, device=dev())
    b2 = torch.empty_like(s2)
    ops.dispatch(ops.function("affine_dequant_bf16", "affine_quant_w4_g64"), [wsrc, c2, s2, b2], K=K, N=N, clip=1.0)
    c3, s3, b3 = ops.quantize(wsrc)
    assert torch.equal(c2, c3) and torch.equal(s2, s3) and torch.equal(b2, b3)


def test_large_plan_with_a_pool_of_chunks_equals_single_launches(vpq, oracle_mod):
    """A plan with enough row tiles hands its last tenth out at run time (chunks claimed by the CTAs
    that finish first). Whoever computes a tile, the bytes must be those of the per-GEMV launches, on
    every run, also back to back without a host synchronise (the next run's claims wait for the
    previous run to put the counter back)."""
    torch.manual_seed(5)
    shapes = [(512, 4096)] * 30 + [(1024, 2064), (3840, 1000), (256, 4096), (512, 4096), (1536, 2048)] * 3
    xs = {}
    problems, singles = [], []
    for i, (K, N) in enumerate(shapes):
        codes = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device=dev())
        s = (torch.rand((N, K // 64), device=dev()) * 0.015 + 0.005).to(torch.bfloat16)
        b = (torch.rand((N, K // 64), device=dev()) * 0.2 - 0.1).to(torch.bfloat16)
        if (K, i % 3) not in xs:
            xs[(K, i % 3)] = torch.randn((1, K), device=dev()).to(torch.bfloat16)
        x = xs[(K, i % 3)]
        y = torch.zeros((1, N), dtype=torch.bfloat16, device=dev())
        problems.append((codes, s, b, x, y))
        singles.append(vpq.ops.qmv(codes, s, b, x))
    assert sum((N + 15) // 16 for _, N in shapes) >= 32 * 2 * torch.cuda.get_device_properties(dev()).multi_processor_count
    plan = vpq.ops.QmvPlan(problems)
    for run in range(3):
        for p in problems:
            p[4].zero_()
        plan.run()
        plan.run()
        plan.run()
        torch.cuda.synchronize()
        for i, (p, want) in enumerate(zip(problems, singles)):
            assert torch.equal(p[4], want), f"run {run}: GEMV {i} differs"
    plan.close()
    assert vpq.ops.device_status() == 0


def test_qmv_and_qmm_agree_on_small_m(vpq, oracle_mod):
    """Both kernels on the same rows: QMM rounds W to bf16 first, so agreement is to tolerance."""
    N, K, M = 1024, 4096, 4
    codes, s, b = quantized_linear(oracle_mod, N, K, 71)
    x = synth.activations_bf16(M, K, 72)
    args = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    yv, ym = vpq.ops.qmv(*args), vpq.ops.qmm(*args)
    assert oracle_mod.err_metrics(f32(ym), f32(yv))["max_rel_rms"] < TOL


def test_qmv_plan_equals_single_launches(vpq, oracle_mod):
    """A plan (all GEMVs in one launch) must give the bytes of the per-GEMV launches: shared x
    (q|k|v), a different K (down), a K whose scales cannot be TMA boxes (3840), ragged N, M = 2."""
    shapes = [(4096, 512, 1), (4096, 128, 1), (4096, 136, 1), (12288, 256, 1), (3840, 40, 1),
              (1024, 33, 2), (4096, 4096, 1)]
    xs = {}
    problems, singles = [], []
    for i, (K, N, M) in enumerate(shapes):
        codes, s, b = quantized_linear(oracle_mod, N, K, 900 + i)
        if (K, M) not in xs:
            xs[(K, M)] = to_dev(synth.activations_bf16(M, K, 950 + K + M), torch.bfloat16)
        x = xs[(K, M)]
        dc, ds, db = to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16)
        y = torch.zeros((M, N), dtype=torch.bfloat16, device=dev())
        problems.append((dc, ds, db, x, y))
        singles.append(vpq.ops.qmv(dc, ds, db, x))
    plan = vpq.ops.QmvPlan(problems)
    for _ in range(2):          # a plan is re-runnable
        for p in problems:
            p[4].zero_()
        plan.run()
        torch.cuda.synchronize()
        for p, want in zip(problems, singles):
            assert torch.equal(p[4], want)
    plan.close()
    assert vpq.ops.device_status() == 0
