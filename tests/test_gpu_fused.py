"""GPU parity of the fused decode GEMVs (residual add, SwiGLU over interleaved gate | up, q | k | v
with three outputs) against the oracle's restatement of the reference's fused stores
(gpu-kernels/metal/quant/affine_qmv.metal:265-270, 806-906, 405-516), through the C ABI.

Two kinds of check: against the fp32 oracle within the 1e-2 tolerance of the plain GEMV, and
bit-exact consistency with the plain GEMV where the fused store is a function of its bf16 output
(add, qkv)."""
import numpy as np
import pytest
import torch

from vpipe_b200 import synth

from test_gpu_parity import TOL, bits16, bits32, dev, f32, quantized_linear, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(vpq):
    assert torch.cuda.is_available(), "the -m gpu tests need a CUDA device"
    torch.cuda.set_device(0)
    yield
    torch.cuda.synchronize()
    assert vpq.ops.device_status() == 0


def _linear(oracle_mod, N, K, M, seed):
    codes, s, b = quantized_linear(oracle_mod, N, K, seed)
    x = synth.activations_bf16(M, K, seed + 1)
    ref = oracle_mod.linear_f32(codes, s, b, x, "fast")
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    return d, ref


@pytest.mark.parametrize("K,N,M", [(4096, 4096, 1), (12288, 4096, 1), (320, 33, 2), (3840, 16, 1)])
def test_qmv_add(vpq, oracle_mod, K, N, M):
    d, ref = _linear(oracle_mod, N, K, M, 7000 + N + K)
    res = synth.activations_bf16(M, N, 7100 + N)
    dres = to_dev(res, torch.bfloat16)
    y = vpq.ops.qmv_add(*d, dres)
    want = synth.bf16_bits_to_f32(oracle_mod.fused_add(ref, res))
    e = oracle_mod.err_metrics(f32(y), want)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, e
    # the same sums as the plain GEMV, rounded to bf16, then one bf16 add
    plain = vpq.ops.qmv(*d)
    assert torch.equal(y, (plain.float() + dres.float()).to(torch.bfloat16))


@pytest.mark.parametrize("K,N,M", [(4096, 2 * 1024, 1), (4096, 2 * 12288, 1), (1088, 18, 2), (64, 2, 1)])
def test_qmv_swiglu(vpq, oracle_mod, K, N, M):
    d, ref = _linear(oracle_mod, N, K, M, 7200 + N + K)
    y = vpq.ops.qmv_swiglu(*d)
    assert y.shape == (M, N // 2)
    want = synth.bf16_bits_to_f32(oracle_mod.fused_swiglu(ref))
    e = oracle_mod.err_metrics(f32(y), want)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, e
    # against silu(gate) * up formed from the plain GEMV's bf16 outputs: equal up to their rounding
    plain = vpq.ops.qmv(*d).float()
    g, u = plain[:, 0::2], plain[:, 1::2]
    approx = (g / (1.0 + torch.exp(-g)) * u).cpu().numpy()
    assert oracle_mod.err_metrics(f32(y), approx)["max_rel_rms"] < 2e-2


def test_qmv_swiglu_does_not_write_past_the_halved_output(vpq, oracle_mod):
    K, N = 1024, 70
    d, _ = _linear(oracle_mod, N, K, 1, 7300)
    pad = 64
    buf = torch.full((pad + N // 2 + pad,), -3.0, dtype=torch.bfloat16, device=dev())
    y = buf[pad:pad + N // 2].view(1, N // 2)
    vpq.ops.qmv_swiglu(*d, out=y)
    assert torch.all(buf[:pad] == -3.0) and torch.all(buf[pad + N // 2:] == -3.0)
    assert torch.all(y != -3.0)


@pytest.mark.parametrize("K,q,k,v,M", [(4096, 4096, 1024, 1024, 1), (1024, 40, 24, 8, 2), (512, 16, 16, 0, 1),
                                         (512, 19, 5, 11, 1)])
def test_qmv_qkv_lands_rows_in_three_buffers(vpq, oracle_mod, K, q, k, v, M):
    N = q + k + v
    d, ref = _linear(oracle_mod, N, K, M, 7400 + N + K)
    yq, yk, yv = vpq.ops.qmv_qkv(*d, q, k, v)
    plain = vpq.ops.qmv(*d)
    assert torch.equal(yq, plain[:, :q])
    assert torch.equal(yk, plain[:, q:q + k])
    assert torch.equal(yv, plain[:, q + k:])
    e = oracle_mod.err_metrics(f32(torch.cat([yq, yk, yv], dim=1)), ref)
    assert e["rel_l2"] < TOL, e


def test_fused_stores_inside_a_plan(vpq, oracle_mod):
    """One launch holding a q|k|v GEMV, a SwiGLU gate|up GEMV and a down GEMV with residual: the
    bytes of the three single calls."""
    K, F = 1024, 1536
    dq, _ = _linear(oracle_mod, 1024 + 256 + 256, K, 1, 7500)
    dg, _ = _linear(oracle_mod, 2 * F, K, 1, 7510)
    dd, _ = _linear(oracle_mod, K, F, 1, 7520)
    res = to_dev(synth.activations_bf16(1, K, 7530), torch.bfloat16)
    want_qkv = vpq.ops.qmv_qkv(*dq, 1024, 256, 256)
    want_act = vpq.ops.qmv_swiglu(*dg)
    want_out = vpq.ops.qmv_add(*dd, res)
    z = lambda n: torch.zeros((1, n), dtype=torch.bfloat16, device=dev())
    yq, yk, yv, act, out = z(1024), z(256), z(256), z(F), z(K)
    plan = vpq.ops.QmvPlan([
        dq + (yq, {"epilogue": "qkv", "aux": yk, "y3": yv, "q_rows": 1024, "k_rows": 256}),
        dg + (act, {"epilogue": "swiglu"}),
        dd + (out, {"epilogue": "add", "aux": res}),
    ])
    plan.run()
    torch.cuda.synchronize()
    assert torch.equal(yq, want_qkv[0]) and torch.equal(yk, want_qkv[1]) and torch.equal(yv, want_qkv[2])
    assert torch.equal(act, want_act)
    assert torch.equal(out, want_out)
    plan.close()


def test_fused_entries_by_reference_names(vpq, oracle_mod):
    ops = vpq.ops
    K, N = 512, 48
    d, _ = _linear(oracle_mod, N, K, 1, 7600)
    res = to_dev(synth.activations_bf16(1, N, 7610), torch.bfloat16)
    y = torch.empty((1, N), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_w4g64_add"),
                 {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: y, 7: res}, K=K, N=N)
    assert torch.equal(y, ops.qmv_add(*d, res))
    y2 = torch.empty((1, N // 2), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_swiglu_w4g64"),
                 {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: y2}, K=K, N=N)
    assert torch.equal(y2, ops.qmv_swiglu(*d))
    yq, yk, yv = (torch.empty((1, n), dtype=torch.bfloat16, device=dev()) for n in (16, 16, 16))
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_qkv_w4g64"),
                 {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: yq, 5: yk, 6: yv}, K=K, q_rows=16, k_rows=16, v_rows=16)
    want = ops.qmv_qkv(*d, 16, 16, 16)
    assert torch.equal(yq, want[0]) and torch.equal(yk, want[1]) and torch.equal(yv, want[2])


# ------------------------------------------------------------------------ GEMM

@pytest.mark.parametrize("M,K,N", [(256, 512, 512), (300, 1024, 154), (129, 64, 2), (2048, 4096, 2 * 1024),
                                   (64, 256, 96)])
def test_qmm_swiglu(vpq, oracle_mod, M, K, N):
    """Fused SwiGLU GEMM (affine_qmm_swiglu_w4g64, affine_qmm_steel.metal:641-827) against the
    oracle's silu(gate) * up over the fp32 dequantise-then-matmul reference; ragged M and N."""
    codes, s, b = quantized_linear(oracle_mod, N, K, 7700 + M + N + K)
    x = synth.activations_bf16(M, K, 7701 + M + N + K)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    y = vpq.ops.qmm_swiglu(*d)
    assert y.shape == (M, N // 2)
    assert vpq.ops.device_status() == 0
    # the GEMM multiplies W rounded to bf16, as the reference's does (affine_qmm_steel.metal:86-95):
    # with the same W the only difference left is the f32 summation order
    w_bf16 = oracle_mod.bf16_to_f32(oracle_mod.dequant_bf16(codes, s, b))
    want = synth.bf16_bits_to_f32(oracle_mod.fused_swiglu(oracle_mod.matmul_f32(x, w_bf16, "fast")))
    e = oracle_mod.err_metrics(f32(y), want)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, e
    # against the fp32 dequantise-then-matmul oracle the bf16 rounding of W (~1e-3 per product
    # sum) is amplified by |up| and |silu'(gate)|: the reference's own GEMM bound, rel-L2 < 3e-2
    ref = oracle_mod.linear_f32(codes, s, b, x, "fast")
    e32 = oracle_mod.err_metrics(f32(y), synth.bf16_bits_to_f32(oracle_mod.fused_swiglu(ref)))
    assert e32["rel_l2"] < 5e-3 and e32["max_rel_rms"] < 3e-2, e32
    # and against silu(gate) * up formed from the plain GEMM's bf16 output
    plain = vpq.ops.qmm(*d).float()
    g, u = plain[:, 0::2], plain[:, 1::2]
    approx = (g / (1.0 + torch.exp(-g)) * u).cpu().numpy()
    assert oracle_mod.err_metrics(f32(y), approx)["max_rel_rms"] < 2e-2


def test_qmm_swiglu_stays_inside_its_output(vpq, oracle_mod):
    M, K, N = 130, 128, 66
    d, _ = _linear(oracle_mod, N, K, M, 7800)
    pad = 128
    buf = torch.full((pad + M * (N // 2) + pad,), -3.0, dtype=torch.bfloat16, device=dev())
    y = buf[pad:pad + M * (N // 2)].view(M, N // 2)
    vpq.ops.qmm_swiglu(*d, out=y)
    assert torch.all(buf[:pad] == -3.0) and torch.all(buf[pad + M * (N // 2):] == -3.0)
    assert torch.all(y != -3.0)


def test_qmm_swiglu_by_reference_names(vpq, oracle_mod):
    ops = vpq.ops
    M, K, N = 256, 256, 256
    d, _ = _linear(oracle_mod, N, K, M, 7900)
    want = ops.qmm_swiglu(*d)
    for entry in ("affine_qmm_swiglu_w4g64", "affine_qmm_swiglu_w4g64_bm64", "affine_qmm_swiglu_w4g64_bm128"):
        y = torch.empty((M, N // 2), dtype=torch.bfloat16, device=dev())
        ops.dispatch(ops.function("affine_qmm_steel_bf16", entry), {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: y},
                     K=K, N=N, M=M)
        assert torch.equal(y, want)


def test_checkpoint_on_disk_loads_and_computes(vpq, oracle_mod, tmp_path):
    """quantize (GPU) -> write the reference's on-disk triple -> load -> dequantize / GEMV: the
    bytes survive the file format and the result equals the oracle's."""
    from vpipe_b200 import checkpoint
    N, K = 96, 512
    w = to_dev(synth.f32_to_bf16_bits(synth.weight_f32(N, K, 8100)), torch.bfloat16)
    codes, s16, b16 = vpq.ops.quantize(w)
    checkpoint.write_model(str(tmp_path), {
        "layers.0.proj.weight": bits32(codes),
        "layers.0.proj.scales": bits16(s16).view(np.float16),
        "layers.0.proj.biases": bits16(b16).view(np.float16),
    }, 64, 4)
    m = checkpoint.Model(str(tmp_path))
    c2, s2, b2 = checkpoint.load_quant_linear(m, "layers.0.proj", dev())
    assert torch.equal(c2, codes)
    want = oracle_mod.dequant_bf16(bits32(codes), oracle_mod.f16_to_bf16(bits16(s16)), oracle_mod.f16_to_bf16(bits16(b16)))
    assert np.array_equal(bits16(vpq.ops.dequantize(c2, s2, b2)), want)


# ------------------------------------------------------------------------ small-batch GEMV

@pytest.mark.parametrize("K,N,M", [(4096, 4096, 4), (4096, 1024, 2), (12288, 4096, 3), (4096, 12288, 8),
                                   (3840, 40, 3), (64, 8, 2), (320, 33, 5), (1088, 8193, 1)])
def test_qmv_batch_rows_share_one_weight_stream(vpq, oracle_mod, K, N, M):
    """affine_qmv_batch(4)_w4g64 (affine_qmv.metal:1553-1705): every row within the GEMV's tolerance
    of the fp32 oracle and equal, up to f32 rounding before the bf16 store, to the M = 1 kernel's."""
    d, ref = _linear(oracle_mod, N, K, M, 8200 + N + K + M)
    y = vpq.ops.qmv_batch_rows(*d)
    assert y.shape == (M, N)
    e = oracle_mod.err_metrics(f32(y), ref)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL and e["max_rel_1e2"] < TOL, e
    serial = vpq.ops.qmv(*d)
    a, b = f32(y), f32(serial)
    # one bf16 ulp of the larger magnitude (2^-7 relative), or f32 noise next to a zero crossing
    assert np.all(np.abs(a - b) <= np.maximum(np.abs(a), np.abs(b)) * 2.0 ** -7 + 1e-5 * np.abs(b).max())
    assert (bits16(y) == bits16(serial)).mean() > (0.97 if y.numel() >= 1000 else 0.85)


def test_qmv_batch_rows_with_very_different_magnitudes(vpq, oracle_mod):
    """Each row of x has its own power-of-two scale: a row 2^40 times larger than its neighbour
    must not cost the small one its accuracy."""
    K, N = 2048, 64
    codes, s, b = quantized_linear(oracle_mod, N, K, 8300)
    x = synth.bf16_bits_to_f32(synth.activations_bf16(3, K, 8301))
    x[1] *= 2.0 ** 40
    x[2] *= 2.0 ** -30
    xb = synth.f32_to_bf16_bits(x)
    y = vpq.ops.qmv_batch_rows(to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16),
                               to_dev(xb, torch.bfloat16))
    ref = oracle_mod.linear_f32(codes, s, b, xb, "f64")
    for m in range(3):
        e = oracle_mod.err_metrics(f32(y)[m:m + 1], ref[m:m + 1])
        assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, (m, e)


def test_qmv_batch_by_reference_names(vpq, oracle_mod):
    ops = vpq.ops
    K, N, M = 512, 48, 4
    d, _ = _linear(oracle_mod, N, K, M, 8400)
    want = ops.qmv_batch_rows(*d)
    for entry in ("affine_qmv_batch_w4g64", "affine_qmv_batch4_w4g64"):
        y = torch.empty((M, N), dtype=torch.bfloat16, device=dev())
        ops.dispatch(ops.function("affine_qmv_bf16", entry), {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: y},
                     K=K, N=N, M=M)
        assert torch.equal(y, want)
