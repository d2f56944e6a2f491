"""The other gated stores of the reference's quantized linears: GeGLU on the GEMV and the GEMM
(affine_qmv_geglu_w4g64, affine_qmm_geglu_w4g64), the per-layer-input gate (affine_qmv_gelu_mul_w4g64)
and both activations over 8-bit weights (affine_qmm_swiglu_w8g64, affine_qmm_geglu_w8g64). The
activation is gelu_pytorch_tanh, restated in the oracle from ops/llm_elementwise.metal:388-407."""
import numpy as np
import pytest
import torch

from vpipe_b200 import synth

from test_gpu_parity import TOL, dev, f32, quantized_linear, to_dev

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


def _gelu_t(x):
    return torch.nn.functional.gelu(x, approximate="tanh")


@pytest.mark.parametrize("K,N,M", [(4096, 2 * 1024, 1), (2560, 2 * 10240, 1), (1088, 18, 2), (64, 2, 1)])
def test_qmv_geglu(vpq, oracle_mod, K, N, M):
    d, ref = _linear(oracle_mod, N, K, M, 8200 + N + K)
    y = vpq.ops.qmv_geglu(*d)
    assert y.shape == (M, N // 2)
    want = synth.bf16_bits_to_f32(oracle_mod.fused_geglu(ref))
    e = oracle_mod.err_metrics(f32(y), want)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, e
    plain = vpq.ops.qmv(*d).float()
    approx = (_gelu_t(plain[:, 0::2]) * plain[:, 1::2]).cpu().numpy()
    assert oracle_mod.err_metrics(f32(y), approx)["max_rel_rms"] < 2e-2


@pytest.mark.parametrize("K,N,M", [(2560, 256, 1), (4096, 4096, 1), (320, 33, 2)])
def test_qmv_gelu_mul(vpq, oracle_mod, K, N, M):
    d, ref = _linear(oracle_mod, N, K, M, 8300 + N + K)
    mul = synth.activations_bf16(M, N, 8301 + N)
    dmul = to_dev(mul, torch.bfloat16)
    y = vpq.ops.qmv_gelu_mul(*d, dmul)
    want = synth.bf16_bits_to_f32(oracle_mod.fused_gelu_mul(ref, mul))
    e = oracle_mod.err_metrics(f32(y), want)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, e
    # the activation reads the bf16-rounded GEMV result: a separate pass over y gives the same values
    # up to the accuracy of tanh
    plain = vpq.ops.qmv(*d).float()
    sep = (_gelu_t(plain) * dmul.float()).to(torch.bfloat16)
    diff = (y.float() - sep.float()).abs()
    assert float((diff <= 2 ** -7 * sep.float().abs() + 1e-30).float().mean()) == 1.0
    assert float((y == sep).float().mean()) > 0.99


def test_gated_gemvs_inside_a_plan_and_by_name(vpq, oracle_mod):
    ops = vpq.ops
    K, N = 1024, 512
    d, _ = _linear(oracle_mod, N, K, 1, 8400)
    mul = to_dev(synth.activations_bf16(1, N, 8401), torch.bfloat16)
    want_g = ops.qmv_geglu(*d)
    want_m = ops.qmv_gelu_mul(*d, mul)
    y_g = torch.zeros((1, N // 2), dtype=torch.bfloat16, device=dev())
    y_m = torch.zeros((1, N), dtype=torch.bfloat16, device=dev())
    ops.qmv_batch(ops.qmv_set([d + (y_g, {"epilogue": "geglu"}),
                               d + (y_m, {"epilogue": "gelu_mul", "aux": mul})]))
    assert torch.equal(y_g, want_g) and torch.equal(y_m, want_m)
    y2 = torch.zeros_like(y_g)
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_geglu_w4g64"), list(d) + [y2], K=K, N=N)
    assert torch.equal(y2, want_g)
    y3 = torch.zeros_like(y_m)
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_gelu_mul_w4g64"),
                 {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: y3, 7: mul}, K=K, N=N)
    assert torch.equal(y3, want_m)


def _w8_linear(oracle_mod, N, K, M, seed):
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, seed))
    codes, s16, b16 = oracle_mod.quant(wb, 8, 64)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, seed + 1)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    return (codes, s, b, x), d


@pytest.mark.parametrize("bits,act", [(4, "geglu"), (8, "swiglu"), (8, "geglu")])
@pytest.mark.parametrize("M,K,N", [(256, 512, 512), (300, 1024, 154), (129, 64, 2), (2048, 2560, 2 * 1024)])
def test_qmm_gated(vpq, oracle_mod, bits, act, M, K, N):
    """With the same bf16 W the only difference from the oracle is the f32 summation order; the
    store applies the activation to the unrounded accumulators (affine_qmm_steel.metal:1535-1545)."""
    seed = 8500 + M + N + K + bits
    if bits == 4:
        codes, s, b = quantized_linear(oracle_mod, N, K, seed)
        x = synth.activations_bf16(M, K, seed + 1)
        d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    else:
        (codes, s, b, x), d = _w8_linear(oracle_mod, N, K, M, seed)
    y = vpq.ops.qmm_swiglu(*d, act=act, bits=bits)
    assert y.shape == (M, N // 2)
    assert vpq.ops.device_status() == 0
    w_bf16 = oracle_mod.bf16_to_f32(oracle_mod.dequant_bf16_any(codes, s, b, bits, 64))
    fuse = oracle_mod.fused_geglu if act == "geglu" else oracle_mod.fused_swiglu
    want = synth.bf16_bits_to_f32(fuse(oracle_mod.matmul_f32(x, w_bf16, "fast")))
    e = oracle_mod.err_metrics(f32(y), want)
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, e
    plain = (vpq.ops.qmm(*d) if bits == 4 else vpq.ops.qmm_w8(*d)).float()
    g, u = plain[:, 0::2], plain[:, 1::2]
    approx = ((_gelu_t(g) if act == "geglu" else g / (1.0 + torch.exp(-g))) * u).cpu().numpy()
    assert oracle_mod.err_metrics(f32(y), approx)["max_rel_rms"] < 2e-2


def test_qmm_gated_by_reference_names(vpq, oracle_mod):
    ops = vpq.ops
    M, K, N = 256, 256, 256
    d4, _ = _linear(oracle_mod, N, K, M, 8600)
    _, d8 = _w8_linear(oracle_mod, N, K, M, 8601)
    for entry, d, act, bits in (("affine_qmm_geglu_w4g64", d4, "geglu", 4),
                                ("affine_qmm_swiglu_w8g64", d8, "swiglu", 8),
                                ("affine_qmm_swiglu_w8g64_bm64", d8, "swiglu", 8),
                                ("affine_qmm_geglu_w8g64", d8, "geglu", 8)):
        want = ops.qmm_swiglu(*d, act=act, bits=bits)
        y = torch.empty((M, N // 2), dtype=torch.bfloat16, device=dev())
        ops.dispatch(ops.function("affine_qmm_steel_bf16", entry), {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: y},
                     K=K, N=N, M=M)
        assert torch.equal(y, want), entry


# ------------------------------------------------------- fused stores of the 8-bit GEMV

@pytest.mark.parametrize("K,N,M", [(1024, 512, 1), (2560, 40, 2), (64, 6, 1)])
def test_qmv_w8_fused_stores_equal_a_separate_pass(vpq, oracle_mod, K, N, M):
    """affine_qmv_w8g64_add / swiglu_w8g64 / qkv_w8g64 / gelu_mul_w8g64: the sums are the plain 8-bit
    GEMV's; add and gelu*mul act on its bf16 output (bit-equal), the gated stores on the f32 sums."""
    ops = vpq.ops
    (codes, s, b, x), d = _w8_linear(oracle_mod, N, K, M, 8700 + N + K)
    plain = ops.qmv_w8(*d)
    aux = to_dev(synth.activations_bf16(M, N, 8701 + N), torch.bfloat16)
    z = lambda *shape: torch.full(shape, -3.0, dtype=torch.bfloat16, device=dev())

    y = ops.qmv_w8_fused(*d, z(M, N), {"epilogue": "add", "aux": aux})
    assert torch.equal(y, (plain.float() + aux.float()).to(torch.bfloat16))

    y = ops.qmv_w8_fused(*d, z(M, N), {"epilogue": "gelu_mul", "aux": aux})
    sep = (_gelu_t(plain.float()) * aux.float()).to(torch.bfloat16)
    assert float((y == sep).float().mean()) > 0.98
    assert oracle_mod.err_metrics(f32(y), f32(sep))["max_rel_rms"] < 1e-2

    q_rows, k_rows = (N // 2) & ~1, N // 4
    yq, yk, yv = z(M, q_rows), z(M, k_rows), z(M, N - q_rows - k_rows)
    ops.qmv_w8_fused(*d, yq, {"epilogue": "qkv", "aux": yk, "y3": yv, "q_rows": q_rows, "k_rows": k_rows})
    assert torch.equal(torch.cat([yq, yk, yv], dim=1), plain)

    # fp32 dequantise-then-matmul reference for the gated stores
    q = codes.view(np.uint8).reshape(N, K).astype(np.float32)
    wf = (np.repeat(synth.bf16_bits_to_f32(s), 64, axis=1) * q + np.repeat(synth.bf16_bits_to_f32(b), 64, axis=1))
    ref = oracle_mod.matmul_f32(x, wf.astype(np.float32), "fast")
    for name, fuse in (("swiglu", oracle_mod.fused_swiglu), ("geglu", oracle_mod.fused_geglu)):
        y = ops.qmv_w8_fused(*d, z(M, N // 2), {"epilogue": name})
        e = oracle_mod.err_metrics(f32(y), synth.bf16_bits_to_f32(fuse(ref)))
        assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, (name, e)


def test_qmv_w8_fused_by_reference_names(vpq, oracle_mod):
    ops = vpq.ops
    K, N = 512, 256
    _, d = _w8_linear(oracle_mod, N, K, 1, 8800)
    aux = to_dev(synth.activations_bf16(1, N, 8801), torch.bfloat16)
    z = lambda n: torch.zeros((1, n), dtype=torch.bfloat16, device=dev())
    for entry, store, width in (("affine_qmv_w8g64_add", {"epilogue": "add", "aux": aux}, N),
                                ("affine_qmv_gelu_mul_w8g64", {"epilogue": "gelu_mul", "aux": aux}, N),
                                ("affine_qmv_swiglu_w8g64", {"epilogue": "swiglu"}, N // 2)):
        want = ops.qmv_w8_fused(*d, z(width), store)
        y = z(width)
        ops.dispatch(ops.function("affine_qmv_bf16", entry), {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: y, 7: aux},
                     K=K, N=N)
        assert torch.equal(y, want), entry
    plain = ops.qmv_w8(*d)
    yq, yk, yv = z(128), z(64), z(64)
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_qkv_w8g64"),
                 {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: yq, 5: yk, 6: yv}, K=K, q_rows=128, k_rows=64, v_rows=64)
    assert torch.equal(torch.cat([yq, yk, yv], dim=1), plain)


# ------------------------------------------------------- SwiGLU GEMM into a column block

@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,K,N,stride,off", [(256, 512, 512, 1024, 512), (300, 256, 154, 203, 61), (130, 64, 64, 32, 0)])
def test_qmm_swiglu_into_a_column_block(vpq, oracle_mod, bits, M, K, N, stride, off):
    """affine_qmm_swiglu_w4g64_bm64_rs / _w8g64_bm64_rs (affine_qmm_steel.metal:657-770,925-947): the
    values of the contiguous call, at y[m * out_stride + out_off + j]; nothing else is written."""
    ops = vpq.ops
    if bits == 4:
        d, _ = _linear(oracle_mod, N, K, M, 8900 + M + N)
    else:
        _, d = _w8_linear(oracle_mod, N, K, M, 8900 + M + N)
    want = ops.qmm_swiglu(*d, bits=bits)
    out = torch.full((M, stride), -3.0, dtype=torch.bfloat16, device=dev())
    ops.qmm_swiglu_into(*d, out, off, bits=bits)
    assert ops.device_status() == 0
    assert torch.equal(out[:, off:off + N // 2], want)
    assert torch.all(out[:, :off] == -3.0) and torch.all(out[:, off + N // 2:] == -3.0)
    name = f"affine_qmm_swiglu_w{bits}g64_bm64_rs"
    out2 = torch.full((M, stride), -3.0, dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmm_steel_bf16", name), {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: out2},
                 K=K, N=N, M=M, out_stride=stride, out_off=off)
    assert torch.equal(out2, out)


def test_qmm_swiglu_block_must_fit_its_row(vpq, oracle_mod):
    ops = vpq.ops
    d, _ = _linear(oracle_mod, 64, 64, 130, 8950)
    out = torch.zeros((130, 40), dtype=torch.bfloat16, device=dev())
    with pytest.raises(vpq.VpqError):
        ops.qmm_swiglu_into(*d, out, 16)


# --------------------------------- fused stores of the small-batch and the group-32 GEMVs

def _stores_against_plain(ops, d, plain, M, N, kind, seed):
    """Every fused store of a GEMV against the same GEMV's plain output `plain` [M, N]."""
    aux = to_dev(synth.activations_bf16(M, N, seed), torch.bfloat16)
    z = lambda *shape: torch.full(shape, 1e30, dtype=torch.bfloat16, device=dev())  # no sum gets near it
    y = ops.qmv_w8_fused(*d, z(M, N), {"epilogue": "add", "aux": aux}, kind=kind)
    assert torch.equal(y, (plain.float() + aux.float()).to(torch.bfloat16))
    y = ops.qmv_w8_fused(*d, z(M, N), {"epilogue": "gelu_mul", "aux": aux}, kind=kind)
    sep = (_gelu_t(plain.float()) * aux.float()).to(torch.bfloat16)
    assert float((y == sep).float().mean()) > 0.98
    q_rows, k_rows = (N // 2) & ~1, N // 4
    yq, yk, yv = z(M, q_rows), z(M, k_rows), z(M, N - q_rows - k_rows)
    ops.qmv_w8_fused(*d, yq, {"epilogue": "qkv", "aux": yk, "y3": yv, "q_rows": q_rows, "k_rows": k_rows}, kind=kind)
    assert torch.equal(torch.cat([yq, yk, yv], dim=1), plain)
    g, u = plain.float()[:, 0::2], plain.float()[:, 1::2]
    for name, act in (("swiglu", lambda t: t / (1.0 + torch.exp(-t))), ("geglu", _gelu_t)):
        y = ops.qmv_w8_fused(*d, z(M, N // 2), {"epilogue": name}, kind=kind)
        assert torch.all(y.float().abs() < 1e29)  # every output written
        # the gated stores use the unrounded sums; against the bf16-rounded ones they agree to ~2 ulp
        e = y.float() - (act(g) * u)
        assert float(e.abs().max()) <= 2e-2 * float((act(g) * u).abs().max()) + 1e-6, name


@pytest.mark.parametrize("K,N,M", [(4096, 1024, 4), (1024, 96, 3), (2048, 40, 2)])
def test_qmv_batch_fused_stores(vpq, oracle_mod, K, N, M):
    """affine_qmv_batch_swiglu_w4g64 and the other stores on rows that share one weight stream."""
    d, _ = _linear(oracle_mod, N, K, M, 9600 + N + K)
    plain = vpq.ops.qmv_batch_rows(*d)
    _stores_against_plain(vpq.ops, d, plain, M, N, "batch", 9601 + N)


@pytest.mark.parametrize("K,N,M", [(4096, 1024, 2), (96, 34, 1), (1024, 64, 3)])
def test_qmv_w4g32_fused_stores(vpq, oracle_mod, K, N, M):
    """affine_qmv_w4g32_add, affine_qmv_geglu_w4g32, affine_qmv_gelu_mul_w4g32."""
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 9700 + N + K))
    codes, s16, b16 = oracle_mod.quant(wb, 4, 32)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, 9701 + N)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    plain = vpq.ops.qmv_g32(*d)
    _stores_against_plain(vpq.ops, d, plain, M, N, "g32", 9702 + N)


def _q40_linear(N, K, M, seed):
    """A GGUF Q4_0 repack as the reference's converter leaves it: nibbles 0..15, one scale per group of
    32 (either sign), bias = -8 * scale."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 2**32, size=(N, K // 8), dtype=np.uint64).astype(np.uint32)
    sf = (rng.standard_normal((N, K // 32)) * 0.02).astype(np.float32)
    s = synth.f32_to_bf16_bits(sf)
    b = synth.f32_to_bf16_bits(-8.0 * synth.bf16_bits_to_f32(s))   # exact
    x = synth.activations_bf16(M, K, seed + 1)
    return codes, s, b, x


@pytest.mark.parametrize("K,N,M", [(4096, 2048, 1), (4096, 1024, 2), (96, 34, 1), (1056, 66, 3), (11008, 256, 2)])
def test_qmv_w4g32_q40_scale_only(vpq, oracle_mod, K, N, M):
    """affine_qmv_w4g32_q40, _add_q40, geglu_w4g32_q40 (affine_qmv.metal:322-341,384-403,1472-1487): the
    bias buffer is not read; bit-identical to the group-32 GEMV given biases = -8 * scales, and within
    tolerance of the fp32 oracle."""
    from test_gpu_formats import _g32_reference
    ops = vpq.ops
    codes, s, b, x = _q40_linear(N, K, M, 9800 + N + K)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    q = (d[0], d[1], None, d[3])
    z = lambda *shape: torch.full(shape, float("nan"), dtype=torch.bfloat16, device=dev())
    plain = ops.qmv_g32(*d)
    y = ops.qmv_w8_fused(*q, z(M, N), {"epilogue": "none"}, kind="q40")
    assert torch.equal(y, plain)
    e = oracle_mod.err_metrics(f32(y), _g32_reference(oracle_mod, codes, s, b, x))
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, e
    aux = to_dev(synth.activations_bf16(M, N, 9801 + N), torch.bfloat16)
    for store in ({"epilogue": "add", "aux": aux}, {"epilogue": "geglu"}):
        width = N // 2 if store["epilogue"] == "geglu" else N
        want = ops.qmv_w8_fused(*d, z(M, width), store, kind="g32")
        got = ops.qmv_w8_fused(*q, z(M, width), store, kind="q40")
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got, want), store["epilogue"]
    # by the reference's names; slot 2 (biases) is left empty
    lib_name = "affine_qmv_bf16"
    y2 = z(M, N)
    ops.dispatch(ops.function(lib_name, "affine_qmv_w4g32_q40"), {0: d[0], 1: d[1], 3: d[3], 4: y2}, K=K, N=N, M=M)
    assert torch.equal(y2, plain)
    y2 = z(M, N)
    ops.dispatch(ops.function(lib_name, "affine_qmv_w4g32_add_q40"), {0: d[0], 1: d[1], 3: d[3], 4: y2, 7: aux},
                 K=K, N=N, M=M)
    assert torch.equal(y2, (plain.float() + aux.float()).to(torch.bfloat16))
    y2 = z(M, N // 2)
    ops.dispatch(ops.function(lib_name, "affine_qmv_geglu_w4g32_q40"), {0: d[0], 1: d[1], 3: d[3], 4: y2}, K=K, N=N, M=M)
    assert torch.equal(y2, ops.qmv_w8_fused(*d, z(M, N // 2), {"epilogue": "geglu"}, kind="g32"))


def test_qmv_w4g32_fused_names(vpq, oracle_mod):
    """affine_qmv_w4g32_add, affine_qmv_geglu_w4g32, affine_qmv_gelu_mul_w4g32, affine_qmv_qkv_w4g32 by name."""
    ops = vpq.ops
    K, N, M = 2048, 768, 2
    codes, s, b, x = _q40_linear(N, K, M, 9900)
    b = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(b) * 0.75)  # a general affine bias
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    aux = to_dev(synth.activations_bf16(M, N, 9901), torch.bfloat16)
    z = lambda *shape: torch.full(shape, float("nan"), dtype=torch.bfloat16, device=dev())
    lib_name = "affine_qmv_bf16"
    for name, store, width in (("affine_qmv_w4g32_add", {"epilogue": "add", "aux": aux}, N),
                               ("affine_qmv_geglu_w4g32", {"epilogue": "geglu"}, N // 2),
                               ("affine_qmv_gelu_mul_w4g32", {"epilogue": "gelu_mul", "aux": aux}, N)):
        want = ops.qmv_w8_fused(*d, z(M, width), store, kind="g32")
        got = z(M, width)
        bufs = {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: got}
        if "aux" in store:
            bufs[7] = aux
        ops.dispatch(ops.function(lib_name, name), bufs, K=K, N=N, M=M)
        assert torch.equal(got, want), name
    q_rows, k_rows = 512, 128
    yq, yk, yv = z(M, q_rows), z(M, k_rows), z(M, N - q_rows - k_rows)
    ops.dispatch(ops.function(lib_name, "affine_qmv_qkv_w4g32"),
                 {0: d[0], 1: d[1], 2: d[2], 3: d[3], 4: yq, 5: yk, 6: yv},
                 K=K, M=M, q_rows=q_rows, k_rows=k_rows, v_rows=N - q_rows - k_rows)
    assert torch.equal(torch.cat([yq, yk, yv], dim=1), ops.qmv_g32(*d))
