"""GPU tests of the decode-chain features of the 4-bit GEMV, through the C ABI, against the CPU
oracle: activations with a large dynamic range inside one row, the RMSNorm prologue
(affine_qmv_qkv_rms_w4g64, gpu-kernels/metal/quant/affine_qmv.metal:570-694), the mixture-of-experts
gather GEMVs (affine_gather_qmv_swiglu_w4g64 / affine_gather_down_qmv_w4g64 /
affine_gather_qmv_geglu_w4g64, affine_qmv.metal:908-955,1262-1291,1488-1521) and a dependent chain of
GEMVs in one launch (the analogue of one command buffer of dependent dispatches,
generative-models/qwen3/metal-qwen-model.cc:3004-3074). Tolerance 1e-2 as in test_gpu_parity.py."""
import numpy as np
import pytest
import torch

from vpipe_b200 import synth

from test_gpu_parity import TOL, bits16, dev, f32, quantized_linear, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(vpq):
    assert torch.cuda.is_available(), "the -m gpu tests need a CUDA device"
    torch.cuda.set_device(0)
    yield
    torch.cuda.synchronize()
    assert vpq.ops.device_status() == 0


def _outlier_x(K, log2_range, seed, n_out=3):
    """N(0,1) activations with a few elements 2^log2_range times larger (the massive activations of
    decoder residual streams), as bf16 bits."""
    rng = np.random.Generator(np.random.Philox(key=seed))
    x = rng.standard_normal((1, K)).astype(np.float32)
    pos = rng.choice(K, size=n_out, replace=False)
    x[0, pos] *= np.float32(2.0 ** log2_range)
    return synth.f32_to_bf16_bits(x), pos


@pytest.mark.parametrize("log2_range", [12, 16, 20])
@pytest.mark.parametrize("kind", ["qmv", "plan", "w8", "batch"])
def test_qmv_with_massive_activations_in_one_row(vpq, oracle_mod, kind, log2_range):
    """One row of x whose largest elements are 2^12 .. 2^20 times the typical one. The kernels turn
    x into fixed point with one power-of-two scale per 256-k (8-bit: 128-k) box, so only the box
    that holds the outlier shares its scale: the result must still meet the 1e-2 bars against the
    f64 dequantise-then-matmul oracle, and the part of the output that does not involve the
    outlier boxes must keep bf16-level accuracy."""
    ops = vpq.ops
    K, N = 4096, 1024
    xb, pos = _outlier_x(K, log2_range, 1700 + log2_range)
    if kind == "w8":
        w = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 1801))
        codes, s, b = oracle_mod.quant(w, 8, 64, True)
        s, b = oracle_mod.f16_to_bf16(s), oracle_mod.f16_to_bf16(b)
        deq = oracle_mod.bf16_to_f32(oracle_mod.dequant_bf16_any(codes, s, b, 8, 64)).astype(np.float64)
        # the oracle's dequantised weight is rounded to bf16; rebuild the unrounded f32 form
        q = codes.view(np.uint8).reshape(N, K).astype(np.float32)
        sf = np.repeat(oracle_mod.bf16_to_f32(s), 64, axis=1)
        bf = np.repeat(oracle_mod.bf16_to_f32(b), 64, axis=1)
        deq = (sf * q + bf).astype(np.float64)
    else:
        codes, s, b = quantized_linear(oracle_mod, N, K, 1800)
        deq = oracle_mod.dequant_f32(codes, s, b).astype(np.float64)
    xf = oracle_mod.bf16_to_f32(xb).astype(np.float64)
    ref = xf @ deq.T
    dc, ds, db = to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16)
    dx = to_dev(xb, torch.bfloat16)
    if kind == "qmv":
        y = ops.qmv(dc, ds, db, dx)
    elif kind == "w8":
        y = ops.qmv_w8(dc, ds, db, dx)
    elif kind == "plan":
        y = torch.zeros((1, N), dtype=torch.bfloat16, device=dev())
        plan = ops.QmvPlan([(dc, ds, db, dx, y)])
        plan.run()
        torch.cuda.synchronize()
        plan.close()
    else:
        x2 = torch.cat([dx, to_dev(synth.activations_bf16(1, K, 1900), torch.bfloat16)])
        y = ops.qmv_batch_rows(dc, ds, db, x2)[:1]
    e = oracle_mod.err_metrics(f32(y), ref.astype(np.float32))
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL, (kind, log2_range, e)
    # Without the outliers' own boxes the sum is an ordinary one: the kernel's error there must be
    # what f32 accumulation and the bf16 store leave, as if the outliers were not in the row.
    if kind in ("qmv", "plan", "w8"):
        box = 128 if kind == "w8" else 256
        keep = np.ones(K, bool)
        for p in pos:
            keep[(p // box) * box:(p // box + 1) * box] = False
        x_rest = xf.copy()
        x_rest[0, ~keep] = 0.0
        xr_bits = synth.f32_to_bf16_bits(x_rest.astype(np.float32))
        fn = ops.qmv_w8 if kind == "w8" else ops.qmv
        y_rest = fn(dc, ds, db, to_dev(xr_bits, torch.bfloat16))
        ref_rest = x_rest @ deq.T
        er = oracle_mod.err_metrics(f32(y_rest), ref_rest.astype(np.float32))
        assert er["max_rel_1e2"] < TOL, er
        # linearity: full = outlier boxes + rest, each computed by the kernel, to bf16 rounding of the parts
        x_out = xf.copy()
        x_out[0, keep] = 0.0
        y_out = fn(dc, ds, db, to_dev(synth.f32_to_bf16_bits(x_out.astype(np.float32)), torch.bfloat16))
        d = np.abs(f32(y) - (f32(y_out) + f32(y_rest)))
        assert np.all(d <= 2.0 ** -6 * (np.abs(f32(y_out)) + np.abs(f32(y_rest))) + 1e-6)


def _norm_weights(K, seed):
    rng = np.random.Generator(np.random.Philox(key=seed))
    return synth.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32))


@pytest.mark.parametrize("K,q_rows,k_rows,v_rows", [(4096, 4096, 1024, 1024), (2048, 256, 64, 72), (5120, 40, 8, 8)])
def test_qkv_with_rmsnorm_prologue(vpq, oracle_mod, K, q_rows, k_rows, v_rows):
    """q|k|v GEMV with the RMSNorm fused into the staging of x: equals the oracle's norm followed by
    the plain GEMV oracle; and equals this library's own q|k|v GEMV fed with the oracle's normed x
    except where the kernel's f32 sum of squares rounds 1/rms differently (rare, one bf16 ulp of x)."""
    ops = vpq.ops
    N = q_rows + k_rows + v_rows
    codes, s, b = quantized_linear(oracle_mod, N, K, 2100 + K)
    xb = synth.f32_to_bf16_bits(3.0 * synth.bf16_bits_to_f32(synth.activations_bf16(2, K, 2200 + K)))
    nw = _norm_weights(K, 2300 + K)
    eps = 1e-6
    xn = oracle_mod.rms_norm_bf16(xb, nw, eps)
    ref = oracle_mod.linear_f32(codes, s, b, xn, "f64")
    dc, ds, db = to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16)
    dx, dnw = to_dev(xb, torch.bfloat16), to_dev(nw, torch.bfloat16)
    q = torch.zeros((2, q_rows), dtype=torch.bfloat16, device=dev())
    k = torch.zeros((2, k_rows), dtype=torch.bfloat16, device=dev())
    v = torch.zeros((2, v_rows), dtype=torch.bfloat16, device=dev())
    store = {"epilogue": "qkv", "aux": k, "y3": v, "q_rows": q_rows, "k_rows": k_rows, "norm_w": dnw, "eps": eps}
    ops.qmv_batch(ops.qmv_set([(dc, ds, db, dx, q, store)]))
    torch.cuda.synchronize()
    got = np.concatenate([f32(q), f32(k), f32(v)], axis=1)
    e = oracle_mod.err_metrics(got, ref.astype(np.float32))
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL and e["max_rel_1e2"] < 2 * TOL, e
    plain = ops.qmv_qkv(dc, ds, db, to_dev(xn, torch.bfloat16), q_rows, k_rows, v_rows)
    same = np.mean(np.concatenate([bits16(t) for t in plain], axis=1) == np.concatenate(
        [bits16(q), bits16(k), bits16(v)], axis=1))
    assert same > 0.98
    # by the reference's (library, entry) name and slot numbers
    q2, k2, v2 = torch.zeros_like(q[:1]), torch.zeros_like(k[:1]), torch.zeros_like(v[:1])
    fn = ops.function("affine_qmv_bf16", "affine_qmv_qkv_rms_w4g64")
    assert fn
    ops.dispatch(fn, [dc, ds, db, dx[:1], dnw, q2, k2, v2], K=K, q_rows=q_rows, k_rows=k_rows, v_rows=v_rows, eps=eps)
    torch.cuda.synchronize()
    assert torch.equal(q2, q[:1]) and torch.equal(k2, k[:1]) and torch.equal(v2, v[:1])


def _expert_weights(oracle_mod, E, N, K, seed):
    cs, ss, bs = [], [], []
    for e in range(E):
        c, s, b = quantized_linear(oracle_mod, N, K, seed + e)
        cs.append(c)
        ss.append(s)
        bs.append(b)
    return np.stack(cs), np.stack(ss), np.stack(bs)


@pytest.mark.parametrize("act", ["swiglu", "geglu"])
def test_moe_gather_gemvs_match_the_oracle_pair_by_pair(vpq, oracle_mod, act):
    """Decode of a mixture of experts: for pair p = (token p // top_k, expert pair_eid[p]) the gate|up
    GEMV with the gated store over the routed expert's slab, then the down GEMV on the pair's own
    activation row. The expert index is read on the GPU. Each pair is checked against the oracle on
    that expert's slab, and against this library's plain GEMV on the same slab (bit-identical, as the
    reference's gathered kernels are token-exact with its plain ones)."""
    ops = vpq.ops
    E, H, F, T, top_k = 6, 1024, 384, 2, 3
    gu = _expert_weights(oracle_mod, E, 2 * F, H, 3100)
    dn = _expert_weights(oracle_mod, E, H, F, 3200)
    xb = synth.activations_bf16(T, H, 3300)
    eid = np.array([4, 0, 5, 2, 2, 1], np.int32)       # [T * top_k]
    npair = T * top_k
    d_gu = [to_dev(gu[0]), to_dev(gu[1], torch.bfloat16), to_dev(gu[2], torch.bfloat16)]
    d_dn = [to_dev(dn[0]), to_dev(dn[1], torch.bfloat16), to_dev(dn[2], torch.bfloat16)]
    dx = to_dev(xb, torch.bfloat16)
    deid = torch.from_numpy(eid).to(dev())
    a = torch.zeros((npair, F), dtype=torch.bfloat16, device=dev())
    part = torch.zeros((npair, H), dtype=torch.bfloat16, device=dev())
    ops.qmv_batch(ops.qmv_set([(d_gu[0], d_gu[1], d_gu[2], dx, a,
                                {"epilogue": act, "expert": deid, "x_div": top_k, "M": npair})]))
    ops.qmv_batch(ops.qmv_set([(d_dn[0], d_dn[1], d_dn[2], a, part, {"expert": deid, "M": npair})]))
    torch.cuda.synchronize()
    fuse = oracle_mod.fused_swiglu if act == "swiglu" else oracle_mod.fused_geglu
    for p in range(npair):
        e, t = int(eid[p]), p // top_k
        ref_a = fuse(oracle_mod.linear_f32(gu[0][e], gu[1][e], gu[2][e], xb[t:t + 1], "f64").astype(np.float32))
        got_a = f32(a[p:p + 1])
        ea = oracle_mod.err_metrics(got_a, synth.bf16_bits_to_f32(ref_a) if ref_a.dtype == np.uint16 else ref_a)
        assert ea["rel_l2"] < TOL and ea["max_rel_rms"] < TOL, (p, ea)
        plain_a = ops.qmv_swiglu(d_gu[0][e], d_gu[1][e], d_gu[2][e], dx[t:t + 1], act=act)
        assert torch.equal(plain_a, a[p:p + 1])
        ref_d = oracle_mod.linear_f32(dn[0][e], dn[1][e], dn[2][e], bits16(a[p:p + 1]), "f64")
        ed = oracle_mod.err_metrics(f32(part[p:p + 1]), ref_d.astype(np.float32))
        assert ed["rel_l2"] < TOL and ed["max_rel_rms"] < TOL, (p, ed)
        assert torch.equal(ops.qmv(d_dn[0][e], d_dn[1][e], d_dn[2][e], a[p:p + 1]), part[p:p + 1])
    # by the reference's names and slots (slot 7 = pair_eid, top_k as a constant)
    a2, part2 = torch.zeros_like(a), torch.zeros_like(part)
    fn = ops.function("affine_qmv_bf16", f"affine_gather_qmv_{act}_w4g64")
    ops.dispatch(fn, {0: d_gu[0], 1: d_gu[1], 2: d_gu[2], 3: dx, 4: a2, 7: deid}, K=H, N=2 * F, M=npair,
                 experts=E, top_k=top_k)
    fn = ops.function("affine_qmv_bf16", "affine_gather_down_qmv_w4g64")
    ops.dispatch(fn, {0: d_dn[0], 1: d_dn[1], 2: d_dn[2], 3: a2, 4: part2, 7: deid}, K=F, N=H, M=npair, experts=E)
    torch.cuda.synchronize()
    assert torch.equal(a2, a) and torch.equal(part2, part)


def _decoder_layers(vpq, oracle_mod, layers, H, KV, F, seed):
    """Weights of `layers` decoder layers (q|k|v, o, gate|up interleaved, down) and the chain of
    fused GEMVs a decode step issues per layer: norm + q|k|v, o_proj + residual, norm + gate|up with
    SwiGLU, down + residual; every GEMV reads what the one before wrote (attention itself is not
    part of this path: o_proj reads the q output)."""
    L = []
    h0 = to_dev(synth.activations_bf16(1, H, seed), torch.bfloat16)
    x = h0
    for i in range(layers):
        ws = []
        for j, (n, k) in enumerate([(H + 2 * KV, H), (H, H), (2 * F, H), (H, F)]):
            c, s, b = quantized_linear(oracle_mod, n, k, seed + 10 * i + j + 1)
            ws.append((to_dev(c), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16)))
        nw1 = to_dev(_norm_weights(H, seed + 100 + i), torch.bfloat16)
        nw2 = to_dev(_norm_weights(H, seed + 200 + i), torch.bfloat16)
        q, k, v, h1, act, h2 = (torch.zeros((1, n), dtype=torch.bfloat16, device=dev()) for n in (H, KV, KV, H, F, H))
        dep = i > 0
        L.append([
            ws[0] + (x, q, {"epilogue": "qkv", "aux": k, "y3": v, "q_rows": H, "k_rows": KV, "norm_w": nw1,
                            "eps": 1e-6, "depends": dep}),
            ws[1] + (q, h1, {"epilogue": "add", "aux": x, "depends": True}),
            ws[2] + (h1, act, {"epilogue": "swiglu", "norm_w": nw2, "eps": 1e-6, "depends": True}),
            ws[3] + (act, h2, {"epilogue": "add", "aux": h1, "depends": True}),
        ])
        x = h2
    return L, x


@pytest.mark.parametrize("H,KV,F,layers", [(1024, 256, 1536, 3), (4096, 1024, 12288, 2)])
def test_dependent_chain_in_one_launch_equals_launch_per_gemv(vpq, oracle_mod, H, KV, F, layers):
    """All GEMVs of several decoder layers as ONE launch in which each waits for its predecessors:
    the bytes must equal those of the same GEMVs launched one by one, on every run."""
    ops = vpq.ops
    L, out = _decoder_layers(vpq, oracle_mod, layers, H, KV, F, 4000 + H)
    problems = [p for layer in L for p in layer]
    for p in problems:          # launch per GEMV (the "depends" mark is a plan-only field)
        plain = dict(p[5])
        plain.pop("depends")
        ops.qmv_batch(ops.qmv_set([p[:5] + (plain,)]))
    torch.cuda.synchronize()
    want = [t.clone() for p in problems for t in ([p[4]] + ([p[5]["aux"], p[5]["y3"]] if p[5]["epilogue"] == "qkv" else []))]
    assert float(out.float().abs().max()) > 0
    plan = ops.QmvPlan(problems)
    for run in range(3):
        for p in problems:
            p[4].fill_(7.0)
        plan.run()
        torch.cuda.synchronize()
        got = [t for p in problems for t in ([p[4]] + ([p[5]["aux"], p[5]["y3"]] if p[5]["epilogue"] == "qkv" else []))]
        for i, (g, w) in enumerate(zip(got, want)):
            assert torch.equal(g, w), f"run {run}: output {i} differs"
    plan.close()
    assert ops.device_status() == 0


def test_chain_first_layer_against_oracle(vpq, oracle_mod):
    """The chained launch against the CPU oracle, GEMV by GEMV, on one small layer."""
    ops = vpq.ops
    H, KV, F = 512, 128, 768
    L, out = _decoder_layers(vpq, oracle_mod, 1, H, KV, F, 5000)
    plan = ops.QmvPlan(L[0])
    plan.run()
    torch.cuda.synchronize()
    plan.close()
    (qkv, o, gu, dn) = L[0]
    host = lambda t: bits16(t) if t.dtype == torch.bfloat16 else t.cpu().numpy().view(np.uint32)  # noqa: E731
    x0 = host(qkv[3])
    xn = oracle_mod.rms_norm_bf16(x0, host(qkv[5]["norm_w"]), 1e-6)
    r_qkv = oracle_mod.linear_f32(host(qkv[0]), host(qkv[1]), host(qkv[2]), xn, "f64").astype(np.float32)
    got_qkv = np.concatenate([f32(qkv[4]), f32(qkv[5]["aux"]), f32(qkv[5]["y3"])], axis=1)
    assert oracle_mod.err_metrics(got_qkv, r_qkv)["max_rel_rms"] < TOL
    r_o = oracle_mod.fused_add(
        oracle_mod.linear_f32(host(o[0]), host(o[1]), host(o[2]), host(qkv[4]), "f64").astype(np.float32), x0)
    assert oracle_mod.err_metrics(f32(o[4]), synth.bf16_bits_to_f32(r_o))["max_rel_rms"] < TOL
    hn = oracle_mod.rms_norm_bf16(host(o[4]), host(gu[5]["norm_w"]), 1e-6)
    r_gu = oracle_mod.fused_swiglu(
        oracle_mod.linear_f32(host(gu[0]), host(gu[1]), host(gu[2]), hn, "f64").astype(np.float32))
    assert oracle_mod.err_metrics(f32(gu[4]), synth.bf16_bits_to_f32(r_gu))["max_rel_rms"] < TOL
    r_dn = oracle_mod.fused_add(
        oracle_mod.linear_f32(host(dn[0]), host(dn[1]), host(dn[2]), host(gu[4]), "f64").astype(np.float32), host(o[4]))
    assert oracle_mod.err_metrics(f32(dn[4]), synth.bf16_bits_to_f32(r_dn))["max_rel_rms"] < TOL


def test_chain_over_buffers_that_the_layers_reuse(vpq, oracle_mod):
    """A decoder keeps one set of activation buffers for all layers: the residual stream ping-pongs
    between two vectors and q | k | v | act are overwritten by every layer. Inside one chained launch
    an SM then reads addresses it has read before with other contents (x, the residual); the bytes
    must still equal those of one launch per GEMV."""
    ops = vpq.ops
    H, KV, F, layers = 1024, 256, 1536, 6
    L, _ = _decoder_layers(vpq, oracle_mod, layers, H, KV, F, 4700)
    h0 = L[0][0][3].clone()
    a, b = torch.zeros_like(h0), torch.zeros_like(h0)
    q, k, v, act = (torch.zeros((1, n), dtype=torch.bfloat16, device=dev()) for n in (H, KV, KV, F))
    problems = []
    for i, (qkv, o, gu, dn) in enumerate(L):
        problems += [
            qkv[:3] + (a, q, dict(qkv[5], aux=k, y3=v, depends=i > 0)),
            o[:3] + (q, b, dict(o[5], aux=a)),
            gu[:3] + (b, act, dict(gu[5])),
            dn[:3] + (act, a, dict(dn[5], aux=b)),
        ]
    outs = [a, b, q, k, v, act]
    a.copy_(h0)
    _per_launch(ops, problems)
    torch.cuda.synchronize()
    want = [t.clone() for t in outs]
    assert float(want[0].float().abs().max()) > 0
    plan = ops.QmvPlan(problems)
    for run in range(4):
        for t in outs:
            t.fill_(5.0)
        a.copy_(h0)
        plan.run()
        torch.cuda.synchronize()
        for i, (g, w) in enumerate(zip(outs, want)):
            assert torch.equal(g, w), f"run {run}: buffer {i} differs"
    plan.close()
    assert ops.device_status() == 0


def _chain_outputs(problems):
    return [t for p in problems for t in ([p[4]] + ([p[5]["aux"], p[5]["y3"]] if p[5]["epilogue"] == "qkv" else []))]


def _per_launch(ops, problems):
    for p in problems:
        plain = dict(p[5])
        plain.pop("depends", None)
        ops.qmv_batch(ops.qmv_set([p[:5] + (plain,)]))


def test_chain_with_an_input_that_is_no_first_output_and_replayed_from_a_graph(vpq, oracle_mod):
    """A chained plan in which one GEMV reads the k output of a q|k|v GEMV (not a first output: it
    waits on the plan's tile counter while the others poll tagged words), run directly, re-created in
    the same workspace, and replayed from a CUDA graph with the layer input changed between replays.
    Every run must give the bytes of the same GEMVs launched one by one on that input."""
    ops = vpq.ops
    H, KV, F = 1024, 256, 1536
    L, out = _decoder_layers(vpq, oracle_mod, 2, H, KV, F, 6100)
    problems = [p for layer in L for p in layer]
    c, s, b = quantized_linear(oracle_mod, 528, KV, 6177)
    side_y = torch.zeros((1, 528), dtype=torch.bfloat16, device=dev())
    side = (to_dev(c), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), L[0][0][5]["aux"], side_y,
            {"epilogue": "none", "depends": True})
    problems.insert(2, side)
    h0 = L[0][0][3]
    inputs = [to_dev(synth.activations_bf16(1, H, 6200 + i), torch.bfloat16) for i in range(3)]

    def reference(x):
        h0.copy_(x)
        _per_launch(ops, problems)
        torch.cuda.synchronize()
        return [t.clone() for t in _chain_outputs(problems)]

    def check(x, run_it, what):
        want = reference(x)
        for t in _chain_outputs(problems):
            t.fill_(7.0)
        run_it()
        torch.cuda.synchronize()
        for i, (g, w) in enumerate(zip(_chain_outputs(problems), want)):
            assert torch.equal(g, w), f"{what}: output {i} differs"

    plan = ops.QmvPlan(problems)
    for i in (0, 1, 0):
        check(inputs[i], plan.run, f"direct run, input {i}")
    # the same workspace, a plan over a different list first, then this one again
    ws = plan.workspace
    plan.close()
    other = ops.QmvPlan(problems[:5], workspace=ws)
    other.run()
    torch.cuda.synchronize()
    other.close()
    plan = ops.QmvPlan(problems, workspace=ws)
    check(inputs[2], plan.run, "plan re-created in its old workspace")
    side_stream = torch.cuda.Stream()
    side_stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side_stream):
        plan.run()
    torch.cuda.current_stream().wait_stream(side_stream)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        plan.run()
    for i in (1, 2, 0, 1):
        check(inputs[i], g.replay, f"graph replay, input {i}")
    plan.close()
    assert ops.device_status() == 0


@pytest.mark.parametrize("act", ["swiglu", "geglu"])
def test_moe_gather_gemvs_over_8_bit_experts(vpq, oracle_mod, act):
    """affine_gather_qmv_swiglu_w8g64 / _geglu_w8g64 / affine_gather_down_qmv_w8g64
    (affine_qmv.metal:957-994,1290-1322,1519-1548), by the reference's names and slots: every pair
    bit-identical to this library's plain 8-bit GEMV on the routed expert's slab (the reference's
    gathered kernels are token-exact with its plain ones) and within tolerance of the fp32 oracle."""
    from test_gpu_formats import _w8_reference
    ops = vpq.ops
    E, H, F, T, top_k = 5, 1024, 320, 2, 2
    def experts(N, K, seed):
        cs, ss, bs = [], [], []
        for e in range(E):
            wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, seed + e))
            c, s16, b16 = oracle_mod.quant(wb, 8, 64)
            cs.append(c), ss.append(oracle_mod.f16_to_bf16(s16)), bs.append(oracle_mod.f16_to_bf16(b16))
        return np.stack(cs), np.stack(ss), np.stack(bs)
    gu, dn = experts(2 * F, H, 3500), experts(H, F, 3600)
    xb = synth.activations_bf16(T, H, 3700)
    eid = np.array([3, 0, 4, 4], np.int32)
    npair = T * top_k
    d_gu = [to_dev(gu[0]), to_dev(gu[1], torch.bfloat16), to_dev(gu[2], torch.bfloat16)]
    d_dn = [to_dev(dn[0]), to_dev(dn[1], torch.bfloat16), to_dev(dn[2], torch.bfloat16)]
    dx, deid = to_dev(xb, torch.bfloat16), torch.from_numpy(eid).to(dev())
    a = torch.full((npair, F), float("nan"), dtype=torch.bfloat16, device=dev())
    part = torch.full((npair, H), float("nan"), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmv_bf16", f"affine_gather_qmv_{act}_w8g64"),
                 {0: d_gu[0], 1: d_gu[1], 2: d_gu[2], 3: dx, 4: a, 7: deid}, K=H, N=2 * F, M=npair, experts=E, top_k=top_k)
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_gather_down_qmv_w8g64"),
                 {0: d_dn[0], 1: d_dn[1], 2: d_dn[2], 3: a, 4: part, 7: deid}, K=F, N=H, M=npair, experts=E)
    torch.cuda.synchronize()
    assert not torch.isnan(a.float()).any() and not torch.isnan(part.float()).any()
    fuse = oracle_mod.fused_swiglu if act == "swiglu" else oracle_mod.fused_geglu
    for p in range(npair):
        e, t = int(eid[p]), p // top_k
        plain_a = ops.qmv_w8_fused(d_gu[0][e], d_gu[1][e], d_gu[2][e], dx[t:t + 1],
                                   torch.zeros((1, F), dtype=torch.bfloat16, device=dev()), {"epilogue": act})
        assert torch.equal(plain_a, a[p:p + 1]), p
        ref_a = fuse(_w8_reference(oracle_mod, gu[0][e], gu[1][e], gu[2][e], xb[t:t + 1], "f64").astype(np.float32))
        ea = oracle_mod.err_metrics(f32(a[p:p + 1]), synth.bf16_bits_to_f32(ref_a))
        assert ea["rel_l2"] < TOL and ea["max_rel_rms"] < TOL, (p, ea)
        assert torch.equal(ops.qmv_w8(d_dn[0][e], d_dn[1][e], d_dn[2][e], a[p:p + 1]), part[p:p + 1]), p
        ref_d = _w8_reference(oracle_mod, dn[0][e], dn[1][e], dn[2][e], bits16(a[p:p + 1]), "f64")
        ed = oracle_mod.err_metrics(f32(part[p:p + 1]), ref_d.astype(np.float32))
        assert ed["rel_l2"] < TOL and ed["max_rel_rms"] < TOL, (p, ed)
    assert ops.device_status() == 0


@pytest.mark.parametrize("K,M", [(2048, 1), (4096, 5), (64, 3), (3136, 2)])
def test_moe_shared_expert_gate(vpq, oracle_mod, K, M):
    """affine_moe_gate_w8g64 (affine_qmv.metal:1323-1347): sigmoid of one 8-bit row's dot product with
    every row of x, against the fp32 oracle (f64 accumulation), and by the reference's name."""
    from test_gpu_formats import _w8_reference
    wb = synth.f32_to_bf16_bits(synth.weight_f32(1, K, 3900 + K) * 3.0)
    codes, s16, b16 = oracle_mod.quant(wb, 8, 64)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    x = synth.activations_bf16(M, K, 3901 + K)
    d = (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16), to_dev(x, torch.bfloat16))
    got = vpq.ops.moe_gate_w8(*d)
    logit = _w8_reference(oracle_mod, codes, s, b, x, "f64").astype(np.float64).reshape(M)
    want = 1.0 / (1.0 + np.exp(-logit))
    assert float(np.abs(want - 0.5).max()) > 0.05           # the logits are not all near zero
    assert np.abs(got.float().cpu().numpy().astype(np.float64) - want).max() < 1e-2 * 0.5 + 2.0 ** -8
    out = torch.full((M,), float("nan"), dtype=torch.bfloat16, device=dev())
    vpq.ops.dispatch(vpq.ops.function("affine_qmv_bf16", "affine_moe_gate_w8g64"), [d[0], d[1], d[2], d[3], out], K=K, M=M)
    assert torch.equal(out, got)


@pytest.mark.parametrize("gate_bits", [4, 8])
def test_moe_gather_swiglu_with_gate_and_up_of_different_widths(vpq, oracle_mod, gate_bits):
    """affine_gather_qmv_swiglu_w4w8g64 / _w8w4g64 (affine_qmv.metal:1153-1259): separate gate and up
    matrices, one at 4 and one at 8 bits, per routed pair; against the fp32 oracle of silu(gate) * up."""
    from test_gpu_formats import _w8_reference
    ops = vpq.ops
    E, H, F, T, top_k = 4, 1024, 256, 2, 2
    up_bits = 12 - gate_bits

    def experts(bits, seed):
        cs, ss, bs = [], [], []
        for e in range(E):
            wb = synth.f32_to_bf16_bits(synth.weight_f32(F, H, seed + e))
            c, s16, b16 = oracle_mod.quant(wb, bits, 64)
            cs.append(c), ss.append(oracle_mod.f16_to_bf16(s16)), bs.append(oracle_mod.f16_to_bf16(b16))
        return np.stack(cs), np.stack(ss), np.stack(bs)

    def linear(w, bits, e, xrow):
        if bits == 8:
            return _w8_reference(oracle_mod, w[0][e], w[1][e], w[2][e], xrow, "f64").astype(np.float64)
        return oracle_mod.linear_f32(w[0][e], w[1][e], w[2][e], xrow, "f64").astype(np.float64)

    g, u = experts(gate_bits, 4100), experts(up_bits, 4200)
    xb = synth.activations_bf16(T, H, 4300)
    eid = np.array([2, 0, 3, 1], np.int32)
    npair = T * top_k
    dg = [to_dev(g[0]), to_dev(g[1], torch.bfloat16), to_dev(g[2], torch.bfloat16)]
    du = [to_dev(u[0]), to_dev(u[1], torch.bfloat16), to_dev(u[2], torch.bfloat16)]
    dx, deid = to_dev(xb, torch.bfloat16), torch.from_numpy(eid).to(dev())
    y = torch.full((npair, F), float("nan"), dtype=torch.bfloat16, device=dev())
    name = "affine_gather_qmv_swiglu_w4w8g64" if gate_bits == 4 else "affine_gather_qmv_swiglu_w8w4g64"
    ops.dispatch(ops.function("affine_qmv_bf16", name),
                 {0: dg[0], 1: dg[1], 2: dg[2], 3: du[0], 4: du[1], 5: du[2], 6: dx, 7: y, 10: deid},
                 K=H, N=F, M=npair, experts=E, top_k=top_k)
    torch.cuda.synchronize()
    assert not torch.isnan(y.float()).any()
    for p in range(npair):
        e, t = int(eid[p]), p // top_k
        gv, uv = linear(g, gate_bits, e, xb[t:t + 1]), linear(u, up_bits, e, xb[t:t + 1])
        want = (gv / (1.0 + np.exp(-gv)) * uv).astype(np.float32)
        err = oracle_mod.err_metrics(f32(y[p:p + 1]), want)
        assert err["rel_l2"] < TOL and err["max_rel_rms"] < TOL, (p, err)
    assert ops.device_status() == 0


@pytest.mark.parametrize("K,q_rows,k_rows,v_rows", [(4096, 2048, 512, 512), (1024, 128, 32, 40), (3136, 48, 16, 16)])
def test_qkv_with_rmsnorm_prologue_over_8_bit_weights(vpq, oracle_mod, K, q_rows, k_rows, v_rows):
    """affine_qmv_qkv_rms_w8g64 (the 8-bit instantiation of affine_qmv.metal:570-694) by the reference's
    name and slots: the oracle's RMSNorm followed by the 8-bit GEMV oracle; and the library's own 8-bit
    q|k|v GEMV on the oracle's normed x, equal except where 1/rms rounds differently (one bf16 ulp of x)."""
    from test_gpu_formats import _w8_reference
    ops = vpq.ops
    N = q_rows + k_rows + v_rows
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 2500 + K))
    codes, s16, b16 = oracle_mod.quant(wb, 8, 64)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    xb = synth.f32_to_bf16_bits(3.0 * synth.bf16_bits_to_f32(synth.activations_bf16(1, K, 2600 + K)))
    nw = _norm_weights(K, 2700 + K)
    eps = 1e-6
    xn = oracle_mod.rms_norm_bf16(xb, nw, eps)
    ref = _w8_reference(oracle_mod, codes, s, b, xn, "f64")
    dc, ds, db = to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16)
    dx, dnw = to_dev(xb, torch.bfloat16), to_dev(nw, torch.bfloat16)
    z = lambda n: torch.full((1, n), float("nan"), dtype=torch.bfloat16, device=dev())  # noqa: E731
    q, k, v = z(q_rows), z(k_rows), z(v_rows)
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_qkv_rms_w8g64"), [dc, ds, db, dx, dnw, q, k, v],
                 K=K, q_rows=q_rows, k_rows=k_rows, v_rows=v_rows, eps=eps)
    torch.cuda.synchronize()
    got = np.concatenate([f32(q), f32(k), f32(v)], axis=1)
    assert not np.isnan(got).any()
    e = oracle_mod.err_metrics(got, ref.astype(np.float32))
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL and e["max_rel_1e2"] < 2 * TOL, e
    pq, pk, pv = z(q_rows), z(k_rows), z(v_rows)
    ops.qmv_w8_fused(dc, ds, db, to_dev(xn, torch.bfloat16), pq,
                     {"epilogue": "qkv", "aux": pk, "y3": pv, "q_rows": q_rows, "k_rows": k_rows})
    same = np.mean(np.concatenate([bits16(t) for t in (pq, pk, pv)], axis=1) == np.concatenate(
        [bits16(q), bits16(k), bits16(v)], axis=1))
    assert same > 0.98
    assert ops.device_status() == 0


@pytest.mark.parametrize("K,q_rows,k_rows,v_rows,M", [(4096, 2048, 512, 512, 1), (1024, 128, 32, 40, 2), (2080, 48, 16, 16, 1)])
def test_qkv_with_rmsnorm_prologue_over_group_32_weights(vpq, oracle_mod, K, q_rows, k_rows, v_rows, M):
    """affine_qmv_qkv_rms_w4g32 (the group-32 instantiation of affine_qmv.metal:570-694) by the
    reference's name and slots, and the same prologue on rows that share one weight stream: the oracle's
    RMSNorm followed by the group-32 GEMV oracle."""
    from test_gpu_formats import _g32_reference
    ops = vpq.ops
    N = q_rows + k_rows + v_rows
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 2800 + K))
    codes, s16, b16 = oracle_mod.quant(wb, 4, 32)
    s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
    xb = synth.f32_to_bf16_bits(3.0 * synth.bf16_bits_to_f32(synth.activations_bf16(M, K, 2900 + K)))
    nw = _norm_weights(K, 3000 + K)
    eps = 1e-6
    xn = np.concatenate([oracle_mod.rms_norm_bf16(xb[m:m + 1], nw, eps) for m in range(M)])
    ref = _g32_reference(oracle_mod, codes, s, b, xn, "f64")
    dc, ds, db = to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16)
    dx, dnw = to_dev(xb, torch.bfloat16), to_dev(nw, torch.bfloat16)
    z = lambda n: torch.full((M, n), float("nan"), dtype=torch.bfloat16, device=dev())  # noqa: E731
    q, k, v = z(q_rows), z(k_rows), z(v_rows)
    ops.dispatch(ops.function("affine_qmv_bf16", "affine_qmv_qkv_rms_w4g32"), [dc, ds, db, dx, dnw, q, k, v],
                 K=K, M=M, q_rows=q_rows, k_rows=k_rows, v_rows=v_rows, eps=eps)
    torch.cuda.synchronize()
    got = np.concatenate([f32(q), f32(k), f32(v)], axis=1)
    assert not np.isnan(got).any()
    e = oracle_mod.err_metrics(got, ref.astype(np.float32))
    assert e["rel_l2"] < TOL and e["max_rel_rms"] < TOL and e["max_rel_1e2"] < 2 * TOL, e
    pq, pk, pv = z(q_rows), z(k_rows), z(v_rows)
    ops.qmv_w8_fused(dc, ds, db, to_dev(xn, torch.bfloat16), pq,
                     {"epilogue": "qkv", "aux": pk, "y3": pv, "q_rows": q_rows, "k_rows": k_rows}, kind="g32")
    same = np.mean(np.concatenate([bits16(t) for t in (pq, pk, pv)], axis=1) == np.concatenate(
        [bits16(q), bits16(k), bits16(v)], axis=1))
    assert same > 0.98
    assert ops.device_status() == 0


@pytest.mark.parametrize("bits", [4, 8])
def test_moe_sorted_slot_gemvs(vpq, oracle_mod, bits):
    """affine_grouped_swiglu_w4g64 / affine_grouped_down_w4g64 and their _w8g64 twins
    (affine_qmv.metal:2551-2719): (token, expert) pairs sorted by expert into tiles of two slots; the
    gate|up GEMV gathers its x rows through srow, the down GEMV reads the sorted activations by slot;
    padding slots and tiles without an expert are not written. Every live slot bit-identical to the
    plain GEMV on its expert's slab."""
    from vpipe_b200 import moe
    ops = vpq.ops
    E, H, F, T, top_k = 5, 1024, 320, 3, 2

    def experts(N, K, seed):
        cs, ss, bs = [], [], []
        for e in range(E):
            if bits == 4:
                c, s, b = quantized_linear(oracle_mod, N, K, seed + e)
            else:
                c, s16, b16 = oracle_mod.quant(synth.f32_to_bf16_bits(synth.weight_f32(N, K, seed + e)), 8, 64)
                s, b = oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)
            cs.append(c), ss.append(s), bs.append(b)
        return [to_dev(np.stack(cs)), to_dev(np.stack(ss), torch.bfloat16), to_dev(np.stack(bs), torch.bfloat16)]

    gu, dn = experts(2 * F, H, 4500), experts(H, F, 4600)
    xb = to_dev(synth.activations_bf16(T, H, 4700), torch.bfloat16)
    eid = np.array([4, 0, 4, 2, 4, 1], np.int32)                  # expert 4 gets three pairs: one padding slot
    tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, 2)
    tile2e = np.concatenate([tile2e, np.array([-1], np.int32)])    # plus a tile without an expert
    srow = np.concatenate([srow, np.array([0, 1], np.int32)])
    npad += 2
    dt, ds = to_dev(tile2e), to_dev(srow)
    sfx = "w4g64" if bits == 4 else "w8g64"
    act = torch.full((npad, F), float("nan"), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmv_bf16", f"affine_grouped_swiglu_{sfx}"),
                 {0: gu[0], 1: gu[1], 2: gu[2], 3: xb, 4: act, 7: ds, 8: dt}, K=H, N=2 * F, M=npad, experts=E)
    y = torch.full((npad, H), float("nan"), dtype=torch.bfloat16, device=dev())
    act_in = torch.nan_to_num(act, nan=0.0)                       # the dead slots' rows are read but never used
    ops.dispatch(ops.function("affine_qmv_bf16", f"affine_grouped_down_{sfx}"),
                 {0: dn[0], 1: dn[1], 2: dn[2], 3: act_in, 4: y, 7: ds, 8: dt}, K=F, N=H, M=npad, experts=E)
    torch.cuda.synchronize()
    live = 0
    for slot in range(npad):
        e, r = int(tile2e[slot // 2]), int(srow[slot])
        if e < 0 or r < 0:
            assert torch.isnan(act[slot].float()).all() and torch.isnan(y[slot].float()).all(), slot
            continue
        live += 1
        zf = torch.zeros((1, F), dtype=torch.bfloat16, device=dev())
        if bits == 4:
            want_a = ops.qmv_swiglu(gu[0][e], gu[1][e], gu[2][e], xb[r:r + 1])
            want_y = ops.qmv(dn[0][e], dn[1][e], dn[2][e], act[slot:slot + 1])
        else:
            want_a = ops.qmv_w8_fused(gu[0][e], gu[1][e], gu[2][e], xb[r:r + 1], zf, {"epilogue": "swiglu"})
            want_y = ops.qmv_w8(dn[0][e], dn[1][e], dn[2][e], act[slot:slot + 1])
        assert torch.equal(act[slot:slot + 1], want_a), slot
        assert torch.equal(y[slot:slot + 1], want_y), slot
    assert live == eid.size
    assert ops.device_status() == 0
