"""Grouped (mixture-of-experts) GEMMs: affine_qmm_grouped_swiglu_w4g64 (gate|up, rows gathered from
the hidden through srow), affine_qmm_grouped_geglu_w4g64, affine_qmm_grouped_w4g64 (down, rows
scattered through sdst), affine_qmm_steel.metal:1026-1176,1186-1288,1371-1440. Checked pair by pair
against the ungrouped entry points run on each expert's own rows, and against the oracle."""
import numpy as np
import pytest
import torch

from vpipe_b200 import moe, synth

from test_gpu_parity import TOL, dev, f32, quantized_linear, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(vpq):
    assert torch.cuda.is_available(), "the -m gpu tests need a CUDA device"
    torch.cuda.set_device(0)
    yield
    torch.cuda.synchronize()
    assert vpq.ops.device_status() == 0


def _experts(oracle_mod, E, N, K, seed):
    per = [quantized_linear(oracle_mod, N, K, seed + 17 * e) for e in range(E)]
    codes = np.stack([p[0] for p in per])
    s = np.stack([p[1] for p in per])
    b = np.stack([p[2] for p in per])
    return per, (to_dev(codes), to_dev(s, torch.bfloat16), to_dev(b, torch.bfloat16))


def _routing(T, E, top_k, seed, idle=()):
    """top_k distinct experts per token, skewed so that block sizes differ; `idle` experts get none."""
    rng = np.random.default_rng(seed)
    live = [e for e in range(E) if e not in idle]
    p = rng.random(len(live)) ** 2 + 0.05
    p /= p.sum()
    eid = np.stack([rng.choice(live, size=top_k, replace=False, p=p) for _ in range(T)]).reshape(-1)
    return eid.astype(np.int32)


@pytest.mark.parametrize("act", ["swiglu", "geglu"])
@pytest.mark.parametrize("T,E,top_k,K,N", [(96, 4, 2, 512, 512), (300, 8, 2, 1024, 2 * 384), (33, 3, 1, 64, 34)])
def test_grouped_gate_up_gathers_rows_and_matches_per_expert_calls(vpq, oracle_mod, act, T, E, top_k, K, N):
    ops = vpq.ops
    tile = ops.qmm_grouped_tile_rows()
    per, d = _experts(oracle_mod, E, N, K, 9100 + T + K)
    x = synth.activations_bf16(T, K, 9101 + T)
    dx = to_dev(x, torch.bfloat16)
    eid = _routing(T, E, top_k, 9102 + T, idle=(1,) if E > 3 else ())
    tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, tile)
    y = torch.full((npad, N // 2), -3.0, dtype=torch.bfloat16, device=dev())
    ops.qmm_grouped_gated(*d, dx, to_dev(tile2e), to_dev(srow), act=act, out=y)
    assert ops.device_status() == 0
    yh = f32(y)
    fuse = oracle_mod.fused_geglu if act == "geglu" else oracle_mod.fused_swiglu
    for e in range(E):
        slots = np.nonzero((np.repeat(tile2e, tile) == e) & (srow >= 0))[0]
        if slots.size == 0:
            continue
        xe = np.ascontiguousarray(x[srow[slots]])
        codes, s, b = per[e]
        w_bf16 = oracle_mod.bf16_to_f32(oracle_mod.dequant_bf16(codes, s, b))
        want = synth.bf16_bits_to_f32(fuse(oracle_mod.matmul_f32(xe, w_bf16, "fast")))
        err = oracle_mod.err_metrics(yh[slots], want)
        assert err["rel_l2"] < TOL and err["max_rel_rms"] < TOL, (e, err)
    # padding slots of a live tile multiply zero rows: act(0) * 0 = 0; whole padding tiles do not exist
    pad = np.nonzero(srow < 0)[0]
    assert np.all(yh[pad] == 0.0)


@pytest.mark.parametrize("T,E,top_k,K,N", [(96, 4, 2, 512, 512), (300, 8, 2, 768, 1000), (40, 3, 1, 64, 33)])
def test_grouped_down_scatters_rows_to_pair_order(vpq, oracle_mod, T, E, top_k, K, N):
    ops = vpq.ops
    tile = ops.qmm_grouped_tile_rows()
    per, d = _experts(oracle_mod, E, N, K, 9200 + T + K)
    eid = _routing(T, E, top_k, 9201 + T)
    tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, tile)
    n_pairs = T * top_k
    xs = synth.activations_bf16(npad, K, 9202 + T)  # the sorted activations (output of the gate|up GEMM)
    y = torch.full((n_pairs + 1, N), -3.0, dtype=torch.bfloat16, device=dev())  # one guard row
    ops.qmm_grouped_down(*d, to_dev(xs, torch.bfloat16), to_dev(tile2e), to_dev(sdst), y_rows=n_pairs, out=y)
    assert ops.device_status() == 0
    yh = f32(y)
    assert np.all(yh[n_pairs] == -3.0)
    assert np.all(yh[:n_pairs] != -3.0)  # every pair has a slot
    for e in range(E):
        slots = np.nonzero((np.repeat(tile2e, tile) == e) & (sdst >= 0))[0]
        if slots.size == 0:
            continue
        codes, s, b = per[e]
        w_bf16 = oracle_mod.bf16_to_f32(oracle_mod.dequant_bf16(codes, s, b))
        want = synth.bf16_bits_to_f32(oracle_mod.narrow_f32_bf16(
            oracle_mod.matmul_f32(np.ascontiguousarray(xs[slots]), w_bf16, "fast")))
        err = oracle_mod.err_metrics(yh[sdst[slots]], want)
        assert err["rel_l2"] < TOL and err["max_rel_rms"] < TOL, (e, err)


def test_grouped_equals_the_plain_gemm_on_one_expert(vpq, oracle_mod):
    """One expert, identity routing: the grouped kernel's tiles are the plain GEMM's arithmetic."""
    ops = vpq.ops
    tile = ops.qmm_grouped_tile_rows()
    M, K, N = tile, 256, 512  # M <= 128: the plain entry runs the same single-CTA kernel
    per, d = _experts(oracle_mod, 1, N, K, 9300)
    x = to_dev(synth.activations_bf16(M, K, 9301), torch.bfloat16)
    tile2e = to_dev(np.zeros(M // tile, np.int32))
    y = ops.qmm_grouped_down(*d, x, tile2e)
    plain = ops.qmm(d[0][0], d[1][0], d[2][0], x)
    assert torch.equal(y, plain)
    # the gated store against the CTA-pair kernel's: the same f32 sums and the same activation
    g = ops.qmm_grouped_gated(*d, x, tile2e)
    want = ops.qmm_swiglu(d[0][0], d[1][0], d[2][0], x)
    assert float((g == want).float().mean()) > 0.99
    assert oracle_mod.err_metrics(f32(g), f32(want))["max_rel_rms"] < 1e-3


def test_grouped_skips_padding_tiles_and_bad_experts(vpq, oracle_mod):
    ops = vpq.ops
    tile = ops.qmm_grouped_tile_rows()
    K, N = 128, 256
    per, d = _experts(oracle_mod, 2, N, K, 9400)
    x = to_dev(synth.activations_bf16(3 * tile, K, 9401), torch.bfloat16)
    tile2e = to_dev(np.array([1, -1, 7], np.int32))  # tile 1: padding; tile 2: no such expert
    y = torch.full((3 * tile, N), -3.0, dtype=torch.bfloat16, device=dev())
    ops.qmm_grouped_down(*d, x, tile2e, out=y)
    assert ops.device_status() == 0
    assert torch.equal(y[:tile], ops.qmm(d[0][1], d[1][1], d[2][1], x[:tile].contiguous()))
    assert torch.all(y[tile:] == -3.0)


def test_grouped_by_reference_names(vpq, oracle_mod):
    ops = vpq.ops
    tile = ops.qmm_grouped_tile_rows()
    T, E, top_k, K, N = 64, 3, 2, 128, 128
    per, d = _experts(oracle_mod, E, N, K, 9500)
    x = to_dev(synth.activations_bf16(T, K, 9501), torch.bfloat16)
    eid = _routing(T, E, top_k, 9502)
    tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, tile)
    t2e, sr, sd = to_dev(tile2e), to_dev(srow), to_dev(sdst)
    lib = "affine_qmm_steel_bf16"
    for entry, act in (("affine_qmm_grouped_swiglu_w4g64", "swiglu"), ("affine_qmm_grouped_geglu_w4g64", "geglu")):
        want = ops.qmm_grouped_gated(*d, x, t2e, sr, act=act)
        y = torch.zeros_like(want)
        scratch = torch.empty((npad, K), dtype=torch.bfloat16, device=dev())
        ops.dispatch(ops.function(lib, entry), {0: d[0], 1: d[1], 2: d[2], 3: x, 4: y, 8: t2e, 9: sr, 10: scratch},
                     K=K, N=N, M=npad, experts=E, rows=T)
        assert torch.equal(y, want), entry
    xs = to_dev(synth.activations_bf16(npad, K, 9503), torch.bfloat16)
    want = ops.qmm_grouped_down(*d, xs, t2e, sd, y_rows=T * top_k)
    y = torch.zeros_like(want)
    ops.dispatch(ops.function(lib, "affine_qmm_grouped_w4g64"), {0: d[0], 1: d[1], 2: d[2], 3: xs, 4: y, 8: t2e, 9: sd},
                 K=K, N=N, M=npad, experts=E, rows=T * top_k)
    assert torch.equal(y, want)


def _experts8(oracle_mod, E, N, K, seed):
    per = []
    for e in range(E):
        wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, seed + 17 * e))
        c, s16, b16 = oracle_mod.quant(wb, 8, 64)
        per.append((c, oracle_mod.f16_to_bf16(s16), oracle_mod.f16_to_bf16(b16)))
    d = (to_dev(np.stack([p[0] for p in per])), to_dev(np.stack([p[1] for p in per]), torch.bfloat16),
         to_dev(np.stack([p[2] for p in per]), torch.bfloat16))
    return per, d


@pytest.mark.parametrize("act", ["swiglu", "geglu"])
def test_grouped_gemms_over_8_bit_experts(vpq, oracle_mod, act):
    """affine_qmm_grouped_swiglu_w8g64 / _geglu_w8g64 / affine_qmm_grouped_w8g64
    (affine_qmm_steel.metal:1069-1094,1290-1312,1341-1367): gate|up with the row gather, then down with
    the scatter, per expert against the oracle (dequantise to bf16, fp32 matmul); also by name."""
    ops = vpq.ops
    tile = ops.qmm_grouped_tile_rows()
    T, E, top_k, H, F = 200, 5, 2, 512, 320
    per_gu, d_gu = _experts8(oracle_mod, E, 2 * F, H, 9500)
    per_dn, d_dn = _experts8(oracle_mod, E, H, F, 9600)
    x = synth.activations_bf16(T, H, 9700)
    dx = to_dev(x, torch.bfloat16)
    eid = _routing(T, E, top_k, 9701, idle=(3,))
    tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, tile)
    dt, dsrow, dsdst = to_dev(tile2e), to_dev(srow), to_dev(sdst)
    act_out = torch.full((npad, F), -3.0, dtype=torch.bfloat16, device=dev())
    ops.qmm_grouped_gated(*d_gu, dx, dt, dsrow, act=act, out=act_out, bits=8)
    n_pairs = T * top_k
    y = torch.full((n_pairs + 1, H), -3.0, dtype=torch.bfloat16, device=dev())
    ops.qmm_grouped_down(*d_dn, act_out, dt, dsdst, y_rows=n_pairs, out=y, bits=8)
    assert ops.device_status() == 0
    ah, yh = f32(act_out), f32(y)
    assert np.all(yh[n_pairs] == -3.0) and np.all(yh[:n_pairs] != -3.0)
    fuse = oracle_mod.fused_geglu if act == "geglu" else oracle_mod.fused_swiglu
    from test_gpu_parity import bits16
    a_bits = bits16(act_out)
    for e in range(E):
        slots = np.nonzero((np.repeat(tile2e, tile) == e) & (srow >= 0))[0]
        if slots.size == 0:
            continue
        c, s, b = per_gu[e]
        w = oracle_mod.bf16_to_f32(oracle_mod.dequant_bf16_any(c, s, b, 8, 64))
        want = synth.bf16_bits_to_f32(fuse(oracle_mod.matmul_f32(np.ascontiguousarray(x[srow[slots]]), w, "fast")))
        err = oracle_mod.err_metrics(ah[slots], want)
        assert err["rel_l2"] < TOL and err["max_rel_rms"] < TOL, ("gate|up", e, err)
        c, s, b = per_dn[e]
        w = oracle_mod.bf16_to_f32(oracle_mod.dequant_bf16_any(c, s, b, 8, 64))
        want = synth.bf16_bits_to_f32(oracle_mod.narrow_f32_bf16(
            oracle_mod.matmul_f32(np.ascontiguousarray(a_bits[slots]), w, "fast")))
        err = oracle_mod.err_metrics(yh[sdst[slots]], want)
        assert err["rel_l2"] < TOL and err["max_rel_rms"] < TOL, ("down", e, err)
    # by the reference's names (slots as for the 4-bit kernels: 8 = tile2e, 9 = srow / sdst, 10 = scratch)
    act2 = torch.full_like(act_out, -3.0)
    scratch = torch.empty((npad, H), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_qmm_steel_bf16", f"affine_qmm_grouped_{act}_w8g64"),
                 {0: d_gu[0], 1: d_gu[1], 2: d_gu[2], 3: dx, 4: act2, 8: dt, 9: dsrow, 10: scratch},
                 K=H, N=2 * F, M=npad, experts=E, rows=T)
    assert torch.equal(act2, act_out)
    y2 = torch.full_like(y, -3.0)
    ops.dispatch(ops.function("affine_qmm_steel_bf16", "affine_qmm_grouped_w8g64"),
                 {0: d_dn[0], 1: d_dn[1], 2: d_dn[2], 3: act_out, 4: y2, 8: dt, 9: dsdst},
                 K=F, N=H, M=npad, experts=E, rows=n_pairs)
    assert torch.equal(y2, y)
