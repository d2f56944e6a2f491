"""Small, self-contained invocations of the kernels for profiling and quick timing.

    python -m vpipe_b200.cases qmv  K N [launches]     # single GEMVs on distinct weight copies
    python -m vpipe_b200.cases plan LAYERS             # the C2 decode set as one plan launch
    python -m vpipe_b200.cases qmv_batch K N M [launches]  # small-batch GEMV vs M serial GEMVs
    python -m vpipe_b200.cases qmv_w8 K N [launches]   # 8-bit GEMV on distinct weight copies (graph replay)
    python -m vpipe_b200.cases decode_layers LAYERS    # 8B-decoder layers as dependent fused launches (graph replay)
    python -m vpipe_b200.cases qmm  M K N [reps]       # the GEMM
    python -m vpipe_b200.cases qmm_swiglu M K N [reps] # the GEMM with the fused SwiGLU store (N = 2 ffn)
    python -m vpipe_b200.cases qmm_w8 M K N [reps]     # the GEMM over 8-bit weights
    python -m vpipe_b200.cases moe T E TOPK HIDDEN FFN [reps]  # grouped gate|up (SwiGLU) + down GEMMs of one MoE layer

Weights are random packed nibbles with bf16 scales / biases (the distribution of the reference's
kernel tests); each command prints one JSON line with the CUDA-event time. Meant to be wrapped by
`ncu -k regex:affine_q… -c 1` on a size that ends in seconds.
"""
from __future__ import annotations

import json
import sys

import torch

from . import ops, synth


def _weight(N, K, dev):
    codes = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device=dev)
    s = (torch.rand((N, K // 64), device=dev) * 0.015 + 0.005).to(torch.bfloat16)
    b = (torch.rand((N, K // 64), device=dev) * 0.2 - 0.1).to(torch.bfloat16)
    return codes, s, b


def _time(fn, reps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / reps


def main(argv):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    kind = argv[0]
    if kind == "qmv":
        K, N = int(argv[1]), int(argv[2])
        n = int(argv[3]) if len(argv) > 3 else 6
        x = torch.randn((1, K), device=dev).to(torch.bfloat16)
        sets = [_weight(N, K, dev) + (x, torch.empty((1, N), dtype=torch.bfloat16, device=dev)) for _ in range(n)]
        it = iter(sets * 2)
        for p in sets:
            ops.qmv(*p[:4], out=p[4])
        torch.cuda.synchronize()
        t = _time(lambda: (lambda p: ops.qmv(*p[:4], out=p[4]))(next(it)), n)
        print(json.dumps({"case": "qmv", "K": K, "N": N, "us": t * 1e6,
                          "GBs": synth.qmv_bytes(K, N) / t / 1e9}))
    elif kind == "decode_layers":
        # What a decode step of an 8B decoder issues per layer when it uses the fused entries:
        # q|k|v (one GEMV, three outputs), o_proj + residual, gate|up with SwiGLU, down + residual;
        # each launch reads what the one before wrote (attention itself is not modelled: o_proj
        # reads the q output). 4 launches per layer instead of 7 plain GEMVs + 3 elementwise passes.
        layers = int(argv[1])
        H, KV, F = 4096, 1024, 12288
        h = torch.randn((1, H), device=dev).to(torch.bfloat16)
        L, nbytes = [], 0
        for _ in range(layers):
            qkv, o, gu, dn = _weight(H + 2 * KV, H, dev), _weight(H, H, dev), _weight(2 * F, H, dev), _weight(H, F, dev)
            bufs = [torch.empty((1, n), dtype=torch.bfloat16, device=dev) for n in (H, KV, KV, H, F, H)]
            L.append((qkv, o, gu, dn, bufs))
            nbytes += (synth.qmv_bytes(H, H + 2 * KV) + synth.qmv_bytes(H, H) + synth.qmv_bytes(H, 2 * F) +
                       synth.qmv_bytes(F, H))

        def step():
            x = h
            for qkv, o, gu, dn, (q, k, v, h1, act, h2) in L:
                check = ops.check
                lib = ops.lib()
                st = torch.cuda.current_stream().cuda_stream
                check(lib.vpq_affine_qmv_qkv_w4g64_bf16(qkv[0].data_ptr(), qkv[1].data_ptr(), qkv[2].data_ptr(),
                                                        x.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                                        H, H, KV, KV, 1, st))
                ops.qmv_add(o[0], o[1], o[2], q, x, out=h1)
                ops.qmv_swiglu(gu[0], gu[1], gu[2], h1, out=act)
                ops.qmv_add(dn[0], dn[1], dn[2], act, h1, out=h2)
                x = h2

        step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        g.replay()
        torch.cuda.synchronize()
        t = _time(g.replay, 5)
        print(json.dumps({"case": "decode_layers", "layers": layers, "launches": 4 * layers, "us": t * 1e6,
                          "us_per_launch": t * 1e6 / (4 * layers), "GBs": nbytes / t / 1e9}))
    elif kind == "qmv_w8":
        K, N = int(argv[1]), int(argv[2])
        n = int(argv[3]) if len(argv) > 3 else 8
        x = torch.randn((1, K), device=dev).to(torch.bfloat16)
        sets = []
        for _ in range(n):
            codes = torch.randint(-2**31, 2**31 - 1, (N, K // 4), dtype=torch.int32, device=dev)
            s = (torch.rand((N, K // 64), device=dev) * 0.001 + 0.0003).to(torch.bfloat16)
            b = (torch.rand((N, K // 64), device=dev) * 0.2 - 0.1).to(torch.bfloat16)
            sets.append((codes, s, b, x, torch.empty((1, N), dtype=torch.bfloat16, device=dev)))
        for p in sets:
            ops.qmv_w8(*p[:4], out=p[4])
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for p in sets:
                ops.qmv_w8(*p[:4], out=p[4])
        g.replay()
        torch.cuda.synchronize()
        t = _time(g.replay, 3) / n
        nbytes = N * K + 2 * N * (K // 64) * 2 + 2 * K + 2 * N
        print(json.dumps({"case": "qmv_w8", "K": K, "N": N, "us": t * 1e6, "GBs": nbytes / t / 1e9}))
    elif kind == "qmv_batch":
        K, N, M = int(argv[1]), int(argv[2]), int(argv[3])
        n = int(argv[4]) if len(argv) > 4 else 8
        x = torch.randn((M, K), device=dev).to(torch.bfloat16)
        sets = [_weight(N, K, dev) + (x, torch.empty((M, N), dtype=torch.bfloat16, device=dev)) for _ in range(n)]
        out = {"case": "qmv_batch", "K": K, "N": N, "M": M}
        for name, fn in (("batch", ops.qmv_batch_rows), ("serial", ops.qmv)):
            for p in sets:
                fn(*p[:4], out=p[4])
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()          # graph replay: launch overhead out of the picture
            with torch.cuda.graph(g):
                for p in sets:
                    fn(*p[:4], out=p[4])
            g.replay()
            torch.cuda.synchronize()
            t = _time(g.replay, 3) / n
            out[name + "_us"] = t * 1e6
            out[name + "_weight_GBs"] = synth.qmv_bytes(K, N) / t / 1e9
        out["speedup"] = out["serial_us"] / out["batch_us"]
        print(json.dumps(out))
    elif kind == "plan":
        layers = int(argv[1])
        xs = {K: torch.randn((1, K), device=dev).to(torch.bfloat16) for K in (4096, 12288)}
        probs = []
        for _ in range(layers):
            for p in synth.CONFIGS["C2"].projs:
                probs.append(_weight(p.N, p.K, dev) + (xs[p.K], torch.empty((1, p.N), dtype=torch.bfloat16, device=dev)))
        plan = ops.QmvPlan(probs)
        for _ in range(3):
            plan.run()
        torch.cuda.synchronize()
        t = _time(plan.run, 1)
        nbytes = sum(synth.qmv_bytes(p.K, p.N) for p in synth.CONFIGS["C2"].projs) * layers
        print(json.dumps({"case": "plan", "layers": layers, "us": t * 1e6, "GBs": nbytes / t / 1e9}))
    elif kind == "qmm_w8":
        M, K, N = int(argv[1]), int(argv[2]), int(argv[3])
        reps = int(argv[4]) if len(argv) > 4 else 3
        x = torch.randn((M, K), device=dev).to(torch.bfloat16)
        codes = torch.randint(-2**31, 2**31 - 1, (N, K // 4), dtype=torch.int32, device=dev)
        s = (torch.rand((N, K // 64), device=dev) * 0.001 + 0.0003).to(torch.bfloat16)
        b = (torch.rand((N, K // 64), device=dev) * 0.2 - 0.1).to(torch.bfloat16)
        y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            ops.qmm_w8(codes, s, b, x, out=y)
        torch.cuda.synchronize()
        t = _time(lambda: ops.qmm_w8(codes, s, b, x, out=y), reps)
        print(json.dumps({"case": kind, "M": M, "K": K, "N": N, "ms": t * 1e3,
                          "tflops": synth.qmm_flops(K, N, M) / t / 1e12}))
    elif kind in ("qmm", "qmm_swiglu"):
        M, K, N = int(argv[1]), int(argv[2]), int(argv[3])
        reps = int(argv[4]) if len(argv) > 4 else 3
        x = torch.randn((M, K), device=dev).to(torch.bfloat16)
        codes, s, b = _weight(N, K, dev)
        fn = ops.qmm if kind == "qmm" else ops.qmm_swiglu
        y = torch.empty((M, N if kind == "qmm" else N // 2), dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            fn(codes, s, b, x, out=y)
        torch.cuda.synchronize()
        t = _time(lambda: fn(codes, s, b, x, out=y), reps)
        print(json.dumps({"case": kind, "M": M, "K": K, "N": N, "ms": t * 1e3,
                          "tflops": synth.qmm_flops(K, N, M) / t / 1e12}))
    elif kind == "moe":
        import numpy as np
        from . import moe
        T, E, top_k, H, F = (int(a) for a in argv[1:6])
        reps = int(argv[6]) if len(argv) > 6 else 3
        tile = ops.qmm_grouped_tile_rows()
        rng = np.random.default_rng(0)
        eid = np.stack([rng.choice(E, size=top_k, replace=False) for _ in range(T)]).reshape(-1).astype(np.int32)
        tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, tile)
        tile2e, srow, sdst = (torch.from_numpy(a).to(dev) for a in (tile2e, srow, sdst))
        hidden = torch.randn((T, H), device=dev).to(torch.bfloat16)
        gu = [t.view(E, 2 * F, -1) for t in _weight(E * 2 * F, H, dev)]
        dn = [t.view(E, H, -1) for t in _weight(E * H, F, dev)]
        act = torch.empty((npad, F), dtype=torch.bfloat16, device=dev)
        part = torch.empty((T * top_k, H), dtype=torch.bfloat16, device=dev)

        def layer():
            ops.qmm_grouped_gated(*gu, hidden, tile2e, srow, out=act)
            ops.qmm_grouped_down(*dn, act, tile2e, sdst, y_rows=T * top_k, out=part)

        for _ in range(2):
            layer()
        torch.cuda.synchronize()
        t = _time(layer, reps)
        useful = 2.0 * T * top_k * (H * 2 * F + F * H)
        padded = 2.0 * npad * (H * 2 * F + F * H)
        print(json.dumps({"case": kind, "tokens": T, "experts": E, "top_k": top_k, "hidden": H, "ffn": F,
                          "rows_padded": npad, "ms": t * 1e3, "tflops_useful": useful / t / 1e12,
                          "tflops_padded": padded / t / 1e12}))
    else:
        raise SystemExit(__doc__)
    assert ops.device_status() == 0


if __name__ == "__main__":
    main(sys.argv[1:])
