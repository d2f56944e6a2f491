#!/usr/bin/env python
"""Benchmark of the 4-bit affine quantized linear on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c3|c4|c5|c1|plan|decode_chain|qmm|qmm_swiglu|qmm_w8|moe|...] [shape ...]

Default workload c2 (what the headline metric is quoted on): the decode-layer QMV set of an 8B
Qwen3-style decoder at batch 1 -- q, k, v, gate, up, down at M = 1 -- for all 36 layers with
distinct weights (3.57 GB, larger than L2, so everything streams from HBM). One step = one pass
over the 36 layers = 216 GEMVs, run as one plan launch (vpq_qmv_plan_run); --no-plan replays 216
separate launches as a graph. `value` is algorithmic GB/s with everything resident in HBM; `e2e`
is the same pass driven through the C ABI with the step's activations copied from pinned host
memory and the result read back, inside the timed region. The same JSON line carries
  c1            the single 4096 x 4096 GEMV of configs[0], cold weights, one launch per GEMV
  decode_chain  36 decoder layers as a DEPENDENT chain (norm + q|k|v, o + residual, norm + gate|up
                with SwiGLU, down + residual; each GEMV reads what the one before wrote), as one
                chained launch and as one launch per GEMV (graph replay), with a bit-identity check
                between them; `value` is the faster form, named in `form`
  qmm, qmm_c3   the tensor-core GEMM on the DiT (C4) and prefill (C3) shapes in TFLOP/s
  cpu_baseline  the reference's CPU arithmetic for the same op on the host cores (QMV and QMM).

With N > 1 (torchrun) the QMV set runs as N independent replicas (decode at batch 1 does not
shard: "replicas only"); the `qmm` section is the part that is partitioned across the GPUs
(column split): per shape the unsharded time on the same box, the fused peer-store form, GEMM +
NCCL all-gather (whole and in 4 row chunks), the bytes that cross NVLink, and a bit-identity
check of the gathered result against the unsharded kernel (the run exits non-zero on a mismatch).

Inputs are synthetic: weights N(0, 0.02) quantised with the reference recipe on the device,
activations N(0, 1) bf16; seeded. The small workloads at the end of the list (plan LAYERS,
decode_chain LAYERS, qmm M K N, qmm_swiglu M K N, qmm_w8 M K N, qmv K N, qmv_w8 K N,
qmv_batch K N M, moe T E TOPK HIDDEN FFN, streams [N K COPIES]) run one kernel on a small case and print one JSON line;
they are what the ncu summaries under profiles/ were taken from.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
LAYERS = 36
MIN_TIMED_SECONDS = 0.5     # the headline's timed blocks are repeated until this much has been timed
NVLINK_GBS_MEASURED = 770.0  # peer copy per direction per GPU on this pool; nominal 900

# DRAM traffic per launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum) as a
# multiple of the launch's algorithmic bytes: a 4-layer plan launch of the C2 set (405.7 MB moved for
# 396.9 MB algorithmic; it grows in proportion to the layers), and the GEMM at M = K = N = 8192
# (402.8 MB moved for 306 MB: x tiles that have left L2 are read again; an upper estimate for the
# smaller C3 / C4 shapes, whose x stays in L2).
QMV_TRAFFIC_RATIO = 1.022
QMM_TRAFFIC_RATIO = 1.32


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_cores() -> int:
    """Cores this process may run on. Not OMP_NUM_THREADS: torchrun sets that to 1."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler:
    """SM clock and throttle reasons sampled while the timed region runs: NVML polled every ~2 ms
    from a thread (reading only), nvidia-smi every 100 ms if NVML is not importable."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                   0x4: "sw_power_cap"}

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.rows = []
        self.max_mhz = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:  # the CUDA index is relative to CUDA_VISIBLE_DEVICES: find the same GPU by its UUID
            import torch
            uuid = str(torch.cuda.get_device_properties(self.idx).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.idx)

    def start(self):
        try:
            nv, h = self._nvml_handle()
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.halt = threading.Event()

            def loop():
                while not self.halt.is_set():
                    try:
                        self.rows.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                          int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.idx), "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.halt.set()
            self.thread.join(timeout=2)
            if self.rows:
                reasons = set()
                for _, mask in self.rows:
                    reasons.update(name for bit, name in self.REASON_BITS.items() if mask & bit)
                out.update(sm_mhz=statistics.median(r[0] for r in self.rows), sm_max_mhz=self.max_mhz,
                           samples=len(self.rows), reasons=sorted(reasons), source="nvml")
            return out
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                    "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm),
                       reasons=sorted(reasons), source="nvidia-smi")
        return out


def dist_env(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    return rank, world, local


# ------------------------------------------------------------------ CPU arms (oracle port)

def _cpu_qmv_layer(synth, tag):
    layer = []
    for p in synth.CONFIGS["C2"].projs:
        codes, s, b = synth.random_qweight(p.N, p.K, synth.seed_for(tag, p.name))
        x = synth.activations_bf16(1, p.K, synth.seed_for(tag + "x", p.name))
        layer.append((codes, s, b, x))
    return layer, sum(synth.qmv_bytes(p.K, p.N, 1) for p in synth.CONFIGS["C2"].projs)


def _cpu_qmm_shapes(synth, key, rows, tag):
    """One M-slice of `rows` rows of every shape of a QMM config: the CPU cost is linear in M (the
    dequantisation of the whole weight is part of every step, as it would be of a full-M step)."""
    shapes = []
    for p in synth.CONFIGS[key].projs:
        codes, s, b = synth.random_qweight(p.N, p.K, synth.seed_for(tag, key, p.name))
        x = synth.activations_bf16(rows, p.K, synth.seed_for(tag + "x", key, p.name))
        shapes.append((codes, s, b, x, synth.qmm_flops(p.K, p.N, rows)))
    return shapes


def cpu_baseline_qmv(synth, seconds_budget=10.0):
    """The oracle port (f32 dequantise + blocked fp32 GEMM, all host cores) on a bounded sample of
    the C2 set: whole decoder layers until the time budget is used."""
    import oracle
    oracle.build()
    layer, bytes_layer = _cpu_qmv_layer(synth, "cpu")
    threads = host_cores()
    for codes, s, b, x in layer:   # warm
        oracle.cpu_linear_seconds(codes, s, b, x, threads)
    t, n = 0.0, 0
    while t < seconds_budget and n < LAYERS:
        for codes, s, b, x in layer:
            t += oracle.cpu_linear_seconds(codes, s, b, x, threads)[0]
        n += 1
    return {"value": bytes_layer * n / t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{n} of {LAYERS} decoder layers (6 QMV projections each), "
                      "f32 dequantise + blocked fp32 GEMM, OpenMP"}


def cpu_baseline_qmm(synth, key, rows=256):
    """The same CPU arithmetic on the GEMM shapes of one config, on an M-slice (linear in M)."""
    import oracle
    oracle.build()
    threads = host_cores()
    shapes = _cpu_qmm_shapes(synth, key, rows, "cpuqmm")
    t, flops = 0.0, 0.0
    for codes, s, b, x, fl in shapes:
        t += oracle.cpu_linear_seconds(codes, s, b, x, threads)[0]
        flops += fl
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{key}: every shape on an M-slice of {rows} of {synth.CONFIGS[key].M} rows "
                      "(cost is linear in M); f32 dequantise of the whole weight + blocked fp32 GEMM, OpenMP"}


def run_reference(args, rank, world):
    """The reference's CPU path for this op, timed on the host cores. The reference has no CPU
    matmul: this is its f32 dequantise routine plus a plain blocked fp32 GEMM (the oracle port), on
    all host cores. Each step is a bounded sample of the workload."""
    if rank != 0:
        return
    import oracle
    from vpipe_b200 import synth
    oracle.build()
    threads = host_cores()
    wl = args.workload if args.workload in ("c3", "c4", "c5") else "c2"
    if wl == "c2":
        layer, per_step = _cpu_qmv_layer(synth, "ref")
        metric, unit, scale = "int4_qmv_hbm_gbps", "GB/s", 1e9
        workload = "C2 decode-layer QMV set, 8B Qwen3-style decoder, M=1"
        sample = "1 of 36 layers per step (6 projections, 99.2 MB of weights)"

        def step():
            return sum(oracle.cpu_linear_seconds(c, s, b, x, threads)[0] for c, s, b, x in layer)
    else:
        key = wl.upper()
        rows = 512 if key != "C5" else 256
        shapes = _cpu_qmm_shapes(synth, key, rows, "ref")
        per_step = sum(sh[4] for sh in shapes)
        metric, unit, scale = "int4_qmm_tflops", "TFLOP/s", 1e12
        workload = f"{key} {synth.CONFIGS[key].what}"
        sample = f"every shape on an M-slice of {rows} of {synth.CONFIGS[key].M} rows per step"

        def step():
            return sum(oracle.cpu_linear_seconds(c, s, b, x, threads)[0] for c, s, b, x, _ in shapes)

    for _ in range(max(min(args.warmup, 3), 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = per_step * args.steps / dt / scale
    line = {
        "impl": "reference", "metric": metric, "value": val, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak" if wl == "c2" else "strong",
        "vs_baseline": None, "dtype": "int4 x bf16 -> f32", "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": {"value": val, "unit": unit, "cores": threads, "kind": "port",
                         "sample": sample + "; f32 dequantise + blocked fp32 GEMM, OpenMP"},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------ our arm

def make_linear(torch, ops, N, K, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    w = (torch.randn((N, K), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    codes, s16, b16 = ops.quantize(w)
    s, b = ops.scales_to_bf16(s16), ops.scales_to_bf16(b16)
    del w, s16, b16
    return codes, s, b


def rand_weight(torch, N, K, dev, bits=4):
    """Random packed codes with bf16 scales / biases (the distribution of the reference's kernel tests)."""
    codes = torch.randint(-2**31, 2**31 - 1, (N, K * bits // 32), dtype=torch.int32, device=dev)
    lo, span = (0.005, 0.015) if bits == 4 else (0.0003, 0.001)
    s = (torch.rand((N, K // 64), device=dev) * span + lo).to(torch.bfloat16)
    b = (torch.rand((N, K // 64), device=dev) * 0.2 - 0.1).to(torch.bfloat16)
    return codes, s, b


def timed(torch, fn, steps, warmup, barrier):
    """W warm-up + K timed steps between barriers; CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / 1e3  # seconds


def max_over_ranks(torch, dist, world, t, dev):
    if world == 1:
        return t
    v = torch.tensor([t], device=dev, dtype=torch.float64)
    dist.all_reduce(v, op=dist.ReduceOp.MAX)
    return float(v.item())


def timed_blocks(torch, dist, world, dev, fn, steps, warmup, barrier, min_seconds=MIN_TIMED_SECONDS, max_blocks=400):
    """Blocks of exactly `steps` steps, each bracketed by a barrier + synchronize and timed with CUDA
    events (max over ranks), repeated until at least `min_seconds` have been timed. Returns the
    list of block times in seconds (every rank runs the same number of blocks)."""
    first = max_over_ranks(torch, dist, world, timed(torch, fn, steps, warmup, barrier), dev)
    blocks = [first]
    n = min(max_blocks, max(2, int(math.ceil(min_seconds / max(first, 1e-6)))))
    for _ in range(n - 1):
        blocks.append(max_over_ranks(torch, dist, world, timed(torch, fn, steps, 0, barrier), dev))
    return blocks


def graph_of(torch, fn):
    """fn captured into a CUDA graph (after one eager run on a side stream)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    return g


def bench_qmv(torch, dist, ops, synth, args, rank, world, dev, pk):
    cfg = synth.CONFIGS["C2"]
    bytes_step = 0
    # the step's activations live in ONE device buffer (one host->device copy per step), the last
    # layer's outputs in another (one device->host copy per step)
    Ks = sorted({p.K for p in cfg.projs})
    x_all = torch.empty((sum(Ks),), dtype=torch.bfloat16, device=dev)
    xs, off = {}, 0
    for K in Ks:
        g = torch.Generator(device=dev).manual_seed(synth.seed_for("x", K, rank))
        xs[K] = x_all[off:off + K].view(1, K)     # offsets are multiples of 4096 elements: 16-byte aligned
        xs[K].copy_(torch.randn((1, K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16))
        off += K
    y_last = torch.empty((sum(p.N for p in cfg.projs),), dtype=torch.bfloat16, device=dev)
    problems = []
    for layer in range(LAYERS):
        off = 0
        for p in cfg.projs:
            codes, s, b = make_linear(torch, ops, p.N, p.K, synth.seed_for("w", layer, p.name, rank), dev)
            if layer == LAYERS - 1:
                y = y_last[off:off + p.N].view(1, p.N)
                off += p.N
            else:
                y = torch.empty((1, p.N), dtype=torch.bfloat16, device=dev)
            problems.append((codes, s, b, xs[p.K], y))
            bytes_step += synth.qmv_bytes(p.K, p.N, 1)
    launches_step = len(problems)
    torch.cuda.synchronize()

    # The whole pass as ONE launch (a plan: "encode once, commit many"), or, with --no-plan, the
    # 216 launches replayed as one CUDA graph. Either must work: there is no quieter fallback.
    if not args.no_plan:
        plan = ops.QmvPlan(problems)
        step = plan.run
        launches_step = 1
        mode = "plan (1 launch per step)"
    else:
        descs = ops.qmv_set(problems)
        graph = graph_of(torch, lambda: ops.qmv_batch(descs))
        step = graph.replay
        mode = "cuda-graph of 216 launches"
    step()
    torch.cuda.synchronize()

    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    sampler = ClockSampler(dev.index)
    sampler.start()
    blocks = timed_blocks(torch, dist, world, dev, step, args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    t = statistics.median(blocks)
    value = bytes_step * args.steps * world / t / 1e9

    # e2e: the step's activations come from pinned host memory, the last layer's outputs go back
    host_x = torch.randn((x_all.numel(),)).to(torch.bfloat16).pin_memory()
    host_y = torch.empty((y_last.numel(),), dtype=torch.bfloat16).pin_memory()
    h2d = host_x.numel() * 2
    d2h = host_y.numel() * 2

    def e2e_step():
        x_all.copy_(host_x, non_blocking=True)
        step()
        host_y.copy_(y_last, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    eblocks = timed_blocks(torch, dist, world, dev, e2e_step, args.steps, args.warmup, barrier, min_seconds=0.25)
    te = statistics.median(eblocks)
    e2e_val = bytes_step * args.steps * world / te / 1e9
    assert ops.device_status() == 0

    per_gpu = bytes_step * args.steps / t / 1e9
    roof = {"bound": "hbm", "achieved": per_gpu, "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": per_gpu / pk["hbm_gbs"], "peak_source": pk["source"],
            "kernel": "affine_qmv_w4g64_kernel", "launches_per_step": launches_step,
            "gemvs_per_step": len(problems), "bytes_per_launch_avg": bytes_step / launches_step,
            "traffic": (QMV_TRAFFIC_RATIO * bytes_step / launches_step) if QMV_TRAFFIC_RATIO else None}
    return {
        "value": value, "t": t, "bytes_step": bytes_step, "launches_step": launches_step,
        "clocks": clocks, "roofline": roof, "mode": mode,
        "timing": {"blocks": len(blocks), "steps_per_block": args.steps, "timed_seconds": sum(blocks),
                   "ms_per_step_median": t / args.steps * 1e3, "ms_per_step_min": min(blocks) / args.steps * 1e3,
                   "ms_per_step_max": max(blocks) / args.steps * 1e3},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": te / args.steps * 1e3},
    }


def bench_c1(torch, ops, synth, dev, pk, copies=32, reps=20):
    """configs[0]: one 4096 x 4096 GEMV. `copies` distinct weights (302 MB > 2 x L2) are cycled so
    every launch streams from HBM; the launches are replayed from a CUDA graph, one launch per GEMV
    (the reference's method: tests/unit-tests/metal-lm/quant-gemv-bench.cc:625-632,680)."""
    K = N = 4096
    x = torch.randn((1, K), device=dev).to(torch.bfloat16)
    sets = [rand_weight(torch, N, K, dev) + (x, torch.empty((1, N), dtype=torch.bfloat16, device=dev))
            for _ in range(copies)]
    g = graph_of(torch, lambda: [ops.qmv(*p[:4], out=p[4]) for p in sets])
    t = timed(torch, g.replay, reps, 3, lambda: None) / (reps * copies)
    gbs = synth.qmv_bytes(K, N) / t / 1e9
    return {"workload": "C1 single int4 GEMV, M=1, K=N=4096", "us_per_gemv": t * 1e6, "value": gbs, "unit": "GB/s",
            "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "launches": copies * reps,
            "method": f"{copies} distinct weight copies (302 MB, cold), graph-replayed single launches"}


def decoder_chain(torch, ops, synth, layers, dev, H=4096, KV=1024, F=12288, seed=0):
    """Weights and buffers of `layers` 8B-style decoder layers and the list of fused GEMVs a decode
    step issues per layer: RMSNorm + q|k|v (three outputs), o_proj + residual, RMSNorm + gate|up with
    SwiGLU, down + residual. Every GEMV reads what the one before wrote (attention itself is not
    part of this path: o_proj reads the q output). Returns (problems, bytes per step)."""
    h = torch.randn((1, H), device=dev).to(torch.bfloat16)
    problems, nbytes = [], 0
    x = h
    for i in range(layers):
        ws = [make_linear(torch, ops, n, k, synth.seed_for("chain", seed, i, j), dev)
              for j, (n, k) in enumerate([(H + 2 * KV, H), (H, H), (2 * F, H), (H, F)])]
        nw1 = (1.0 + 0.1 * torch.randn((H,), device=dev)).to(torch.bfloat16)
        nw2 = (1.0 + 0.1 * torch.randn((H,), device=dev)).to(torch.bfloat16)
        q, k, v, h1, act, h2 = (torch.zeros((1, n), dtype=torch.bfloat16, device=dev) for n in (H, KV, KV, H, F, H))
        problems += [
            ws[0] + (x, q, {"epilogue": "qkv", "aux": k, "y3": v, "q_rows": H, "k_rows": KV, "norm_w": nw1,
                            "eps": 1e-6, "depends": i > 0}),
            ws[1] + (q, h1, {"epilogue": "add", "aux": x, "depends": True}),
            ws[2] + (h1, act, {"epilogue": "swiglu", "norm_w": nw2, "eps": 1e-6, "depends": True}),
            ws[3] + (act, h2, {"epilogue": "add", "aux": h1, "depends": True}),
        ]
        nbytes += (synth.qmv_bytes(H, H + 2 * KV) + synth.qmv_bytes(H, H) + synth.qmv_bytes(H, 2 * F) +
                   synth.qmv_bytes(F, H))
        x = h2
    return problems, nbytes


def chain_outputs(problems):
    out = []
    for p in problems:
        out.append(p[4])
        if p[5]["epilogue"] == "qkv":
            out += [p[5]["aux"], p[5]["y3"]]
    return out


def bench_decode_chain(torch, ops, synth, dev, pk, layers=LAYERS, reps=10):
    """The decode step as a decoder issues it: a dependent chain. One chained launch (every GEMV
    waits on-chip for its predecessors while the weight stream runs ahead) against one launch per
    GEMV replayed from a CUDA graph; the two must produce the same bytes."""
    problems, nbytes = decoder_chain(torch, ops, synth, layers, dev)
    plain = [p[:5] + ({k: v for k, v in p[5].items() if k != "depends"},) for p in problems]
    descs = [ops.qmv_set([p]) for p in plain]

    def per_launch():
        for d in descs:
            ops.qmv_batch(d)

    per_launch()
    torch.cuda.synchronize()
    want = [t.clone() for t in chain_outputs(problems)]
    for t in chain_outputs(problems):
        t.fill_(3.0)
    plan = ops.QmvPlan(problems)
    plan.run()
    torch.cuda.synchronize()
    same = all(torch.equal(a, b) for a, b in zip(chain_outputs(problems), want))
    g = graph_of(torch, per_launch)
    t_launch = timed(torch, g.replay, reps, 3, lambda: None) / reps
    t_chain = timed(torch, plan.run, reps, 3, lambda: None) / reps
    assert ops.device_status() == 0
    plan.close()
    forms = {
        "launch_per_gemv": {"value": nbytes / t_launch / 1e9, "unit": "GB/s", "ms_per_step": t_launch * 1e3,
                            "launches_per_step": len(problems),
                            "mode": "one launch per GEMV, programmatic dependent launch, cuda-graph replay"},
        "chained_launch": {"value": nbytes / t_chain / 1e9, "unit": "GB/s", "ms_per_step": t_chain * 1e3,
                           "launches_per_step": 1, "mode": "one cooperative launch, dependencies waited for on chip"},
    }
    best = max(forms, key=lambda k: forms[k]["value"])
    gbs = forms[best]["value"]
    # `value` is the faster of the two ways this library runs a dependent chain; both are listed.
    return {"workload": f"{layers} decoder layers (8B shapes) as a dependent chain of {len(problems)} fused GEMVs",
            "value": gbs, "unit": "GB/s", "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "form": best,
            "ms_per_step": forms[best]["ms_per_step"], "launches_per_step": forms[best]["launches_per_step"],
            "bytes_per_step": nbytes, "launch_per_gemv": forms["launch_per_gemv"],
            "chained_launch": forms["chained_launch"], "bit_identical_to_launch_per_gemv": bool(same)}


def bench_qmm(torch, dist, ops, synth, args, dev, pk, key):
    """QMM on one config's shapes on one GPU."""
    cfg = synth.CONFIGS[key]
    M = cfg.M
    out = {"config": key, "M": M, "shapes": []}
    steps = max(3, min(args.steps, 10))
    tot_flops, tot_t = 0.0, 0.0
    e2e_t, e2e_flops, h2d, d2h = 0.0, 0.0, 0, 0
    for p in cfg.projs:
        flops = synth.qmm_flops(p.K, p.N, M)
        codes, s, b = make_linear(torch, ops, p.N, p.K, synth.seed_for("w", key, p.name), dev)
        g = torch.Generator(device=dev).manual_seed(synth.seed_for("x", key, p.name))
        x = torch.randn((M, p.K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        y = torch.empty((M, p.N), dtype=torch.bfloat16, device=dev)
        t = timed(torch, lambda: ops.qmm(codes, s, b, x, out=y), steps, 3, lambda: None) / steps
        rec = {"name": p.name, "K": p.K, "N": p.N, "ms": t * 1e3, "tflops": flops / t / 1e12}
        if not args.no_e2e:
            # end to end: the activations come from pinned host memory and the product goes back,
            # inside the timed region (PCIe-bound for the large shapes, and reported as such)
            hx = torch.empty((M, p.K), dtype=torch.bfloat16).pin_memory()
            hx.copy_(x)
            hy = torch.empty((M, p.N), dtype=torch.bfloat16).pin_memory()

            def e2e_step():
                x.copy_(hx, non_blocking=True)
                ops.qmm(codes, s, b, x, out=y)
                hy.copy_(y, non_blocking=True)
                torch.cuda.current_stream().synchronize()

            te = timed(torch, e2e_step, 3, 3, lambda: None) / 3
            rec["e2e_ms"] = te * 1e3
            e2e_t += te
            e2e_flops += flops
            h2d += hx.numel() * 2
            d2h += hy.numel() * 2
            del hx, hy
        out["shapes"].append(rec)
        tot_flops += flops
        tot_t += t
        del codes, s, b, x, y
        torch.cuda.empty_cache()
    if key == "C3":
        # q | k | v as the reference keeps them: one row-concatenated weight, here also one GEMM with three
        # outputs (vpq_affine_qmm_qkv_w4g64_bf16). The config's value counts this launch in place of the
        # three separate ones; those stay listed above, and `value_separate_launches` is the sum over them.
        q, k, v = (p for p in cfg.projs if p.name in ("q", "k", "v"))
        codes, s_, b_ = make_linear(torch, ops, q.N + k.N + v.N, q.K, synth.seed_for("w", key, "qkv"), dev)
        x = torch.randn((M, q.K), device=dev).to(torch.bfloat16)
        outs = [torch.empty((M, n), dtype=torch.bfloat16, device=dev) for n in (q.N, k.N, v.N)]
        t = timed(torch, lambda: ops.qmm_qkv(codes, s_, b_, x, q.N, k.N, v.N, outs=outs), steps, 3, lambda: None) / steps
        fl = sum(synth.qmm_flops(p.K, p.N, M) for p in (q, k, v))
        out["shapes"].append({"name": "q|k|v (one GEMM, three outputs)", "K": q.K, "N": q.N + k.N + v.N, "ms": t * 1e3,
                              "tflops": fl / t / 1e12})
        t_sep = sum(r["ms"] for r in out["shapes"] if r["name"] in ("q", "k", "v")) / 1e3
        out["value_separate_launches"] = tot_flops / tot_t / 1e12
        tot_t += t - t_sep
        del codes, s_, b_, x, outs
        torch.cuda.empty_cache()
    assert ops.device_status() == 0
    agg = tot_flops / tot_t / 1e12
    alg_bytes = sum(p.N * p.K // 2 + 4 * p.N * (p.K // 64) + 2 * M * (p.K + p.N) for p in cfg.projs) / len(cfg.projs)
    out.update(metric="int4_qmm_tflops", value=agg, unit="TFLOP/s", n_gpus=1, scaling="weak",
               launches=len(cfg.projs) * (steps + 3),
               roofline={"bound": "tensor", "achieved": agg, "peak": pk["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": agg / pk["bf16_tflops"],
                         "frac_of_sustained": agg / pk["bf16_tflops_sustained"],
                         "peak_source": pk["source"] + " (burst, cuBLAS bf16)",
                         "kernel": "affine_qmm_w4g64_2cta_kernel",
                         "traffic": (QMM_TRAFFIC_RATIO * alg_bytes) if QMM_TRAFFIC_RATIO else None})
    if e2e_t > 0:
        out["e2e"] = {"value": e2e_flops / e2e_t / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": d2h,
                      "note": "one step = every shape once, x from and y to pinned host memory"}
    return out


def bench_qmm_sharded(torch, dist, ops, shard, synth, args, rank, world, dev, pk, comm, keys):
    """The column split on `world` GPUs, strong scaling. Per shape: the unsharded GEMM on this box,
    the fused form (sender warps store finished tiles into every peer's row-major y), GEMM + NCCL
    all-gather whole and in 4 row chunks, the bytes each GPU must receive and the time that takes at
    the link rate, and a bit-identity check of the gathered y against the unsharded kernel."""
    barrier = lambda: dist.barrier()  # noqa: E731
    steps = max(3, min(args.steps, 10))
    out = {"n_gpus": world, "scaling": "strong", "configs": {}, "parity": {"bit_identical": True, "checked": []}}
    for key in keys:
        cfg = synth.CONFIGS[key]
        M = cfg.M
        projs = [p for p in cfg.projs if not (key == "C3" and p.name not in ("gate", "up"))]
        recs, sums = [], {"flops": 0.0, "one_gpu": 0.0, "fused": 0.0, "nccl_allgather": 0.0, "nccl_chunks4": 0.0}
        for p in projs:
            if p.N % (8 * world) or M <= 128:
                continue
            flops = synth.qmm_flops(p.K, p.N, M)
            ns = p.N // world
            # every rank builds the same full weight (same seed), keeps its row shard
            codes, s, b = make_linear(torch, ops, p.N, p.K, synth.seed_for("w", key, p.name), dev)
            g = torch.Generator(device=dev).manual_seed(synth.seed_for("x", key, p.name))
            x = torch.randn((M, p.K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
            y_full = torch.empty((M, p.N), dtype=torch.bfloat16, device=dev)
            t_one = max_over_ranks(torch, dist, world, timed(torch, lambda: ops.qmm(codes, s, b, x, out=y_full),
                                                             steps, 3, barrier), dev) / steps
            lo, hi = shard.shard_rows(p.N, world, rank)
            cs, ss, bs = codes[lo:hi].contiguous(), s[lo:hi].contiguous(), b[lo:hi].contiguous()
            ymine = torch.empty((M, ns), dtype=torch.bfloat16, device=dev)
            t_gemm = max_over_ranks(torch, dist, world, timed(torch, lambda: ops.qmm(cs, ss, bs, x, out=ymine),
                                                              steps, 2, barrier), dev) / steps
            # fused
            y_sym, y_ptr = comm.alloc_symmetric((M, p.N), torch.bfloat16)
            y_sym.zero_()
            torch.cuda.synchronize()
            barrier()
            comm.qmm_fused(cs, ss, bs, x, y_ptr)
            torch.cuda.synchronize()
            ok_fused = bool(torch.equal(y_sym, y_full))
            t_fused = max_over_ranks(torch, dist, world, timed(torch, lambda: comm.qmm_fused(cs, ss, bs, x, y_ptr),
                                                               steps, 3, barrier), dev) / steps
            # GEMM + NCCL
            y_sh = torch.zeros((world, M, ns), dtype=torch.bfloat16, device=dev)
            y_row = torch.zeros((M, p.N), dtype=torch.bfloat16, device=dev)
            comm.qmm(cs, ss, bs, x, y_sh, y_row, 1)
            torch.cuda.synchronize()
            ok_nccl = bool(torch.equal(y_row, y_full))
            t_ag = max_over_ranks(torch, dist, world, timed(torch, lambda: comm.qmm(cs, ss, bs, x, y_sh, None, 1),
                                                            steps, 3, barrier), dev) / steps
            t_ch = max_over_ranks(torch, dist, world, timed(torch, lambda: comm.qmm(cs, ss, bs, x, y_sh, None, 4),
                                                            steps, 3, barrier), dev) / steps
            # a checksum of the gathered result, the same on every rank
            chk = y_sym.view(torch.int16).to(torch.int64).sum().reshape(1)
            allchk = [torch.zeros_like(chk) for _ in range(world)]
            dist.all_gather(allchk, chk)
            ok_sum = all(int(c.item()) == int(allchk[0].item()) for c in allchk)
            flag = torch.tensor([int(ok_fused and ok_nccl and ok_sum)], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            good = bool(int(flag.item()))
            out["parity"]["bit_identical"] = out["parity"]["bit_identical"] and good
            out["parity"]["checked"].append({"shape": f"{key}.{p.name}", "elements": M * p.N, "fused": ok_fused,
                                             "nccl_rowmajor": ok_nccl, "checksum_equal_on_all_ranks": ok_sum})
            recv = (world - 1) * M * ns * 2
            recs.append({"name": p.name, "K": p.K, "N": p.N, "one_gpu_ms": t_one * 1e3, "shard_gemm_only_ms": t_gemm * 1e3,
                         "fused_ms": t_fused * 1e3, "nccl_allgather_ms": t_ag * 1e3, "nccl_chunks4_ms": t_ch * 1e3,
                         "fused_tflops": flops / t_fused / 1e12, "speedup_vs_1gpu": t_one / t_fused,
                         "exchange_bytes_per_gpu": recv,
                         "link_floor_ms": recv / (NVLINK_GBS_MEASURED * 1e9) * 1e3,
                         "link_gbs_over_fused_call": recv / t_fused / 1e9})
            sums["flops"] += flops
            sums["one_gpu"] += t_one
            sums["fused"] += t_fused
            sums["nccl_allgather"] += t_ag
            sums["nccl_chunks4"] += t_ch
            comm.free_symmetric(y_ptr)
            del codes, s, b, x, y_full, y_sym, y_sh, y_row, ymine, cs, ss, bs
            torch.cuda.empty_cache()
        if sums["fused"] > 0:
            f = sums["flops"] / 1e12
            out["configs"][key] = {
                "M": M, "shapes": recs, "one_gpu_tflops": f / sums["one_gpu"],
                "fused_tflops": f / sums["fused"], "nccl_allgather_tflops": f / sums["nccl_allgather"],
                "nccl_chunks4_tflops": f / sums["nccl_chunks4"], "speedup_vs_1gpu": sums["one_gpu"] / sums["fused"],
                "strong_scaling_efficiency": sums["one_gpu"] / sums["fused"] / world}
    assert ops.device_status() == 0
    first = out["configs"].get(keys[0])
    if first:
        out.update(metric="int4_qmm_tflops", value=first["fused_tflops"], unit="TFLOP/s", config=keys[0],
                   speedup_vs_1gpu=first["speedup_vs_1gpu"],
                   roofline={"bound": "tensor", "achieved": first["fused_tflops"] / world, "peak": pk["bf16_tflops"],
                             "unit": "TFLOP/s", "frac": first["fused_tflops"] / world / pk["bf16_tflops"],
                             "peak_source": pk["source"] + " (burst, cuBLAS bf16)", "traffic": None})
    return out


# ------------------------------------------------------------- small single-kernel workloads

def small_case(torch, ops, synth, dev, pk, kind, a):
    def tm(fn, reps):
        return timed(torch, fn, reps, 0, lambda: None) / reps

    if kind == "plan":
        layers = int(a[0]) if a else 4
        xs = {K: torch.randn((1, K), device=dev).to(torch.bfloat16) for K in (4096, 12288)}
        probs = []
        for _ in range(layers):
            for p in synth.CONFIGS["C2"].projs:
                probs.append(rand_weight(torch, p.N, p.K, dev) +
                             (xs[p.K], torch.empty((1, p.N), dtype=torch.bfloat16, device=dev)))
        plan = ops.QmvPlan(probs)
        for _ in range(3):
            plan.run()
        torch.cuda.synchronize()
        t = tm(plan.run, 1)
        nbytes = sum(synth.qmv_bytes(p.K, p.N) for p in synth.CONFIGS["C2"].projs) * layers
        return {"case": "plan", "layers": layers, "us": t * 1e6, "GBs": nbytes / t / 1e9}
    if kind == "decode_chain":
        layers = int(a[0]) if a else 4
        r = bench_decode_chain(torch, ops, synth, dev, pk, layers=layers, reps=3)
        r["case"] = "decode_chain"
        return r
    if kind in ("qmv", "qmv_w8"):
        K, N = int(a[0]), int(a[1])
        n = int(a[2]) if len(a) > 2 else 8
        bits = 8 if kind == "qmv_w8" else 4
        fn = ops.qmv_w8 if bits == 8 else ops.qmv
        x = torch.randn((1, K), device=dev).to(torch.bfloat16)
        sets = [rand_weight(torch, N, K, dev, bits) + (x, torch.empty((1, N), dtype=torch.bfloat16, device=dev))
                for _ in range(n)]
        g = graph_of(torch, lambda: [fn(*p[:4], out=p[4]) for p in sets])
        t = tm(g.replay, 3) / n
        nbytes = N * K * bits // 8 + 4 * N * (K // 64) + 2 * K + 2 * N
        return {"case": kind, "K": K, "N": N, "us": t * 1e6, "GBs": nbytes / t / 1e9}
    if kind == "qmv_batch":
        K, N, M = int(a[0]), int(a[1]), int(a[2])
        n = int(a[3]) if len(a) > 3 else 8
        x = torch.randn((M, K), device=dev).to(torch.bfloat16)
        sets = [rand_weight(torch, N, K, dev) + (x, torch.empty((M, N), dtype=torch.bfloat16, device=dev))
                for _ in range(n)]
        out = {"case": "qmv_batch", "K": K, "N": N, "M": M}
        for name, fn in (("batch", ops.qmv_batch_rows), ("serial", ops.qmv)):
            g = graph_of(torch, lambda fn=fn: [fn(*p[:4], out=p[4]) for p in sets])
            t = tm(g.replay, 3) / n
            out[name + "_us"] = t * 1e6
            out[name + "_weight_GBs"] = synth.qmv_bytes(K, N) / t / 1e9
        out["speedup"] = out["serial_us"] / out["batch_us"]
        return out
    if kind in ("qmm", "qmm_swiglu", "qmm_w8"):
        M, K, N = int(a[0]), int(a[1]), int(a[2])
        reps = int(a[3]) if len(a) > 3 else 3
        x = torch.randn((M, K), device=dev).to(torch.bfloat16)
        codes, s, b = rand_weight(torch, N, K, dev, 8 if kind == "qmm_w8" else 4)
        fn = {"qmm": ops.qmm, "qmm_swiglu": ops.qmm_swiglu, "qmm_w8": ops.qmm_w8}[kind]
        y = torch.empty((M, N // 2 if kind == "qmm_swiglu" else N), dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            fn(codes, s, b, x, out=y)
        torch.cuda.synchronize()
        t = tm(lambda: fn(codes, s, b, x, out=y), reps)
        return {"case": kind, "M": M, "K": K, "N": N, "ms": t * 1e3, "tflops": synth.qmm_flops(K, N, M) / t / 1e12}
    if kind == "moe":
        import numpy as np

        from vpipe_b200 import moe
        T, E, top_k, H, F = (int(v) for v in a[:5])
        reps = int(a[5]) if len(a) > 5 else 3
        tile = ops.qmm_grouped_tile_rows()
        rng = np.random.default_rng(0)
        eid = np.stack([rng.choice(E, size=top_k, replace=False) for _ in range(T)]).reshape(-1).astype(np.int32)
        tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, tile)
        tile2e, srow, sdst = (torch.from_numpy(v).to(dev) for v in (tile2e, srow, sdst))
        hidden = torch.randn((T, H), device=dev).to(torch.bfloat16)
        gu = [t.view(E, 2 * F, -1) for t in rand_weight(torch, E * 2 * F, H, dev)]
        dn = [t.view(E, H, -1) for t in rand_weight(torch, E * H, F, dev)]
        act = torch.empty((npad, F), dtype=torch.bfloat16, device=dev)
        part = torch.empty((T * top_k, H), dtype=torch.bfloat16, device=dev)

        def layer():
            ops.qmm_grouped_gated(*gu, hidden, tile2e, srow, out=act)
            ops.qmm_grouped_down(*dn, act, tile2e, sdst, y_rows=T * top_k, out=part)

        for _ in range(2):
            layer()
        torch.cuda.synchronize()
        t = tm(layer, reps)
        useful = 2.0 * T * top_k * (H * 2 * F + F * H)
        padded = 2.0 * npad * (H * 2 * F + F * H)
        return {"case": kind, "tokens": T, "experts": E, "top_k": top_k, "hidden": H, "ffn": F, "rows_padded": npad,
                "ms": t * 1e3, "tflops_useful": useful / t / 1e12, "tflops_padded": padded / t / 1e12}
    if kind == "streams":
        # the HBM-bound streams of the path: quantizer, dequantizer, requantizer, conversions, on an
        # [N, K] weight (default 12288 x 4096 x 8 copies: every pass moves more than L2 holds)
        N, K = (int(a[0]), int(a[1])) if len(a) >= 2 else (12288, 4096)
        copies = int(a[2]) if len(a) > 2 else 8
        reps = 5
        w = [(torch.randn((N, K), device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        out = {"case": "streams", "N": N, "K": K, "copies": copies, "hbm_peak_GBs": pk["hbm_gbs"]}

        def rate(name, fn, nbytes):
            g = graph_of(torch, fn)   # the calls allocate their outputs: replayed from a graph, the timing is the kernels'
            t = tm(g.replay, reps)
            out[name] = {"us": t * 1e6 / copies, "GBs": nbytes * copies / t / 1e9,
                         "frac_of_hbm_peak": nbytes * copies / t / 1e9 / pk["hbm_gbs"]}

        q4 = [ops.quantize(t) for t in w]
        q8 = [ops.quantize(t, bits=8) for t in w]
        G = K // 64
        rate("quant_w4_g64", lambda: [ops.quantize(t) for t in w], N * K * 2 + N * K // 2 + 4 * N * G)
        rate("quant_w8_g64", lambda: [ops.quantize(t, bits=8) for t in w], N * K * 2 + N * K + 4 * N * G)
        sb4 = [(c, ops.scales_to_bf16(s_), ops.scales_to_bf16(b_)) for c, s_, b_ in q4]
        sb8 = [(c, ops.scales_to_bf16(s_), ops.scales_to_bf16(b_)) for c, s_, b_ in q8]
        dense = torch.empty((N, K), dtype=torch.bfloat16, device=dev)
        rate("dequant_w4g64", lambda: [ops.dequantize(*t, out=dense) for t in sb4], N * K // 2 + 4 * N * G + N * K * 2)
        rate("dequant_w8g64", lambda: [ops.dequantize_any(*t, 8, 64, out=dense) for t in sb8],
             N * K + 4 * N * G + N * K * 2)
        rate("requant_w8_to_w4_g64", lambda: [ops.requant_w8_to_w4(*t) for t in sb8],
             N * K + 4 * N * G + N * K // 2 + 4 * N * G)
        # what the memory system gives torch's own fill and copy kernels on the same sizes (a write-only and a
        # read + write stream), for scale next to the copy rate in MEASURED_PEAKS.json
        rate("torch_fill_bf16", lambda: [dense.fill_(1.0) for _ in range(copies)], N * K * 2)
        rate("torch_copy_bf16", lambda: [dense.copy_(t) for t in w], N * K * 4)
        f32 = [t.float() for t in w[:max(1, copies // 2)]]
        rate("narrow_f32_bf16", lambda: [ops.narrow_f32_bf16(t) for _ in range(copies // len(f32)) for t in f32], N * K * 6)
        return out
    raise SystemExit(__doc__)


SMALL = ("plan", "decode_chain", "qmv", "qmv_w8", "qmv_batch", "qmm", "qmm_swiglu", "qmm_w8", "moe", "streams")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5", "c1"] + list(SMALL),
                    help="c2: the headline line; c3/c4/c5: the GEMM config as the line's metric; the rest: one small case")
    ap.add_argument("shape", nargs="*", help="sizes of a small workload (see the module docstring)")
    ap.add_argument("--with-c5", action="store_true",
                    help="add the C5 GEMM config to the 1-GPU headline line (~10 s; with more GPUs it is always there)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-memory end-to-end pass of the GEMM sections")
    ap.add_argument("--no-plan", action="store_true", help="QMV set as 216 graph-replayed launches")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world, local = dist_env(args)

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import vpipe_b200
    from vpipe_b200 import ops, shard, synth
    vpipe_b200.lib()  # raises if the CUDA library is missing: there is no fallback

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (vpipe_b200 has no CPU path)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    pk = peaks()

    if args.workload in SMALL or args.workload == "c1":
        r = bench_c1(torch, ops, synth, dev, pk) if args.workload == "c1" else \
            small_case(torch, ops, synth, dev, pk, args.workload, args.shape)
        assert ops.device_status() == 0
        print(json.dumps(r), flush=True)
        return

    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = shard.NsplitComm(rank, world, dev)
    parity_ok = True

    if args.workload == "c2":
        q = bench_qmv(torch, dist, ops, synth, args, rank, world, dev, pk)
        torch.cuda.empty_cache()
        line = {
            "metric": "int4_qmv_hbm_gbps", "value": q["value"], "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": q["t"] / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 x bf16 -> f32", "data": "synthetic",
            "config": {"workload": "C2 decode-layer QMV set, 8B Qwen3-style decoder, M=1",
                       "layers": LAYERS, "projections": "q,k,v,gate,up,down",
                       "bytes_per_step": q["bytes_step"], "launch_mode": q["mode"],
                       "l2": "36 layers of distinct weights (3.57 GB) exceed L2; no flush needed",
                       "parallelism": "replicas only" if world > 1 else "1 GPU"},
            "roofline": q["roofline"], "e2e": q["e2e"], "clocks": q["clocks"], "timing": q["timing"],
            "gpu_launches": q["launches_step"] * args.steps * q["timing"]["blocks"],
        }
        if world == 1:
            line["c1"] = bench_c1(torch, ops, synth, dev, pk)
            torch.cuda.empty_cache()
            line["decode_chain"] = bench_decode_chain(torch, ops, synth, dev, pk)
            parity_ok = parity_ok and line["decode_chain"]["bit_identical_to_launch_per_gemv"]
            torch.cuda.empty_cache()
            line["qmm"] = bench_qmm(torch, dist, ops, synth, args, dev, pk, "C4")
            line["qmm_c3"] = bench_qmm(torch, dist, ops, synth, args, dev, pk, "C3")
            if args.with_c5:
                line["qmm_c5"] = bench_qmm(torch, dist, ops, synth, args, dev, pk, "C5")
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline_qmv(synth)
                line["qmm"]["cpu_baseline"] = cpu_baseline_qmm(synth, "C4")
                line["qmm_c3"]["cpu_baseline"] = cpu_baseline_qmm(synth, "C3")
        else:
            # every config BASELINE.json shards: C4, C3 gate / up, C5
            line["qmm"] = bench_qmm_sharded(torch, dist, ops, shard, synth, args, rank, world, dev, pk, comm,
                                            ["C4", "C3", "C5"])
            parity_ok = parity_ok and line["qmm"]["parity"]["bit_identical"]
    else:
        key = args.workload.upper()
        sampler = ClockSampler(dev.index)
        sampler.start()
        if world == 1:
            qmm = bench_qmm(torch, dist, ops, synth, args, dev, pk, key)
            ms = sum(s["ms"] for s in qmm["shapes"])
            extra = {"shapes": qmm["shapes"], "e2e": qmm.get("e2e")}
            launches = qmm["launches"]
        else:
            qmm = bench_qmm_sharded(torch, dist, ops, shard, synth, args, rank, world, dev, pk, comm, [key])
            parity_ok = qmm["parity"]["bit_identical"]
            ms = sum(s["fused_ms"] for s in qmm["configs"][key]["shapes"])
            extra = {"sharded": qmm["configs"][key], "parity": qmm["parity"]}
            launches = len(qmm["configs"][key]["shapes"]) * 5 * max(3, min(args.steps, 10))
        clocks = sampler.stop()
        line = {
            "metric": "int4_qmm_tflops", "value": qmm.get("value"), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "int4 x bf16 -> f32", "data": "synthetic",
            "config": {"workload": f"{key} {synth.CONFIGS[key].what}", "M": synth.CONFIGS[key].M,
                       "l2": "x + y of every shape exceed L2",
                       "parallelism": f"column-split x{world}, fused peer-store senders over NVLink"
                       if world > 1 else "1 GPU"},
            "roofline": qmm.get("roofline"), "clocks": clocks, "gpu_launches": launches,
        }
        line.update(extra)
        if world == 1 and rank == 0 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_qmm(synth, key)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if not parity_ok:
        sys.stderr.write("bench.py: a bit-identity check failed (see the parity fields of the line)\n")
        sys.exit(3)


if __name__ == "__main__":
    main()
