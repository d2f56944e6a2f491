#!/usr/bin/env python
"""Benchmark of the 4-bit affine quantized linear on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5]
                    [--impl ours|reference]

Default (what the headline metric is quoted on): the decode-layer QMV set of an
8B Qwen3-style decoder at batch 1 -- q, k, v, gate, up, down at M = 1 -- for all
36 layers with distinct weights (3.57 GB, larger than L2, so everything
streams from HBM). One step = one pass over the 36 layers = 216 GEMVs, run as one
plan launch (vpq_qmv_plan_run); --no-plan replays 216 separate launches as a graph.
`value` is algorithmic GB/s with everything resident in HBM; `e2e` is the same
pass driven through the C ABI with the step's activations copied from pinned
host memory and the result read back, inside the timed region. The same JSON
line carries `qmm`: the tensor-core GEMM on the prefill / DiT shapes in
TFLOP/s (column-split with an NCCL all-gather when N > 1).

With N > 1 (launched under torchrun) the QMV set runs as N independent replicas
(decode at batch 1 does not shard; weak scaling); the QMM section is the part
that is partitioned across GPUs.

Inputs are synthetic: weights N(0, 0.02) quantised with the reference recipe on
the device, activations N(0, 1) bf16; seeded.
"""
from __future__ import annotations

import argparse
import json
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

# DRAM traffic per launch measured once with ncu (dram__bytes_read.sum +
# dram__bytes_write.sum) as a multiple of the algorithmic bytes of that launch, from a 4-layer
# plan (profiles/qmv_plan_c2_4layers.md: 401.4 MB moved for 396.9 MB algorithmic); traffic grows
# in proportion to the layers, so the 36-layer launch is scaled by it. The QMM is tensor-bound
# and its y stays in L2 during a capture, so no DRAM figure is reported for it.
QMV_TRAFFIC_RATIO = 1.011
QMM_TRAFFIC_RATIO = None


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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


# ------------------------------------------------------------------ reference arm

def run_reference(args, rank, world):
    """The reference's CPU path for this op, timed on the host cores. The reference has no
    CPU matmul: this is its f32 dequantise routine plus a plain blocked fp32 GEMM (the
    oracle port), all host threads. Each step is a bounded sample of the workload."""
    if rank != 0:
        return
    import numpy as np

    import oracle
    from vpipe_b200 import synth
    oracle.build()
    cfg = synth.CONFIGS["C2"]
    layer = []
    for p in cfg.projs:   # one decoder layer = the sample processed per step
        codes, s, b = synth.random_qweight(p.N, p.K, synth.seed_for("ref", p.name))
        x = synth.activations_bf16(1, p.K, synth.seed_for("refx", p.name))
        layer.append((codes, s, b, x, synth.qmv_bytes(p.K, p.N, 1)))
    bytes_step = sum(t[4] for t in layer)
    threads = oracle.max_threads()

    def step():
        t = 0.0
        for codes, s, b, x, _ in layer:
            t += oracle.cpu_linear_seconds(codes, s, b, x, threads)[0]
        return t

    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = bytes_step * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": "int4_qmv_hbm_gbps", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int4*bf16->f32", "data": "synthetic",
        "config": {"workload": "C2 decode-layer QMV set, 8B Qwen3-style decoder, M=1",
                   "sample": "1 of 36 layers per step (6 projections, 99.2 MB of weights)"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "one decoder layer (q,k,v,gate,up,down at M=1) per step; "
                                   "f32 dequantise + blocked fp32 GEMM, OpenMP"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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


def bench_qmv(torch, dist, ops, synth, args, rank, world, dev, pk):
    cfg = synth.CONFIGS["C2"]
    layers = []
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
        layers.append(problems[-len(cfg.projs):])
    descs = ops.qmv_set(problems)
    launches_step = len(problems)
    torch.cuda.synchronize()

    def direct():
        ops.qmv_batch(descs)

    # The whole pass as ONE launch (a plan: "encode once, commit many"); failing that, replay the
    # 216 launches as one CUDA graph.
    mode = "plan (1 launch per step)"
    plan = None
    if not args.no_plan:
        try:
            plan = ops.QmvPlan(problems)
            step = plan.run
            launches_step = 1
            step()
            torch.cuda.synchronize()
        except Exception as e:
            plan = None
            mode = f"cuda-graph (plan unavailable: {type(e).__name__})"
    else:
        mode = "cuda-graph"
    try:
        if plan is not None:
            raise StopIteration
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            direct()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            direct()
        step = graph.replay
        step()
        torch.cuda.synchronize()
    except StopIteration:
        pass
    except Exception as e:  # fall back to plain launches, and say so
        mode = f"direct-launches ({type(e).__name__})"
        step = direct

    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    sampler = ClockSampler(dev.index)
    sampler.start()
    t = timed(torch, step, args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    t = max_over_ranks(torch, dist, world, t, dev)
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

    te = timed(torch, e2e_step, args.steps, args.warmup, barrier)
    te = max_over_ranks(torch, dist, world, te, dev)
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
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": te / args.steps * 1e3},
    }


def bench_qmm(torch, dist, ops, synth, args, rank, world, dev, pk, key, comm):
    """QMM on one config's shapes; column-split + all-gather when world > 1."""
    cfg = synth.CONFIGS[key]
    M = cfg.M
    out = {"config": key, "M": M, "shapes": []}
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)
    steps = max(3, min(args.steps, 10))
    tot_flops, tot_t = 0.0, 0.0
    e2e_t, e2e_flops, h2d, d2h = 0.0, 0.0, 0, 0
    for p in cfg.projs:
        if world > 1 and p.N % (8 * world):
            continue
        flops = synth.qmm_flops(p.K, p.N, M)
        ns = p.N // world
        codes, s, b = make_linear(torch, ops, ns, p.K, synth.seed_for("w", key, p.name, rank), dev)
        g = torch.Generator(device=dev).manual_seed(synth.seed_for("x", key, p.name))
        x = torch.randn((M, p.K), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        if world == 1:
            y = torch.empty((M, p.N), dtype=torch.bfloat16, device=dev)
            fn = lambda: ops.qmm(codes, s, b, x, out=y)  # noqa: E731
        elif args.nccl_gather or M <= 128:
            y = torch.empty((world, M, ns), dtype=torch.bfloat16, device=dev)
            fn = lambda: comm.qmm(codes, s, b, x, y, None, args.m_chunks)  # noqa: E731
        else:   # fused: the epilogue stores into every rank's row-major y; no collective
            y, y_ptr = comm.alloc_symmetric((M, p.N), torch.bfloat16)
            fn = lambda: comm.qmm_fused(codes, s, b, x, y_ptr)  # noqa: E731
        t = timed(torch, fn, steps, 3, barrier)
        t = max_over_ranks(torch, dist, world, t, dev) / steps
        rec = {"name": p.name, "K": p.K, "N": p.N, "ms": t * 1e3, "tflops": flops / t / 1e12}
        if world > 1:   # compute alone, for the split between GEMM and the exchange
            ymine = torch.empty((M, ns), dtype=torch.bfloat16, device=dev)
            tc = timed(torch, lambda: ops.qmm(codes, s, b, x, out=ymine), steps, 2, barrier)
            rec["gemm_only_ms"] = max_over_ranks(torch, dist, world, tc, dev) / steps * 1e3
            rec["gather_bytes_per_gpu"] = (world - 1) * M * ns * 2
        if world == 1:
            # end to end: the activations come from pinned host memory and the product goes back,
            # inside the timed region (PCIe-bound for the large shapes, and reported as such)
            try:
                hx = torch.empty((M, p.K), dtype=torch.bfloat16).pin_memory()
                hx.copy_(x)
                hy = torch.empty((M, p.N), dtype=torch.bfloat16).pin_memory()

                def e2e_step():
                    x.copy_(hx, non_blocking=True)
                    ops.qmm(codes, s, b, x, out=y)
                    hy.copy_(y, non_blocking=True)
                    torch.cuda.current_stream().synchronize()

                te = timed(torch, e2e_step, 3, 3, barrier) / 3
                rec["e2e_ms"] = te * 1e3
                e2e_t += te
                e2e_flops += flops
                h2d += hx.numel() * 2
                d2h += hy.numel() * 2
                del hx, hy
            except Exception as e:   # not enough pinned memory for this shape: say so
                rec["e2e_ms"] = None
                rec["e2e_error"] = type(e).__name__
        out["shapes"].append(rec)
        tot_flops += flops
        tot_t += t
        del codes, s, b, x, y
        torch.cuda.empty_cache()
    assert ops.device_status() == 0
    if tot_t > 0:
        agg = tot_flops / tot_t / 1e12
        out.update(metric="int4_qmm_tflops", value=agg, unit="TFLOP/s", n_gpus=world,
                   scaling="strong" if world > 1 else "weak",
                   roofline={"bound": "tensor", "achieved": agg / world, "peak": pk["bf16_tflops"],
                             "unit": "TFLOP/s", "frac": agg / world / pk["bf16_tflops"],
                             "peak_source": pk["source"] + " (burst, cuBLAS bf16)",
                             "kernel": "affine_qmm_w4g64_kernel",
                             "traffic": None})
        if e2e_t > 0:
            out["e2e"] = {"value": e2e_flops / e2e_t / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                          "d2h_bytes_per_step": d2h, "note": "one step = every shape once, x from and y to pinned host memory"}
    return out


def cpu_baseline(synth, seconds_budget=12.0):
    """The oracle port (f32 dequantise + blocked fp32 GEMM, all host threads) on a bounded
    sample of the C2 set: whole decoder layers until the time budget is used."""
    import oracle
    oracle.build()
    cfg = synth.CONFIGS["C2"]
    layer = []
    for p in cfg.projs:
        codes, s, b = synth.random_qweight(p.N, p.K, synth.seed_for("cpu", p.name))
        x = synth.activations_bf16(1, p.K, synth.seed_for("cpux", p.name))
        layer.append((codes, s, b, x))
    bytes_layer = sum(synth.qmv_bytes(p.K, p.N, 1) for p in cfg.projs)
    threads = oracle.max_threads()
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5"],
                    help="c2: the headline line (QMV set + QMM section); c3/c4/c5: QMM only")
    ap.add_argument("--qmm", default="C4", help="config of the QMM section of the headline line")
    ap.add_argument("--m-chunks", dest="m_chunks", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-plan", action="store_true", help="QMV set as 216 graph-replayed launches")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N > 1: GEMM then NCCL all-gather instead of the fused peer-store epilogue")
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
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        comm = shard.NsplitComm(rank, world, dev)
    pk = peaks()

    if args.workload == "c2":
        q = bench_qmv(torch, dist, ops, synth, args, rank, world, dev, pk)
        torch.cuda.empty_cache()
        qmm = bench_qmm(torch, dist, ops, synth, args, rank, world, dev, pk, args.qmm, comm)
        line = {
            "metric": "int4_qmv_hbm_gbps", "value": q["value"], "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": q["t"] / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4*bf16->f32", "data": "synthetic",
            "config": {"workload": "C2 decode-layer QMV set, 8B Qwen3-style decoder, M=1",
                       "layers": LAYERS, "projections": "q,k,v,gate,up,down",
                       "bytes_per_step": q["bytes_step"], "launch_mode": q["mode"],
                       "l2": "36 layers of distinct weights (3.57 GB) exceed L2; no flush needed",
                       "parallelism": "replicas only" if world > 1 else "1 GPU"},
            "roofline": q["roofline"], "e2e": q["e2e"], "clocks": q["clocks"],
            "gpu_launches": q["launches_step"] * args.steps,
            "qmm": qmm,
        }
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(synth)
    else:
        key = args.workload.upper()
        sampler = ClockSampler(dev.index)
        sampler.start()
        qmm = bench_qmm(torch, dist, ops, synth, args, rank, world, dev, pk, key, comm)
        clocks = sampler.stop()
        line = {
            "metric": "int4_qmm_tflops", "value": qmm.get("value"), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sum(s["ms"] for s in qmm["shapes"]),
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "int4*bf16->f32", "data": "synthetic",
            "config": {"workload": f"{key} {synth.CONFIGS[key].what}", "M": synth.CONFIGS[key].M,
                       "l2": "x + y of every shape exceed L2", "m_chunks": args.m_chunks,
                       "parallelism": (f"column-split x{world}, " + ("GEMM + NCCL all-gather" if args.nccl_gather else
                                        "fused peer-store epilogue over NVLink")) if world > 1 else "1 GPU"},
            "roofline": qmm.get("roofline"), "e2e": qmm.get("e2e"), "clocks": clocks, "shapes": qmm["shapes"],
            "gpu_launches": len(qmm["shapes"]) * max(3, min(args.steps, 10)),
        }
    if comm is not None:
        comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
