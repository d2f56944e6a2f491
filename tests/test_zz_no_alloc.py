"""GPU test of the no-allocation GEMV-set entry point. Collected last on purpose: a run that stops
at the first failure has then already run every other test.

Some callers cannot allocate device memory when they call into this library: they live inside a
host whose allocator owns all of HBM, or sit on a latency path where a cudaMalloc (which may
synchronise the device) is unacceptable, and they have no workspace to lend either. For them
vpq_affine_qmv_w4g64_bf16_set_noalloc runs a set of GEMVs in one launch with its descriptor list
in a fixed array inside the library. Here it is called through the C ABI twice in a row (the
second time with different activations, so stale descriptors or stale results would show) and
must give exactly the bytes of the existing per-GEMV entry point. It must pass alone in a fresh
process and after all other tests."""
import ctypes as C

import numpy as np
import pytest
import torch

from vpipe_b200 import synth

pytestmark = pytest.mark.gpu


def _dev_bits(a, dtype=None):
    t = torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a.view(np.int32)).to("cuda:0")
    return t.view(dtype) if dtype is not None else t


def test_noalloc_set_matches_existing_entry_point_twice(vpq, oracle_mod):
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    ops = vpq.ops
    shapes = [(4096, 1024, 1), (4096, 264, 1), (12288, 512, 1), (3840, 48, 1), (1024, 33, 2)]
    problems = []
    for i, (K, N, M) in enumerate(shapes):
        bits = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 7000 + i))
        codes, s, b = oracle_mod.quant_w4_g64(bits, True)
        s, b = oracle_mod.f16_to_bf16(s), oracle_mod.f16_to_bf16(b)
        x = _dev_bits(synth.activations_bf16(M, K, 7100 + i), torch.bfloat16)
        y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda:0")
        problems.append((_dev_bits(codes), _dev_bits(s, torch.bfloat16), _dev_bits(b, torch.bfloat16), x, y))
    descs = ops.qmv_set(problems)
    for call in range(2):
        if call == 1:   # new activations in the same buffers
            for p in problems:
                p[3].copy_(torch.randn(p[3].shape, device="cuda:0").to(torch.bfloat16))
        want = [ops.qmv(p[0], p[1], p[2], p[3]) for p in problems]     # the existing entry point
        for p in problems:
            p[4].fill_(-3.0)
        ops.qmv_set_noalloc(descs)
        torch.cuda.synchronize()
        for p, w in zip(problems, want):
            assert torch.equal(p[4], w), f"call {call}: outputs differ"
    assert ops.device_status() == 0


def _problem(oracle_mod, K, N, M, seed):
    bits = synth.f32_to_bf16_bits(synth.weight_f32(N, K, seed))
    codes, s, b = oracle_mod.quant_w4_g64(bits, True)
    s, b = oracle_mod.f16_to_bf16(s), oracle_mod.f16_to_bf16(b)
    x = _dev_bits(synth.activations_bf16(M, K, seed + 1), torch.bfloat16)
    y = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda:0")
    return (_dev_bits(codes), _dev_bits(s, torch.bfloat16), _dev_bits(b, torch.bfloat16), x, y)


def test_noalloc_back_to_back_calls_with_different_sets_and_no_host_sync(vpq, oracle_mod):
    """Two calls in a row on one stream with nothing between them: the second rewrites the shared
    descriptor array (other weights, other K and N in the same slots) while the first may still be
    running; stream order alone must keep them apart. The first set has exactly 64 rows, the most
    the array holds."""
    torch.cuda.set_device(0)
    ops = vpq.ops
    set_a = [_problem(oracle_mod, 1024, 24, 16, 7300 + 10 * i) for i in range(4)]         # 4 x 16 = 64 rows
    set_b = [_problem(oracle_mod, K, N, M, 7400 + 10 * i)
             for i, (K, N, M) in enumerate([(2048, 40, 1), (512, 264, 3), (4096, 1024, 1), (3840, 17, 2)])]
    want_a = [ops.qmv(p[0], p[1], p[2], p[3]) for p in set_a]
    want_b = [ops.qmv(p[0], p[1], p[2], p[3]) for p in set_b]
    da, db = ops.qmv_set(set_a), ops.qmv_set(set_b)
    torch.cuda.synchronize()
    for rep in range(3):
        ops.qmv_set_noalloc(da)
        ops.qmv_set_noalloc(db)       # no synchronisation in between
        ops.qmv_set_noalloc(da)
        torch.cuda.synchronize()
        for p, w in zip(set_a, want_a):
            assert torch.equal(p[4], w), f"rep {rep}: 64-row set differs"
        for p, w in zip(set_b, want_b):
            assert torch.equal(p[4], w), f"rep {rep}: second set differs"
        for p in set_a + set_b:
            p[4].zero_()
    assert ops.device_status() == 0


def test_noalloc_refuses_to_be_captured_into_a_graph(vpq, oracle_mod):
    """The call copies its descriptors from the host stack with stream-ordered copies; recorded into
    a graph those copies would replay dead stack memory, so a capturing stream is refused with a
    clear error and nothing is enqueued."""
    torch.cuda.set_device(0)
    ops = vpq.ops
    prob = _problem(oracle_mod, 1024, 32, 1, 7500)
    descs = ops.qmv_set([prob])
    ops.qmv_set_noalloc(descs)          # the first call per device stays outside any capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        g.capture_begin()
        try:
            with pytest.raises(vpq.VpqError) as e:
                ops.qmv_set_noalloc(descs, stream=side)
        finally:
            g.capture_end()
    assert e.value.status == 3 and "captur" in str(e.value)
    ops.qmv_set_noalloc(descs)          # and it still works afterwards
    torch.cuda.synchronize()
    assert torch.equal(prob[4], ops.qmv(prob[0], prob[1], prob[2], prob[3]))


def test_noalloc_set_rejects_more_rows_than_its_array_holds(vpq):
    torch.cuda.set_device(0)
    ops = vpq.ops
    K, N = 64, 16
    codes = torch.zeros((N, K // 8), dtype=torch.int32, device="cuda:0")
    s = torch.zeros((N, 1), dtype=torch.bfloat16, device="cuda:0")
    x = torch.zeros((1, K), dtype=torch.bfloat16, device="cuda:0")
    y = torch.zeros((1, N), dtype=torch.bfloat16, device="cuda:0")
    descs = ops.qmv_set([(codes, s, s, x, y)] * 65)
    with pytest.raises(vpq.VpqError) as e:
        ops.qmv_set_noalloc(descs)
    assert e.value.status == 3 and "64" in str(e.value)
