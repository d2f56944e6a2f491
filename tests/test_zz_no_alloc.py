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
