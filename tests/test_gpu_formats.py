"""GPU parity of the format twins (w8g64, w8g32, w4g32) of the quantizer and dequantizer: bit-exact
against the oracle and against fixtures the reference's own shader source produced
(gpu-kernels/metal/quant/affine_dequant.metal:60-135, 243-306), through the C ABI."""
import os

import numpy as np
import pytest
import torch

from vpipe_b200 import synth

from test_gpu_parity import bits16, bits32, dev, to_dev

pytestmark = pytest.mark.gpu

TWINS = ["twin_w8g64_bf16_n12_k256", "twin_w8g32_bf16_n12_k160", "twin_w4g32_bf16_n12_k160",
         "twin_w8g64_f16_n12_k128"]


@pytest.mark.parametrize("name", TWINS)
def test_twin_quantizer_and_dequantizer_on_reference_fixtures(vpq, golden_dir, name):
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    bits, group = int(g["bits"]), int(g["group"])
    w = to_dev(g["w_bits"], torch.bfloat16 if int(g["src_is_bf16"]) else torch.float16)
    codes, s, b = vpq.ops.quantize(w, clip=float(g["clip"]), bits=bits, group=group)
    assert np.array_equal(bits32(codes), g["codes"])
    assert np.array_equal(bits16(s), g["scales_f16"])
    assert np.array_equal(bits16(b), g["biases_f16"])
    if "deq_bf16" in g:
        got = vpq.ops.dequantize_any(to_dev(g["codes"]), to_dev(g["scales_bf16"], torch.bfloat16),
                                     to_dev(g["biases_bf16"], torch.bfloat16), bits, group)
        assert np.array_equal(bits16(got), g["deq_bf16"])


@pytest.mark.parametrize("bits,group", [(8, 64), (8, 32), (4, 32), (4, 64)])
@pytest.mark.parametrize("N,K,bf16,clip", [(33, 1024, True, 1.0), (7, 4096, True, 0.9), (130, 320, False, 1.0)])
def test_twin_quantize_then_dequantize_bit_exact_vs_oracle(vpq, oracle_mod, bits, group, N, K, bf16, clip):
    w = synth.weight_f32(N, K, synth.seed_for("twin", bits, group, N, K))
    wb = synth.f32_to_bf16_bits(w) if bf16 else w.astype(np.float16).view(np.uint16)
    wb[0, :group] = 0x8000 if bf16 else 0x8000        # a group of -0
    wb[1, :group] = wb[1, 0]                          # a constant group: scale 0
    want = oracle_mod.quant(wb, bits, group, bf16, clip)
    got = vpq.ops.quantize(to_dev(wb, torch.bfloat16 if bf16 else torch.float16), clip=clip, bits=bits, group=group)
    assert np.array_equal(bits32(got[0]), want[0])
    assert np.array_equal(bits16(got[1]), want[1])
    assert np.array_equal(bits16(got[2]), want[2])
    sb, bb = oracle_mod.f16_to_bf16(want[1]), oracle_mod.f16_to_bf16(want[2])
    deq = vpq.ops.dequantize_any(got[0], to_dev(sb, torch.bfloat16), to_dev(bb, torch.bfloat16), bits, group)
    assert np.array_equal(bits16(deq), oracle_mod.dequant_bf16_any(want[0], sb, bb, bits, group))


def test_twins_by_reference_names_and_dense_route(vpq, oracle_mod):
    """A w8 layer through the route the reference takes for formats without a fused kernel:
    dequantise once, multiply densely (affine_dequant.metal:100-106)."""
    ops = vpq.ops
    N, K, M = 96, 512, 8
    wb = synth.f32_to_bf16_bits(synth.weight_f32(N, K, 8800))
    w = to_dev(wb, torch.bfloat16)
    codes = torch.empty((N, K // 4), dtype=torch.int32, device=dev())
    s = torch.empty((N, K // 64), dtype=torch.float16, device=dev())
    b = torch.empty_like(s)
    ops.dispatch(ops.function("affine_dequant_bf16", "affine_quant_w8_g64"), [w, codes, s, b], K=K, N=N, clip=1.0)
    want = oracle_mod.quant(wb, 8, 64)
    assert np.array_equal(bits32(codes), want[0]) and np.array_equal(bits16(s), want[1])
    sb, bb = ops.scales_to_bf16(s), ops.scales_to_bf16(b)
    deq = torch.empty((N, K), dtype=torch.bfloat16, device=dev())
    ops.dispatch(ops.function("affine_dequant_bf16", "affine_dequant_w8g64"), [codes, sb, bb, deq], K=K, N=N)
    assert np.array_equal(bits16(deq), oracle_mod.dequant_bf16_any(want[0], bits16(sb), bits16(bb), 8, 64))
    x = to_dev(synth.activations_bf16(M, K, 8801), torch.bfloat16)
    y = (x.float() @ deq.float().T)
    ref = x.float() @ w.float().T
    assert float((y - ref).norm() / ref.norm()) < 0.03      # w8 round-trip bound of the reference's tests
    # unknown width / group: refused, not guessed
    with pytest.raises(vpq.VpqError):
        ops.quantize(w, bits=2, group=64)
