"""Generates tests/golden/*.npz from the REFERENCE's own shader source.

Run in a container that has the reference checkout (it is compiled as C++ by
oracle/Makefile into oracle/_ref/libvpq_ref.so):

    python tests/golden/make_golden.py

The fixtures hold small inputs and the outputs the reference source produced
for them, so the oracle (and through it the CUDA kernels) can be pinned on
machines where the reference checkout is absent. Inputs follow the
distributions of the reference's tests: N(0, 0.02) weights for the quantizer
round trip (tests/unit-tests/model-quantize-roundtrip.cc:84-164) and random
nibbles with bf16 scales U(0.005,0.02) / biases U(-0.1,0.1) for the dequantizer
(tests/unit-tests/metal-compute-gemm-mma.cc:253-288).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from vpipe_b200 import synth  # noqa: E402


def quant_case(name, N, K, bf16, clip, seed, special=False):
    w = synth.weight_f32(N, K, seed)
    if bf16:
        bits = synth.f32_to_bf16_bits(w)
    else:
        bits = w.astype(np.float16).view(np.uint16)
    if special:
        z, nz = (0x0000, 0x8000)
        bits[0, :64] = z                       # all +0
        bits[1, :64] = nz                      # all -0
        bits[2, :64] = bits[2, 0]              # constant non-zero group
        bits[3, 0:64:2], bits[3, 1:64:2] = nz, z   # -0 first, then +0
        bits[4, 0:64:2], bits[4, 1:64:2] = z, nz   # +0 first
        bits[5, :64] = np.where(np.arange(64) % 3 == 0, nz, bits[5, :64] & 0x7FFF)  # min is -0
        bits[6, 1] = bits[6, 0]                # duplicate extremes
    codes, s, b = oracle.quant_w4_g64(bits, bf16, clip, use_ref=True)
    out = {"w_bits": bits, "src_is_bf16": np.array(int(bf16)), "clip": np.array(clip, np.float32),
           "codes": codes, "scales_f16": s, "biases_f16": b}
    if bf16:
        sb, bb = oracle.f16_to_bf16(s), oracle.f16_to_bf16(b)
        out["scales_bf16"], out["biases_bf16"] = sb, bb
        out["deq_bf16"] = oracle.dequant_bf16(codes, sb, bb, use_ref=True)
    else:
        out["deq_f16"] = oracle.dequant_f16_ref(codes, s, b)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


def dequant_case(name, N, K, seed):
    codes, s, b = synth.random_qweight(N, K, seed)
    # include extreme scale/bias pairs: tiny scale vs large bias and the reverse
    s[0, 0], b[0, 0] = 0x0080, 0x3F80      # smallest normal bf16 scale, bias 1.0
    s[1, 0], b[1, 0] = 0x3F80, 0x0080
    s[2, 0], b[2, 0] = 0x0000, 0xBF80      # zero scale
    s[3, 0], b[3, 0] = 0x3C23, 0x8000      # bias -0
    out = {"codes": codes, "scales_bf16": s, "biases_bf16": b,
           "deq_bf16": oracle.dequant_bf16(codes, s, b, use_ref=True)}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


def twin_case(name, N, K, bits, group, bf16, clip, seed):
    """The other (bits, group) instantiations of the quantizer template and their dequantizers
    (affine_dequant.metal:60-135, 191-225, 303-306)."""
    w = synth.weight_f32(N, K, seed)
    wb = synth.f32_to_bf16_bits(w) if bf16 else w.astype(np.float16).view(np.uint16)
    wb[0, :group] = 0x8000                     # all -0
    wb[1, :group] = wb[1, 0]                   # constant group
    wb[2, 0:group:2], wb[2, 1:group:2] = 0x8000, 0x0000
    codes, s, b = oracle.quant(wb, bits, group, bf16, clip, use_ref=True)
    out = {"w_bits": wb, "src_is_bf16": np.array(int(bf16)), "clip": np.array(clip, np.float32),
           "bits": np.array(bits), "group": np.array(group), "codes": codes, "scales_f16": s, "biases_f16": b}
    if bf16:
        sb, bb = oracle.f16_to_bf16(s), oracle.f16_to_bf16(b)
        out["scales_bf16"], out["biases_bf16"] = sb, bb
        out["deq_bf16"] = oracle.dequant_bf16_any(codes, sb, bb, bits, group, use_ref=True)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


def requant_case(name, N, K, seed):
    """affine_requant_w8_to_w4_g64 (affine_dequant.metal:135-189) on 8-bit weights the reference's own
    quantizer produced, with a constant group (scale 0) and an evenly spread one."""
    w = synth.weight_f32(N, K, seed)
    w[0, :64] = 0.25
    w[1, :64] = np.linspace(-1.0, 1.0, 64, dtype=np.float32)
    codes8, s, b = oracle.quant(synth.f32_to_bf16_bits(w), 8, 64, True, 1.0, use_ref=True)
    s8, b8 = oracle.f16_to_bf16(s), oracle.f16_to_bf16(b)
    w4, s4, b4 = oracle.requant_w8_to_w4_g64(codes8, s8, b8, use_ref=True)
    out = {"codes8": codes8, "scales8_bf16": s8, "biases8_bf16": b8, "codes4": w4, "scales4_bf16": s4, "biases4_bf16": b4}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    oracle.build()
    if not oracle.have_ref():
        sys.exit("oracle/_ref/libvpq_ref.so is missing: the reference checkout is needed")
    quant_case("quant_bf16_n24_k256", 24, 256, True, 1.0, 11, special=True)
    quant_case("quant_bf16_n8_k4096", 8, 4096, True, 1.0, 12)
    quant_case("quant_f16_n16_k192", 16, 192, False, 1.0, 13, special=True)
    quant_case("quant_bf16_clip09_n16_k128", 16, 128, True, 0.9, 14, special=True)
    dequant_case("dequant_bf16_n33_k320", 33, 320, 15)
    twin_case("twin_w8g64_bf16_n12_k256", 12, 256, 8, 64, True, 1.0, 16)
    twin_case("twin_w8g32_bf16_n12_k160", 12, 160, 8, 32, True, 0.9, 17)
    twin_case("twin_w4g32_bf16_n12_k160", 12, 160, 4, 32, True, 1.0, 18)
    twin_case("twin_w8g64_f16_n12_k128", 12, 128, 8, 64, False, 1.0, 19)
    requant_case("requant_w8g64_bf16_n10_k320", 10, 320, 20)
