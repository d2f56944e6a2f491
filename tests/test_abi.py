"""CPU tests of the C-ABI library: it loads, exports every symbol the header
declares, validates arguments before touching a device, and fails loudly (no
CPU path) when asked to compute without a GPU."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "vpq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vpq_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(vpq):
    from vpipe_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 20
    L = vpq.lib()
    for n in names:
        assert hasattr(L, n), f"libvpq.so lacks {n}"
    assert set(names) == {s[0] for s in _lib.SYMBOLS}


def test_version_and_status_strings(vpq):
    L = vpq.lib()
    assert L.vpq_version() == 100
    assert vpq.status_string(0) == "ok"
    for code in range(1, 8):
        assert vpq.status_string(code) not in ("ok", "unknown status")


def test_byte_sizes_mirror_the_quantizer(vpq):
    # AffineQuantizer::weight_bytes / scale_bytes, affine-quantizer.h:37-40
    L = vpq.lib()
    assert L.vpq_weight_bytes(12288, 4096, 4) == 12288 * (4096 * 4 // 32) * 4
    assert L.vpq_scale_bytes(12288, 4096, 64) == 12288 * 64 * 2
    assert L.vpq_weight_bytes(16, 128, 8) == 16 * 32 * 4


def test_function_table_uses_reference_names(vpq):
    ops = vpq.ops
    for libname, entry in [("affine_qmv_bf16", "affine_qmv_w4g64"),
                           ("affine_qmv_bf16", "affine_qmv_w4g64_add"),
                           ("affine_qmv_bf16", "affine_qmv_swiglu_w4g64"),
                           ("affine_qmv_bf16", "affine_qmv_qkv_w4g64"),
                           ("affine_qmv_bf16", "affine_qmv_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_w4g32"),
                           ("affine_qmv_bf16", "affine_qmv_w4g32_add"),
                           ("affine_qmv_bf16", "affine_qmv_geglu_w8g64"),
                           ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w8g64"),
                           ("affine_qmv_bf16", "affine_gather_qmv_geglu_w8g64"),
                           ("affine_qmv_bf16", "affine_gather_down_qmv_w8g64"),
                           ("affine_qmv_bf16", "affine_moe_gate_w8g64"),
                           ("affine_qmv_bf16", "affine_grouped_swiglu_w4g64"),
                           ("affine_qmv_bf16", "affine_grouped_down_w4g64"),
                           ("affine_qmv_bf16", "affine_grouped_swiglu_w8g64"),
                           ("affine_qmv_bf16", "affine_grouped_down_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_qkv_rms_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_qkv_rms_w4g32"),
                           ("affine_qmv_bf16", "affine_qmv_w8g32"),
                           ("affine_qmv_bf16", "affine_qmv_w4g64_r8p2"),
                           ("affine_qmv_bf16", "affine_qmv_w8g64_r8p2"),
                           ("affine_qmm_steel_bf16", "affine_qmm_grouped_w8g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_grouped_swiglu_w8g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_grouped_geglu_w8g64"),
                           ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w4w8g64"),
                           ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w8w4g64"),
                           ("affine_dequant_bf16", "affine_dequant_w4g32"),
                           ("affine_dequant_bf16", "affine_requant_w8_to_w4_g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64_rs_acc16"),
                           ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g64_bm64_acc16"),
                           ("affine_qmv_bf16", "affine_qmv_geglu_w4g32"),
                           ("affine_qmv_bf16", "affine_qmv_gelu_mul_w4g32"),
                           ("affine_qmv_bf16", "affine_qmv_qkv_w4g32"),
                           ("affine_qmv_bf16", "affine_qmv_w4g32_q40"),
                           ("affine_qmv_bf16", "affine_qmv_w4g32_add_q40"),
                           ("affine_qmv_bf16", "affine_qmv_geglu_w4g32_q40"),
                           ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_batch_w4g64"),
                           ("affine_qmv_bf16", "affine_qmv_batch4_w4g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm128"),
                           ("affine_qmm_mma_bf16", "affine_qmm_mma_w4g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_geglu_w4g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_geglu_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_geglu_w4g64"),
                           ("affine_qmv_bf16", "affine_qmv_w8g64_add"),
                           ("affine_qmv_bf16", "affine_qmv_swiglu_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_qkv_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_gelu_mul_w8g64"),
                           ("affine_qmv_bf16", "affine_qmv_gelu_mul_w4g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm128"),
                           ("affine_dequant_bf16", "affine_dequant_w4g64"),
                           ("affine_dequant_bf16", "affine_quant_w4_g64"),
                           ("affine_dequant", "affine_quant_w4_g64"),
                           ("affine_dequant_bf16", "affine_dequant_w8g64"),
                           ("affine_dequant_bf16", "affine_dequant_w8g32"),
                           ("affine_dequant_bf16", "affine_quant_w8_g64"),
                           ("affine_dequant", "affine_quant_w4_g32"),
                           ("affine_qmv_bf16", "affine_qmv_qkv_rms_w4g64"),
                           ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w4g64"),
                           ("affine_qmv_bf16", "affine_gather_qmv_geglu_w4g64"),
                           ("affine_qmv_bf16", "affine_gather_down_qmv_w4g64"),
                           ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g32"),
                           ("affine_qmm_steel_bf16", "affine_qmm_geglu_w4g32"),
                           ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g32")]:
        fn = ops.function(libname, entry)
        assert fn, (libname, entry)
        assert vpq.lib().vpq_function_name(fn).decode() == entry
    # unknown names give an invalid handle, as the reference's .valid()==false
    assert not ops.function("affine_qmv_bf16", "no_such_entry")
    assert not ops.function("no_such_library", "affine_qmv_w4g64")
    assert "no entry" in vpq.lib().vpq_last_error().decode()


def test_argument_validation_happens_before_any_device_work(vpq):
    L = vpq.lib()
    buf = (C.c_ubyte * 4096)()
    p = C.addressof(buf)
    p16 = (p + 15) & ~15
    INVALID, ALIGN, UNSUP = 1, 2, 3
    # null pointers
    assert L.vpq_affine_qmv_w4g64_bf16(None, p16, p16, p16, p16, 64, 8, 1, None) == INVALID
    assert L.vpq_affine_qmm_w4g64_bf16(p16, p16, p16, None, p16, 64, 8, 1, None) == INVALID
    assert L.vpq_affine_dequant_w4g64_bf16(p16, None, p16, p16, 64, 8, None) == INVALID
    assert L.vpq_affine_quant_w4_g64(p16, 1, p16, p16, None, 64, 8, 1.0, None) == INVALID
    # K must be a positive multiple of the group size (affine-quantizer.cc:57)
    assert L.vpq_affine_quant_w4_g64(p16, 1, p16, p16, p16, 96, 8, 1.0, None) == INVALID
    assert L.vpq_affine_qmv_w4g64_bf16(p16, p16, p16, p16, p16, 100, 8, 1, None) == INVALID
    assert L.vpq_affine_qmm_w4g64_bf16(p16, p16, p16, p16, p16, 64, 0, 1, None) == INVALID
    assert L.vpq_affine_dequant_w4g64_bf16(p16, p16, p16, p16, -64, 8, None) == INVALID
    assert "K%64" in L.vpq_last_error().decode()
    # alignment
    assert L.vpq_affine_qmv_w4g64_bf16(p16 + 4, p16, p16, p16, p16, 64, 8, 1, None) == ALIGN
    assert L.vpq_affine_qmm_w4g64_bf16(p16, p16, p16, p16 + 8, p16, 64, 8, 1, None) == ALIGN
    # outside the supported range
    assert L.vpq_affine_qmv_w4g64_bf16(p16, p16, p16, p16, p16, 65536, 8, 1, None) == UNSUP
    # fused stores: residual missing, odd N for swiglu, row counts beyond N
    assert L.vpq_affine_qmv_w4g64_bf16_add(p16, p16, p16, p16, p16, 64, 8, 1, None, None) == INVALID
    assert L.vpq_affine_qmv_swiglu_w4g64_bf16(p16, p16, p16, p16, p16, 64, 7, 1, None) == INVALID
    assert L.vpq_affine_qmv_qkv_w4g64_bf16(p16, p16, p16, p16, p16, p16, p16, 64, 0, 8, 8, 1, None) == INVALID
    assert L.vpq_affine_qmv_qkv_w4g64_bf16(p16, p16, p16, p16, p16, None, p16, 64, 8, 8, 8, 1, None) == INVALID
    assert L.vpq_affine_qmm_swiglu_w4g64_bf16(p16, p16, p16, p16, p16, 64, 9, 4, None) == INVALID
    assert L.vpq_affine_qmm_geglu_w4g64_bf16(p16, p16, p16, p16, p16, 64, 9, 4, None) == INVALID
    assert L.vpq_affine_qmm_swiglu_w8g64_bf16(p16, p16, p16, p16, p16, 96, 8, 4, None) == INVALID
    assert L.vpq_affine_qmm_geglu_w8g64_bf16(None, p16, p16, p16, p16, 64, 8, 4, None) == INVALID
    assert L.vpq_affine_qmv_w8g64_bf16_fused(None, None) == INVALID
    assert L.vpq_affine_qmv_w8g32_bf16_fused(None, None) == INVALID
    assert L.vpq_affine_moe_gate_w8g64_bf16(p16, p16, p16, p16, p16, 96, 1, None) == INVALID   # K % 64
    assert L.vpq_affine_qmv_batch_w4g64_bf16_fused(None, None) == INVALID
    assert L.vpq_affine_qmv_w4g32_bf16_fused(None, None) == INVALID
    assert L.vpq_affine_qmv_w4g32_q40_bf16_fused(None, None) == INVALID
    assert L.vpq_affine_qmm_swiglu_bf16_rs(p16, p16, p16, p16, p16, 64, 64, 4, 4, 40, 16, None) == INVALID
    assert L.vpq_affine_qmm_swiglu_bf16_rs(p16, p16, p16, p16, p16, 64, 64, 4, 5, 64, 0, None) == INVALID
    assert L.vpq_qmm_grouped_tile_rows() == 128
    assert L.vpq_affine_qmm_grouped_w4g64_bf16(p16, p16, p16, p16, p16, 64, 8, 128, None, None, 1, 128, None) == INVALID
    assert L.vpq_affine_qmm_grouped_swiglu_w4g64_bf16(p16, p16, p16, p16, p16, 64, 9, 128, p16, None, 1, 0, None,
                                                      None) == INVALID
    assert L.vpq_affine_qmm_grouped_geglu_w4g64_bf16(p16, p16, p16, p16, p16, 64, 8, 128, p16, p16, 1, 0, None,
                                                     None) == INVALID
    assert L.vpq_affine_qmv_geglu_w4g64_bf16(p16, p16, p16, p16, p16, 64, 7, 1, None) == INVALID
    assert L.vpq_affine_qmv_gelu_mul_w4g64_bf16(p16, p16, p16, p16, p16, 64, 8, 1, None, None) == INVALID
    assert L.vpq_affine_qmv_batch_w4g64_bf16(p16, p16, p16, p16, None, 64, 8, 4, None) == INVALID
    assert L.vpq_affine_qmv_batch_w4g64_bf16(p16, p16, p16, p16 + 2, p16, 64, 8, 4, None) == ALIGN
    assert L.vpq_affine_qmv_w8g64_bf16(p16, p16, p16, p16, p16, 32768, 8, 1, None) == UNSUP
    # format twins: width and group are validated as AffineQuantizer::quantize_linear does
    assert L.vpq_affine_quant(p16, 1, p16, p16, p16, 64, 8, 3, 64, 1.0, None) == UNSUP
    assert L.vpq_affine_quant(p16, 1, p16, p16, p16, 48, 8, 8, 32, 1.0, None) == INVALID
    assert L.vpq_affine_dequant_bf16(p16, p16, p16, p16, 64, 8, 8, 16, None) == UNSUP
    # nsplit argument checks need no communicator
    assert L.vpq_affine_qmm_w4g64_bf16_nsplit(None, p16, p16, p16, p16, p16, None, 64, 8, 1, 1, None) == INVALID
    assert L.vpq_dispatch(None, None, None) == INVALID


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful without a GPU")
def test_no_cpu_fallback_without_a_gpu(vpq):
    """Valid arguments but no device: a loud VPQ_ERR_CUDA, never a silent CPU result."""
    L = vpq.lib()
    buf = (C.c_ubyte * 65536)()
    p16 = (C.addressof(buf) + 15) & ~15
    CUDA = 4
    assert L.vpq_affine_qmv_w4g64_bf16(p16, p16, p16, p16, p16, 64, 8, 1, None) == CUDA
    assert "no CPU path" in L.vpq_last_error().decode() or "CUDA" in L.vpq_last_error().decode()
    assert L.vpq_affine_qmm_w4g64_bf16(p16, p16, p16, p16, p16, 64, 8, 1, None) == CUDA
    assert L.vpq_affine_dequant_w4g64_bf16(p16, p16, p16, p16, 64, 8, None) == CUDA
    assert L.vpq_affine_quant_w4_g64(p16, 1, p16, p16, p16, 64, 8, 1.0, None) == CUDA
    with pytest.raises(Exception):
        vpq.ops.qmv(torch.zeros(8, 8, dtype=torch.int32), torch.zeros(8, 1), torch.zeros(8, 1),
                    torch.zeros(1, 64))


def test_python_front_end_refuses_cpu_tensors(vpq):
    with pytest.raises(Exception):
        vpq.ops.dequantize(torch.zeros(8, 8, dtype=torch.int32), torch.zeros(8, 1), torch.zeros(8, 1))


def test_descriptor_extensions_are_validated_on_the_host(vpq):
    """The plan dependency, the RMSNorm prologue and the expert gather of a GEMV descriptor are
    checked before any device work; the other GEMV kernels refuse them."""
    from vpipe_b200 import _lib
    L = vpq.lib()
    d = _lib.LinearDesc()
    d.w, d.scales, d.biases, d.x, d.y = 0x1000, 0x2000, 0x3000, 0x4000, 0x5000
    d.K, d.N, d.M = 128, 32, 1
    d.depends = 1                       # honoured by plans only
    assert L.vpq_affine_qmv_w4g64_bf16_batch(C.byref(d), 1, None) == 3
    assert b"depends" in L.vpq_last_error()
    d.depends = 0
    d.norm_w = 0x6008                   # not 16-byte aligned
    assert L.vpq_affine_qmv_w4g64_bf16_batch(C.byref(d), 1, None) == 2
    d.norm_w = 0
    d.expert, d.experts = 0x7000, 0    # an expert gather needs the number of slabs
    assert L.vpq_affine_qmv_w4g64_bf16_batch(C.byref(d), 1, None) == 1
    assert L.vpq_affine_qmv_w8g64_bf16_fused(C.byref(d), None) == 1     # the 8-bit kernel takes the gather too
    d.experts = 4
    assert L.vpq_affine_qmv_batch_w4g64_bf16_fused(C.byref(d), None) == 3   # the small-batch kernel does not
    d.expert, d.experts = 0, 0
    d.norm_w = 0x6008
    assert L.vpq_affine_qmv_w8g64_bf16_fused(C.byref(d), None) == 2     # ... and the RMSNorm prologue (aligned weights)
    assert L.vpq_affine_qmv_batch_w4g64_bf16_fused(C.byref(d), None) == 2   # the small-batch kernel likewise
    d.norm_w = 0x6000


def test_qkv_gemm_and_format_gemm_validate_their_arguments(vpq):
    L = vpq.lib()
    p = 0x10000
    # q and k row counts must be multiples of 128
    assert L.vpq_affine_qmm_qkv_w4g64_bf16(p, p, p, p, p, p, p, 1024, 100, 128, 128, 256, None) == 3
    assert L.vpq_affine_qmm_qkv_w4g64_bf16(p, p, p, p, None, p, p, 1024, 128, 128, 128, 256, None) == 1
    assert L.vpq_affine_qmm_bf16(p, p, p, p, p, 1024, 64, 256, 5, 64, 0, None) == 1      # bits
    assert L.vpq_affine_qmm_bf16(p, p, p, p, p, 1024, 64, 256, 4, 48, 0, None) == 1      # group
    assert L.vpq_affine_qmm_bf16(p, p, p, p, p, 1024, 63, 256, 4, 32, 2, None) == 1      # a gated store needs an even N
    assert L.vpq_wait_probe(0, 1000, None) == 1
    assert L.vpq_peer_barrier_probe(None, 2, 1, 100, None) == 1


# Every kernel entry point of the reference's quant shaders (gpu-kernels/metal/quant/*.metal, plain
# `kernel void` definitions and the names its instantiation macros produce), bf16 libraries. The legacy
# f16-only affine_qmm_w4g64 (library affine_qmm, which has no bf16 build) is the one name left out.
REFERENCE_QUANT_KERNELS = [
    ("affine_dequant_bf16", "affine_dequant_w4g32"),
    ("affine_dequant_bf16", "affine_dequant_w4g64"),
    ("affine_dequant_bf16", "affine_dequant_w8g32"),
    ("affine_dequant_bf16", "affine_dequant_w8g64"),
    ("affine_qmv_bf16", "affine_gather_down_qmv_w4g64"),
    ("affine_qmv_bf16", "affine_gather_down_qmv_w8g64"),
    ("affine_qmv_bf16", "affine_gather_qmv_geglu_w4g64"),
    ("affine_qmv_bf16", "affine_gather_qmv_geglu_w8g64"),
    ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w4g64"),
    ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w4w8g64"),
    ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w8g64"),
    ("affine_qmv_bf16", "affine_gather_qmv_swiglu_w8w4g64"),
    ("affine_qmv_bf16", "affine_grouped_down_w4g64"),
    ("affine_qmv_bf16", "affine_grouped_down_w8g64"),
    ("affine_qmv_bf16", "affine_grouped_swiglu_w4g64"),
    ("affine_qmv_bf16", "affine_grouped_swiglu_w8g64"),
    ("affine_qmv_bf16", "affine_moe_gate_w8g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_geglu_w4g32"),
    ("affine_qmm_steel_bf16", "affine_qmm_geglu_w4g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_geglu_w8g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_grouped_geglu_w4g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_grouped_geglu_w8g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_grouped_swiglu_w4g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_grouped_swiglu_w8g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_grouped_w4g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_grouped_w8g64"),
    ("affine_qmm_mma_bf16", "affine_qmm_mma_w4g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g32"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm128"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm64"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm64_acc16"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g32"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g64_bm128"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g64_bm64"),
    ("affine_qmm_steel_bf16", "affine_qmm_steel_w8g64_bm64_acc16"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_acc16"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm128"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64_acc16"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64_rs"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64_rs_acc16"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_acc16"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm128"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64_acc16"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64_rs"),
    ("affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64_rs_acc16"),
    ("affine_qmv_bf16", "affine_qmv_batch4_swiglu_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch4_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch4_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_batch4_xp_swiglu_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch4_xp_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch4_xp_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_tg4_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_tg4_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_tg_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xd_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xd_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xh16_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xh_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xp1_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xp2_swiglu_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xp2_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch8_xp2_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_batch_geglu_w4g32"),
    ("affine_qmv_bf16", "affine_qmv_batch_geglu_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch_swiglu_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch_w4g32"),
    ("affine_qmv_bf16", "affine_qmv_batch_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_batch_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_geglu_w4g32"),
    ("affine_qmv_bf16", "affine_qmv_geglu_w4g32_q40"),
    ("affine_qmv_bf16", "affine_qmv_geglu_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_geglu_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_gelu_mul_w4g32"),
    ("affine_qmv_bf16", "affine_qmv_gelu_mul_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_gelu_mul_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_qkv_rms_w4g32"),
    ("affine_qmv_bf16", "affine_qmv_qkv_rms_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_qkv_rms_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_qkv_w4g32"),
    ("affine_qmv_bf16", "affine_qmv_qkv_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_qkv_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_swiglu_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_swiglu_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_w4g32"),
    ("affine_qmv_bf16", "affine_qmv_w4g32_add"),
    ("affine_qmv_bf16", "affine_qmv_w4g32_add_q40"),
    ("affine_qmv_bf16", "affine_qmv_w4g32_q40"),
    ("affine_qmv_bf16", "affine_qmv_w4g64"),
    ("affine_qmv_bf16", "affine_qmv_w4g64_add"),
    ("affine_qmv_bf16", "affine_qmv_w8g32"),
    ("affine_qmv_bf16", "affine_qmv_w8g64"),
    ("affine_qmv_bf16", "affine_qmv_w8g64_add"),
    ("affine_dequant_bf16", "affine_quant_w4_g32"),
    ("affine_dequant_bf16", "affine_quant_w4_g64"),
    ("affine_dequant_bf16", "affine_quant_w8_g32"),
    ("affine_dequant_bf16", "affine_quant_w8_g64"),
    ("affine_dequant_bf16", "affine_requant_w8_to_w4_g64"),
]


def test_every_reference_quant_kernel_name_resolves(vpq):
    ops = vpq.ops
    assert len(REFERENCE_QUANT_KERNELS) == 103
    for libname, entry in REFERENCE_QUANT_KERNELS:
        assert ops.function(libname, entry), (libname, entry)
