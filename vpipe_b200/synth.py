"""Shapes of the five benchmark configurations and seeded synthetic inputs.

No checkpoint is involved: weights are N(0, 0.02^2) narrowed to bf16 and
quantised with the reference recipe (group 64, F16 scales / biases as on disk,
converted to bf16 as at load); activations are bf16 N(0, 1).
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Proj:
    name: str
    K: int
    N: int


@dataclass(frozen=True)
class Config:
    key: str
    what: str
    M: int
    projs: tuple


CONFIGS = {
    "C1": Config("C1", "single int4 GEMV", 1, (Proj("gemv", 4096, 4096),)),
    "C2": Config("C2", "decode-layer QMV set, 8B Qwen3-style decoder, batch 1", 1, (
        Proj("q", 4096, 4096), Proj("k", 4096, 1024), Proj("v", 4096, 1024),
        Proj("gate", 4096, 12288), Proj("up", 4096, 12288), Proj("down", 12288, 4096))),
    "C3": Config("C3", "prefill QMM, 8B decoder shapes, 2048 tokens", 2048, (
        Proj("q", 4096, 4096), Proj("k", 4096, 1024), Proj("v", 4096, 1024),
        Proj("gate", 4096, 12288), Proj("up", 4096, 12288), Proj("down", 12288, 4096))),
    "C4": Config("C4", "DiT image-model linear stack, 4096 tokens", 4096, (
        Proj("qkv", 4096, 12288), Proj("proj", 4096, 4096),
        Proj("mlp_up", 4096, 16384), Proj("mlp_down", 16384, 4096))),
    "C5": Config("C5", "video DiT linear stack, 65280 tokens", 65280, (
        Proj("qkv", 5120, 15360), Proj("out", 5120, 5120),
        Proj("ffn_up", 5120, 13824), Proj("ffn_down", 13824, 5120))),
}


def qmv_bytes(K: int, N: int, M: int = 1) -> int:
    """Algorithmic bytes of one QMV: codes + scales + biases + x + y."""
    return N * K // 2 + 2 * N * (K // 64) * 2 + M * K * 2 + M * N * 2


def qmm_flops(K: int, N: int, M: int) -> int:
    """Algorithmic flops of one QMM (dequantisation work not counted)."""
    return 2 * M * N * K


def seed_for(*parts) -> int:
    return zlib.crc32("/".join(str(p) for p in parts).encode()) & 0x7FFFFFFF


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=seed))


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even narrowing on the bit pattern (finite inputs)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, np.uint16).astype(np.uint32) << 16).view(np.float32)


def weight_f32(N: int, K: int, seed: int, std: float = 0.02) -> np.ndarray:
    return (_rng(seed).standard_normal((N, K), dtype=np.float32) * np.float32(std))


def activations_bf16(M: int, K: int, seed: int) -> np.ndarray:
    """bf16 bit patterns of x ~ N(0, 1)."""
    return f32_to_bf16_bits(_rng(seed).standard_normal((M, K), dtype=np.float32))


def random_qweight(N: int, K: int, seed: int):
    """Random nibbles with bf16 scales U(0.005, 0.02) and biases U(-0.1, 0.1):
    the distribution of the reference's own QMM tests
    (tests/unit-tests/metal-compute-gemm-mma.cc:253-288). Returns
    (codes u32 [N,K/8], scales bf16 bits, biases bf16 bits)."""
    g = _rng(seed)
    nib = g.integers(0, 16, size=(N, K), dtype=np.uint32)
    codes = np.zeros((N, K // 8), np.uint32)
    for i in range(8):
        codes |= nib[:, i::8] << np.uint32(4 * i)
    s = f32_to_bf16_bits(g.uniform(0.005, 0.02, size=(N, K // 64)).astype(np.float32))
    b = f32_to_bf16_bits(g.uniform(-0.1, 0.1, size=(N, K // 64)).astype(np.float32))
    return codes, s, b
