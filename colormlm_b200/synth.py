"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: MXFP4 experts (E2M1 codes uniform over the 16 codes, one UE8M0 scale per
32 drawn from 2^[-8,-4]), FP8 E4M3 matrices (uniform over the 254 non-NaN codes), BF16
router weights ~N(0, 0.02), bias ~U(-0.1, 0.1), F32 activations ~N(0, 1).  They stand in
for the real checkpoint tensors, which are not distributed with the reference.  numpy's
PCG64 generator makes the bytes reproducible on any host."""
from __future__ import annotations

import numpy as np

from ._lib import PAGE_FP8, PAGE_MXFP4
from .pages import ExpertPageLayout


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def activations(g: np.random.Generator, n_tokens: int, hidden: int) -> np.ndarray:
    return g.standard_normal((n_tokens, hidden), dtype=np.float32)


def mxfp4_codes(g: np.random.Generator, n: int, k: int) -> np.ndarray:
    """[n, k/2] bytes; each nibble uniform over the 16 E2M1 codes."""
    return g.integers(0, 256, size=(n, k // 2), dtype=np.uint8)


def mxfp4_scales(g: np.random.Generator, n: int, k: int, lo: int = 119, hi: int = 123) -> np.ndarray:
    """[n, k/32] UE8M0 codes uniform in [lo, hi] (2^-8 .. 2^-4 by default)."""
    return g.integers(lo, hi + 1, size=(n, k // 32), dtype=np.uint8)


def mxfp4_expert_page(g: np.random.Generator, hidden: int, inter: int) -> np.ndarray:
    lay = ExpertPageLayout(hidden, inter, PAGE_MXFP4)
    w1, w3 = mxfp4_codes(g, inter, hidden), mxfp4_codes(g, inter, hidden)
    w2 = mxfp4_codes(g, hidden, inter)
    s1, s3 = mxfp4_scales(g, inter, hidden), mxfp4_scales(g, inter, hidden)
    s2 = mxfp4_scales(g, hidden, inter)
    return lay.pack(w1, w3, w2, s1, s3, s2)


def e4m3_codes(g: np.random.Generator, n: int, k: int) -> np.ndarray:
    """[n, k] bytes uniform over the 254 E4M3FN codes that are not NaN."""
    c = g.integers(0, 254, size=(n, k), dtype=np.uint8)
    c = c + (c >= 0x7F).astype(np.uint8)  # skip 0x7F; 0xFF is never reached
    return c


def fp8_block_scales_ue8m0(g: np.random.Generator, n: int, k: int, lo: int = 119, hi: int = 121) -> np.ndarray:
    return g.integers(lo, hi + 1, size=((n + 127) // 128, (k + 127) // 128), dtype=np.uint8)


def fp8_block_scales_f32(g: np.random.Generator, n: int, k: int) -> np.ndarray:
    """One F32 per 128x128 block, U(0.5, 2) * 2^-7."""
    u = g.uniform(0.5, 2.0, size=((n + 127) // 128, (k + 127) // 128)).astype(np.float32)
    return (u * np.float32(2.0 ** -7)).astype(np.float32)


def fp8_expert_page(g: np.random.Generator, hidden: int, inter: int) -> np.ndarray:
    lay = ExpertPageLayout(hidden, inter, PAGE_FP8)
    return lay.pack(e4m3_codes(g, inter, hidden), e4m3_codes(g, inter, hidden),
                    e4m3_codes(g, hidden, inter), fp8_block_scales_ue8m0(g, inter, hidden),
                    fp8_block_scales_ue8m0(g, inter, hidden), fp8_block_scales_ue8m0(g, hidden, inter))


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even BF16 bit patterns of finite F32 values."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def router_weight_bf16(g: np.random.Generator, n_experts: int, hidden: int, std: float = 0.02) -> np.ndarray:
    return f32_to_bf16_bits((g.standard_normal((n_experts, hidden), dtype=np.float32) * np.float32(std)))


def router_bias(g: np.random.Generator, n_experts: int) -> np.ndarray:
    return g.uniform(-0.1, 0.1, size=n_experts).astype(np.float32)


def head_weight_bf16(g: np.random.Generator, vocab: int, hidden: int, std: float = 0.02) -> np.ndarray:
    return f32_to_bf16_bits((g.standard_normal((vocab, hidden), dtype=np.float32) * np.float32(std)))
