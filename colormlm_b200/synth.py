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


def hc_params(g: np.random.Generator, hidden: int, hc: int = 4, head: bool = False):
    """Hyper-connection parameters of one site: (fn [(2 + hc) * hc or hc, hc * hidden], scale [3 or 1], base)."""
    rows = hc if head else (2 + hc) * hc
    fn = g.standard_normal((rows, hc * hidden), dtype=np.float32) * np.float32(0.02)
    scale = g.uniform(0.2, 0.8, size=1 if head else 3).astype(np.float32)
    base = g.uniform(-1.0, 1.0, size=rows).astype(np.float32)
    return fn, scale, base


def hc_streams(g: np.random.Generator, n_tokens: int, hidden: int, hc: int = 4) -> np.ndarray:
    """The state of a token: hc streams [n_tokens, hc, hidden], F32."""
    return g.standard_normal((n_tokens, hc, hidden), dtype=np.float32)


def head_weight_bf16(g: np.random.Generator, vocab: int, hidden: int, std: float = 0.02) -> np.ndarray:
    return f32_to_bf16_bits((g.standard_normal((vocab, hidden), dtype=np.float32) * np.float32(std)))


# ---- expert pages from a counter: the same bytes on the GPU (torch integer ops) and on the host ------
# The benchmark holds thousands of pages (48 GB); drawing them with numpy and uploading them would take
# minutes, so a page is a function of (layer, expert, byte position) that both sides can evaluate:
# every 32-bit word is a mixed counter (the finaliser of MurmurHash3 over word index xor page key), the
# E2M1 code bytes take it as it is (uniform over the 16 codes per nibble), the scale bytes (the last
# 1 KB of every 17 408-byte unit of the expert page) become 119 + byte % 5 (2^-8 .. 2^-4).  The page is in
# the byte order the GPU reads (pages.py); ``hashed_tensor_page`` converts it for the CPU oracle.

UNIT_BYTES, UNIT_STRIDE = 16384, 17408


def page_key(layer: int, expert: int, seed: int = 0x5314) -> int:
    return (seed * 0x01000193 + layer * 0x10001 + expert * 0x9E3779B1 + 0x7F4A7C15) & 0xFFFFFFFF


def _mix32_np(h: np.ndarray) -> np.ndarray:
    m = np.uint64(0xFFFFFFFF)
    h = (h * np.uint64(0x9E3779B1)) & m
    h ^= h >> np.uint64(15)
    h = (h * np.uint64(0x85EBCA77)) & m
    h ^= h >> np.uint64(13)
    h = (h * np.uint64(0xC2B2AE3D)) & m
    h ^= h >> np.uint64(16)
    return h


def hashed_expert_page(layer: int, expert: int, hidden: int, inter: int, seed: int = 0x5314) -> np.ndarray:
    """The expert page (GPU byte order) of (layer, expert) as uint8, on the host."""
    n_bytes = ExpertPageLayout(hidden, inter).page_bytes
    words = _mix32_np(np.arange(n_bytes // 4, dtype=np.uint64) ^ np.uint64(page_key(layer, expert, seed)))
    page = words.astype(np.uint32).view(np.uint8).copy()
    units = page.reshape(-1, UNIT_STRIDE)
    units[:, UNIT_BYTES:] = 119 + units[:, UNIT_BYTES:] % 5
    return page


def hashed_tensor_page(layer: int, expert: int, hidden: int, inter: int, seed: int = 0x5314) -> np.ndarray:
    """The same page as the six checkpoint tensors (what the CPU oracle reads)."""
    import ctypes as C

    from . import _lib as L

    page = hashed_expert_page(layer, expert, hidden, inter, seed)
    out = np.empty_like(page)
    L.check(L.lib().s14_mxfp4_expert_page_to_tensors(hidden, inter, page.ctypes.data_as(C.c_void_p),
                                                     out.ctypes.data_as(C.c_void_p)))
    return out


class HashedPageWriter:
    """Fills device buffers with hashed expert pages (torch integer ops, no host copy)."""

    def __init__(self, torch, hidden: int, inter: int, device="cuda", seed: int = 0x5314):
        self.torch, self.hidden, self.inter, self.seed = torch, hidden, inter, seed
        self.n_bytes = ExpertPageLayout(hidden, inter).page_bytes
        self.idx = torch.arange(self.n_bytes // 4, dtype=torch.int64, device=device)
        pos = torch.arange(self.n_bytes, dtype=torch.int64, device=device) % UNIT_STRIDE
        self.scale_at = pos >= UNIT_BYTES

    def fill(self, out, layer: int, expert: int) -> None:
        """out: uint8 tensor of page_bytes on the device."""
        m = 0xFFFFFFFF
        h = self.idx ^ page_key(layer, expert, self.seed)
        h = (h * 0x9E3779B1) & m
        h ^= h >> 15
        h = (h * 0x85EBCA77) & m
        h ^= h >> 13
        h = (h * 0xC2B2AE3D) & m
        h ^= h >> 16
        b = h.to(self.torch.int32).view(self.torch.uint8)
        out.copy_(self.torch.where(self.scale_at, 119 + b % 5, b))


# ---- head weight from a counter (the same bits on the host and on the GPU) ----------------------------

HEAD_KEY = 0x48EAD001


def _head_bits_from_hash(h, xp):
    """BF16 bits from mixed 32-bit words: sign and mantissa from the word, exponent 117..121 (|w| in
    2^-10 .. 2^-5), so that a 4096-long dot product with unit-scale activations stays around one."""
    return (h & 0x807F) | ((117 + ((h >> 8) % 5)) << 7)


def hashed_head_rows(row0: int, n_rows: int, hidden: int) -> np.ndarray:
    """Rows [row0, row0 + n_rows) of the head weight as BF16 bits (uint16), on the host."""
    idx = np.arange(row0 * hidden, (row0 + n_rows) * hidden, dtype=np.uint64)
    h = _mix32_np(idx ^ np.uint64(HEAD_KEY))
    return _head_bits_from_hash(h, np).astype(np.uint16).reshape(n_rows, hidden)


def hashed_head_rows_torch(torch, row0: int, n_rows: int, hidden: int, device="cuda", chunk_rows: int = 8192):
    """The same rows on the device (int16 tensor holding the BF16 bits), built in chunks."""
    out = torch.empty((n_rows, hidden), dtype=torch.int16, device=device)
    m = 0xFFFFFFFF
    for r in range(0, n_rows, chunk_rows):
        n = min(chunk_rows, n_rows - r)
        h = torch.arange((row0 + r) * hidden, (row0 + r + n) * hidden, dtype=torch.int64, device=device) ^ HEAD_KEY
        h = (h * 0x9E3779B1) & m
        h ^= h >> 15
        h = (h * 0x85EBCA77) & m
        h ^= h >> 13
        h = (h * 0xC2B2AE3D) & m
        h ^= h >> 16
        bits = _head_bits_from_hash(h, torch)
        out[r:r + n] = (bits - ((bits >> 15) << 16)).to(torch.int16).view(n, hidden)  # two's complement of the 16 bits
    return out
