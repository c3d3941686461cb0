"""In-slot byte layout of an expert page.

The reference uploads an expert's six tensors as six separate buffers and never fixes
a layout inside a pool slot (examples/s14_vulkan_numeric.rs:331-366), so the layout is
this library's choice: the three weight matrices first, then the three scale arrays.
Every tensor starts on a 16-byte boundary for the supported sizes.

    MXFP4 page: w1 | w3 | w2 | s1 | s3 | s2   (13 369 344 B at hidden 4096 / inter 2048)
    FP8   page: w1 | w3 | w2 | s1 | s3 | s2   (25 167 360 B at hidden 4096 / inter 2048)

Two byte orders of the same page exist:

* the *tensor page* holds every tensor in the reference's tensor ABI (weights ``[N, K/2]``
  bytes with the low nibble at even k, MXFP4 scales ``[N, K/32]`` UE8M0 bytes, FP8 scales
  ``[ceil(N/128), ceil(K/128)]``).  The CPU oracle reads this one;
* the *expert page* the GPU reads differs for MXFP4 only: each scale array is stored atom by
  atom, the order the sm_100 block-scaled tensor-core instructions take scales into tensor
  memory (an atom = 128 rows x 4 scale blocks = 512 bytes; byte ``(n % 32) * 16 +
  ((n % 128) // 32) * 4 + kb % 4`` of atom ``(n // 128, kb // 4)``; atoms of a 128-row tile follow
  each other along K).  A unit of the kernel's stream is then 16 KB of codes plus 1 KB of
  scales, both consecutive bytes.  ``to_expert_page`` converts once, at load time.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ._lib import PAGE_FP8, PAGE_MXFP4


@dataclass(frozen=True)
class ExpertPageLayout:
    hidden: int
    inter: int
    kind: int = PAGE_MXFP4

    @property
    def weight_bytes(self) -> int:
        e = self.hidden * self.inter
        return e // 2 if self.kind == PAGE_MXFP4 else e

    @property
    def up_scale_bytes(self) -> int:  # s1, s3: scales of the [inter, hidden] matrices
        if self.kind == PAGE_MXFP4:
            return self.inter * self.hidden // 32
        return ((self.inter + 127) // 128) * ((self.hidden + 127) // 128)

    @property
    def down_scale_bytes(self) -> int:  # s2: scales of the [hidden, inter] matrix
        if self.kind == PAGE_MXFP4:
            return self.hidden * self.inter // 32
        return ((self.hidden + 127) // 128) * ((self.inter + 127) // 128)

    @property
    def offsets(self) -> dict:
        wb = self.weight_bytes
        o = {"w1": 0, "w3": wb, "w2": 2 * wb, "s1": 3 * wb}
        o["s3"] = o["s1"] + self.up_scale_bytes
        o["s2"] = o["s3"] + self.up_scale_bytes
        return o

    @property
    def page_bytes(self) -> int:
        return 3 * self.weight_bytes + 2 * self.up_scale_bytes + self.down_scale_bytes

    def pack(self, w1, w3, w2, s1, s3, s2) -> np.ndarray:
        page = np.empty(self.page_bytes, np.uint8)
        o = self.offsets
        for name, t in (("w1", w1), ("w3", w3), ("w2", w2), ("s1", s1), ("s3", s3), ("s2", s2)):
            t = np.ascontiguousarray(t, dtype=np.uint8).ravel()
            page[o[name]:o[name] + t.size] = t
        return page

    # ---- MXFP4 scale order of the page the GPU reads --------------------------------------
    @staticmethod
    def scales_to_page_order(s: np.ndarray, n: int, k: int) -> np.ndarray:
        """[n, k/32] row-major codes -> page order (see the module docstring)."""
        if n % 128 or k % 128:
            raise ValueError("MXFP4 page scales: rows and K must be multiples of 128")
        a = np.ascontiguousarray(s, np.uint8).reshape(n // 128, 4, 32, k // 128, 4)  # tile, r/32, r%32, atom, kb%4
        return np.ascontiguousarray(a.transpose(0, 3, 2, 1, 4)).ravel()

    @staticmethod
    def scales_from_page_order(s: np.ndarray, n: int, k: int) -> np.ndarray:
        a = np.ascontiguousarray(s, np.uint8).reshape(n // 128, k // 128, 32, 4, 4)  # tile, atom, r%32, r/32, kb%4
        return np.ascontiguousarray(a.transpose(0, 3, 2, 1, 4)).reshape(n, k // 32)

    def to_expert_page(self, tensor_page: np.ndarray) -> np.ndarray:
        """Tensor page -> the page the GPU kernels read (a copy; FP8 pages are unchanged)."""
        page = np.array(tensor_page, dtype=np.uint8, copy=True)
        if self.kind != PAGE_MXFP4:
            return page
        o = self.offsets
        for name, n, k in (("s1", self.inter, self.hidden), ("s3", self.inter, self.hidden),
                           ("s2", self.hidden, self.inter)):
            size = n * k // 32
            page[o[name]:o[name] + size] = self.scales_to_page_order(tensor_page[o[name]:o[name] + size], n, k)
        return page

    def split(self, page: np.ndarray) -> dict:
        o = self.offsets
        sizes = {"w1": self.weight_bytes, "w3": self.weight_bytes, "w2": self.weight_bytes,
                 "s1": self.up_scale_bytes, "s3": self.up_scale_bytes, "s2": self.down_scale_bytes}
        return {k: page[o[k]:o[k] + sizes[k]] for k in o}
