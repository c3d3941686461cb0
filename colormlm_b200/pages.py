"""In-slot byte layout of an expert page.

The reference uploads an expert's six tensors as six separate buffers and never fixes
a layout inside a pool slot (examples/s14_vulkan_numeric.rs:331-366), so the layout is
this library's choice.  Two byte orders of the same page exist:

* the *tensor page* is the six tensors one after the other, each in the reference's tensor
  ABI: ``w1 | w3 | w2 | s1 | s3 | s2`` with weights ``[N, K/2]`` bytes (low nibble = even k),
  MXFP4 scales ``[N, K/32]`` UE8M0 bytes, FP8 scales ``[ceil(N/128), ceil(K/128)]``.  The CPU
  oracle reads this one;
* the *expert page* is what the GPU reads.  FP8 pages are tensor pages.  An MXFP4 expert page,
  ``up | down`` (same size: 13 369 344 B at hidden 4096 / inter 2048), is stored so that
  everything the tcgen05 layer kernel fetches in one step is one contiguous run of bytes, already in
  the order the tensor cores read shared memory.  A *unit* is 128 matrix rows x 256 K-elements:
  16 KB of E2M1 codes, 128 rows of 128 bytes, the 16-byte chunks of row ``m`` at position
  ``chunk ^ (m % 8)`` (the 128-byte swizzle of a K-major operand tile), followed by the rows' scale
  codes for the unit's eight scale blocks: two atoms of 512 bytes (four blocks each) in the order
  the sm_100 block-scaled MMA takes scales into tensor memory, byte
  ``(m % 32) * 16 + (m // 32) * 4 + block % 4``.  17 408 bytes per unit.

  - ``up``: ``[inter/64 slices][hidden/256 units]``; rows 0-63 of a unit are w1 rows of the slice,
    rows 64-127 the same rows of w3;
  - ``down``: ``[hidden/128 row tiles][inter/256 units]`` of w2.

``to_expert_page`` converts once, at load time (hidden and inter multiples of 256).
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

    # ---- the page the GPU reads -------------------------------------------------------------
    def to_expert_page(self, tensor_page: np.ndarray) -> np.ndarray:
        """Tensor page -> expert page (a copy; FP8 pages are unchanged)."""
        page = np.array(tensor_page, dtype=np.uint8, copy=True)
        if self.kind != PAGE_MXFP4:
            return page
        h, i = self.hidden, self.inter
        if h % 256 or i % 256:
            raise ValueError("MXFP4 expert page: hidden and inter must be multiples of 256")
        t = self.split(np.asarray(tensor_page, np.uint8))
        m = np.arange(128)[:, None]
        swz = (np.arange(8)[None, :] ^ (m & 7))[None, None, :, :, None]  # position p of row m holds chunk p ^ (m % 8)
        # w1, w3 [i, h/2] -> (slice, row in slice, unit, chunk, 16) -> rows of both matrices -> (slice, unit, m, chunk, 16)
        w1 = t["w1"].reshape(i // 64, 64, h // 256, 8, 16)
        w3 = t["w3"].reshape(i // 64, 64, h // 256, 8, 16)
        up = np.concatenate([w1, w3], axis=1).transpose(0, 2, 1, 3, 4)
        up = np.take_along_axis(up, np.broadcast_to(swz, up.shape), axis=3).reshape(i // 64, h // 256, 16384)
        # s1, s3 [i, h/32] -> (slice, atom, m % 32, m // 32, block % 4), m = row in slice (+ 64 for w3); two atoms per unit
        s13 = np.concatenate([t["s1"].reshape(i // 64, 64, h // 128, 4), t["s3"].reshape(i // 64, 64, h // 128, 4)],
                             axis=1)  # (slice, m, atom, c)
        s13 = s13.reshape(i // 64, 4, 32, h // 128, 4).transpose(0, 3, 2, 1, 4).reshape(i // 64, h // 256, 1024)
        up_units = np.concatenate([up, s13], axis=2)
        # w2 [h, i/2] -> (row tile, row, unit, chunk, 16) -> (row tile, unit, row, chunk, 16)
        dn = t["w2"].reshape(h // 128, 128, i // 256, 8, 16).transpose(0, 2, 1, 3, 4)
        dn = np.take_along_axis(dn, np.broadcast_to(swz, dn.shape), axis=3).reshape(h // 128, i // 256, 16384)
        # s2 [h, i/32] -> (row tile, atom, r % 32, r // 32, block % 4)
        s2 = t["s2"].reshape(h // 128, 4, 32, i // 128, 4).transpose(0, 3, 2, 1, 4).reshape(h // 128, i // 256, 1024)
        down_units = np.concatenate([dn, s2], axis=2)
        page[:up_units.size] = up_units.ravel()
        page[up_units.size:] = down_units.ravel()
        return page

    def split(self, page: np.ndarray) -> dict:
        o = self.offsets
        sizes = {"w1": self.weight_bytes, "w3": self.weight_bytes, "w2": self.weight_bytes,
                 "s1": self.up_scale_bytes, "s3": self.up_scale_bytes, "s2": self.down_scale_bytes}
        return {k: page[o[k]:o[k] + sizes[k]] for k in o}
