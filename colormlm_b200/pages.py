"""In-slot byte layout of an expert page.

The reference uploads an expert's six tensors as six separate buffers and never fixes
a layout inside a pool slot (examples/s14_vulkan_numeric.rs:331-366), so the layout is
this library's choice.  Two byte orders of the same page exist:

* the *tensor page* is the six tensors one after the other, each in the reference's tensor
  ABI: ``w1 | w3 | w2 | s1 | s3 | s2`` with weights ``[N, K/2]`` bytes (low nibble = even k),
  MXFP4 scales ``[N, K/32]`` UE8M0 bytes, FP8 scales ``[ceil(N/128), ceil(K/128)]``.  The CPU
  oracle reads this one;
* the *expert page* is what the GPU reads.  FP8 pages are tensor pages.  An MXFP4 expert page,
  ``up | down | s13 | s2`` (same size: 13 369 344 B at hidden 4096 / inter 2048), is stored so that
  everything the tcgen05 layer kernel fetches in one step is one contiguous run of bytes, already in
  the order the tensor cores read shared memory.  A *unit* is 128 matrix rows x 256 K-elements of
  E2M1 codes: 16 KB, 128 rows of 128 bytes, the 16-byte chunks of row ``m`` at position
  ``chunk ^ (m % 8)`` (the 128-byte swizzle of a K-major operand tile).

  - ``up``: ``[inter/64 slices][hidden/256 units]``; rows 0-63 of a unit are w1 rows of the slice,
    rows 64-127 the same rows of w3;
  - ``down``: ``[hidden/128 row tiles][inter/256 units]`` of w2;
  - ``s13``: by (slice s, K-atom a) 512-byte atoms holding the codes of the slice's 64 rows of
    w1 (MMA rows 0-63) and 64 rows of w3 (MMA rows 64-127) for four scale blocks, in the order
    the sm_100 block-scaled MMA takes scales into tensor memory: byte
    ``(m % 32) * 16 + (m // 32) * 4 + block % 4``;
  - ``s2``: by (row tile rt, K-atom a) atoms with the codes of 128 rows of w2, same byte order.

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
        o = self.offsets
        wb = self.weight_bytes
        m = np.arange(128)[:, None]
        swz = (np.arange(8)[None, :] ^ (m & 7))[None, None, :, :, None]  # position p of row m holds chunk p ^ (m % 8)
        # w1, w3 [i, h/2] -> (slice, row in slice, unit, chunk, 16) -> rows of both matrices -> (slice, unit, m, chunk, 16)
        w1 = t["w1"].reshape(i // 64, 64, h // 256, 8, 16)
        w3 = t["w3"].reshape(i // 64, 64, h // 256, 8, 16)
        up = np.concatenate([w1, w3], axis=1).transpose(0, 2, 1, 3, 4)
        page[0:2 * wb] = np.take_along_axis(up, np.broadcast_to(swz, up.shape), axis=3).ravel()
        # w2 [h, i/2] -> (row tile, row, unit, chunk, 16) -> (row tile, unit, row, chunk, 16)
        dn = t["w2"].reshape(h // 128, 128, i // 256, 8, 16).transpose(0, 2, 1, 3, 4)
        page[2 * wb:3 * wb] = np.take_along_axis(dn, np.broadcast_to(swz, dn.shape), axis=3).ravel()
        # s1, s3 [i, h/32] -> (slice, atom, m % 32, m // 32, block % 4), m = row in slice (+ 64 for w3)
        s13 = np.concatenate([t["s1"].reshape(i // 64, 64, h // 128, 4), t["s3"].reshape(i // 64, 64, h // 128, 4)],
                             axis=1)  # (slice, m, atom, c)
        s13 = s13.reshape(i // 64, 4, 32, h // 128, 4).transpose(0, 3, 2, 1, 4)
        page[o["s1"]:o["s1"] + 2 * self.up_scale_bytes] = np.ascontiguousarray(s13).ravel()
        # s2 [h, i/32] -> (row tile, atom, r % 32, r // 32, block % 4)
        s2 = t["s2"].reshape(h // 128, 4, 32, i // 128, 4).transpose(0, 3, 2, 1, 4)
        page[o["s2"]:o["s2"] + self.down_scale_bytes] = np.ascontiguousarray(s2).ravel()
        return page

    def split(self, page: np.ndarray) -> dict:
        o = self.offsets
        sizes = {"w1": self.weight_bytes, "w3": self.weight_bytes, "w2": self.weight_bytes,
                 "s1": self.up_scale_bytes, "s3": self.up_scale_bytes, "s2": self.down_scale_bytes}
        return {k: page[o[k]:o[k] + sizes[k]] for k in o}
