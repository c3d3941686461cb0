// Byte order inside an MXFP4 expert page, shared by the host converter and the kernels.
//
// The reference uploads an expert's six tensors as six buffers and fixes no layout inside a pool
// slot (examples/s14_vulkan_numeric.rs:331-366), so the layout is this library's.  It is chosen so
// that everything the tcgen05 layer kernel asks for in one step is ONE contiguous run of page bytes,
// already in the order the tensor cores read shared memory.  A *unit* is 128 matrix rows x 256
// K-elements: 16 KB of E2M1 codes stored as 128 rows of 128 bytes with the 16-byte chunks of row m
// at position (chunk ^ (m % 8)) -- the 128-byte swizzle of a K-major operand tile -- followed by
// the rows' UE8M0 scale codes for the unit's eight scale blocks: two atoms of 512 bytes (four
// blocks each) in the order tensor memory takes them, byte (m % 32) * 16 + (m / 32) * 4 + block % 4.
// 17 408 bytes in all, one bulk copy.
//
//   up    [inter/64 slices][hidden/256 units]: rows 0-63 of a unit are w1 rows 64 s .. 64 s + 63,
//         rows 64-127 the same rows of w3 (gate and up projection of one slice in one MMA tile);
//   down  [hidden/128 row tiles][inter/256 units]: rows of w2.
//
// The page has the size of the six tensors (13 369 344 B at hidden 4096, intermediate 2048).  hidden
// and intermediate are multiples of 256.  A scale block's sixteen code bytes (32 codes, low nibble =
// even k) stay together, so every kernel can fetch them with one 16-byte load.
#ifndef S14_PAGE_LAYOUT_H
#define S14_PAGE_LAYOUT_H

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define S14_HD __host__ __device__ __forceinline__
#else
#define S14_HD inline
#endif

namespace s14 {

constexpr uint32_t kUnitBytes = 16384;  // the codes of a unit
constexpr uint32_t kAtomBytes = 512;    // scale codes of 128 rows x 4 blocks
constexpr uint32_t kUnitStride = kUnitBytes + 2 * kAtomBytes;  // a unit with its scales

S14_HD size_t mxfp4_up_units(uint32_t hidden, uint32_t inter) { return (size_t)(inter >> 6) * (hidden >> 8); }
S14_HD size_t mxfp4_down_units(uint32_t hidden, uint32_t inter) { return (size_t)(hidden >> 7) * (inter >> 8); }
S14_HD size_t mxfp4_down_offset(uint32_t hidden, uint32_t inter) { return mxfp4_up_units(hidden, inter) * kUnitStride; }
S14_HD size_t mxfp4_page_bytes(uint32_t hidden, uint32_t inter) {
    return (mxfp4_up_units(hidden, inter) + mxfp4_down_units(hidden, inter)) * kUnitStride;
}

// position inside a unit of the 16 code bytes of row m, scale block kb (kb % 8 inside the unit)
S14_HD uint32_t unit_chunk_offset(uint32_t m, uint32_t kb) { return m * 128u + (((kb & 7u) ^ (m & 7u)) << 4); }
// ... of the scale code of row m, block kb
S14_HD uint32_t unit_scale_offset(uint32_t m, uint32_t kb) {
    return kUnitBytes + ((kb >> 2) & 1u) * kAtomBytes + (m & 31u) * 16u + (m >> 5) * 4u + (kb & 3u);
}
// the unit that holds scale block kb of w1 / w3 row i (both matrices share it), from the page start
S14_HD size_t mxfp4_up_unit_offset(uint32_t i, uint32_t kb, uint32_t hidden) {
    return ((size_t)(i >> 6) * (hidden >> 8) + (kb >> 3)) * kUnitStride;
}
// ... of w2 row n
S14_HD size_t mxfp4_down_unit_offset(uint32_t n, uint32_t kb, uint32_t hidden, uint32_t inter) {
    return mxfp4_down_offset(hidden, inter) + ((size_t)(n >> 7) * (inter >> 8) + (kb >> 3)) * kUnitStride;
}
// the sixteen code bytes of scale block kb of w1 (mat 0) or w3 (mat 1) row i, from the page start
S14_HD size_t mxfp4_up_chunk_offset(uint32_t mat, uint32_t i, uint32_t kb, uint32_t hidden) {
    return mxfp4_up_unit_offset(i, kb, hidden) + unit_chunk_offset((i & 63u) + mat * 64u, kb);
}
// ... of w2 row n
S14_HD size_t mxfp4_down_chunk_offset(uint32_t n, uint32_t kb, uint32_t hidden, uint32_t inter) {
    return mxfp4_down_unit_offset(n, kb, hidden, inter) + unit_chunk_offset(n & 127u, kb);
}
// the scale code of block kb of w1 / w3 row i
S14_HD size_t mxfp4_up_scale_offset(uint32_t mat, uint32_t i, uint32_t kb, uint32_t hidden, uint32_t inter) {
    (void)inter;
    return mxfp4_up_unit_offset(i, kb, hidden) + unit_scale_offset((i & 63u) + mat * 64u, kb);
}
// ... of w2 row n
S14_HD size_t mxfp4_down_scale_offset(uint32_t n, uint32_t kb, uint32_t hidden, uint32_t inter) {
    return mxfp4_down_unit_offset(n, kb, hidden, inter) + unit_scale_offset(n & 127u, kb);
}

}  // namespace s14

#endif
