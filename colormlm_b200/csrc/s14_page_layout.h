// Byte order inside an MXFP4 expert page, shared by the host converter and the kernels.
//
// The reference uploads an expert's six tensors as six buffers and fixes no layout inside a pool
// slot (examples/s14_vulkan_numeric.rs:331-366), so the layout is this library's.  It is chosen so
// that everything the tcgen05 layer kernel asks for in one step is ONE contiguous run of page bytes,
// already in the order the tensor cores read shared memory: a *unit* is 128 matrix rows x 256
// K-elements of E2M1 codes, 16 KB, stored as 128 rows of 128 bytes with the 16-byte chunks of row m
// at position (chunk ^ (m % 8)) -- the 128-byte swizzle of a K-major operand tile.
//
//   up    [inter/64 slices][hidden/256 units]: rows 0-63 of a unit are w1 rows 64 s .. 64 s + 63,
//         rows 64-127 the same rows of w3 (gate and up projection of one slice in one MMA tile);
//   down  [hidden/128 row tiles][inter/256 units]: rows of w2;
//   s13   [slice][hidden/128 atoms]: the UE8M0 codes of a slice's 128 MMA rows for four scale
//         blocks, 512 bytes in the order tensor memory takes them: byte (m % 32) * 16 + (m / 32) * 4
//         + block % 4;
//   s2    [row tile][inter/128 atoms]: the same for 128 rows of w2.
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

constexpr uint32_t kUnitBytes = 16384;  // one unit of codes
constexpr uint32_t kAtomBytes = 512;    // scale codes of 128 rows x 4 blocks

S14_HD size_t mxfp4_weight_bytes(uint32_t hidden, uint32_t inter) { return (size_t)hidden * inter / 2; }
S14_HD size_t mxfp4_up_offset() { return 0; }
S14_HD size_t mxfp4_down_offset(uint32_t hidden, uint32_t inter) { return 2 * mxfp4_weight_bytes(hidden, inter); }
S14_HD size_t mxfp4_s13_offset(uint32_t hidden, uint32_t inter) { return 3 * mxfp4_weight_bytes(hidden, inter); }
S14_HD size_t mxfp4_s2_offset(uint32_t hidden, uint32_t inter) {
    return 3 * mxfp4_weight_bytes(hidden, inter) + (size_t)hidden * inter / 16;
}
S14_HD size_t mxfp4_page_bytes(uint32_t hidden, uint32_t inter) {
    return 3 * mxfp4_weight_bytes(hidden, inter) + 3 * ((size_t)hidden * inter / 32);
}

// position inside a unit of the 16 code bytes of row m, scale block kb (kb % 8 inside the unit)
S14_HD uint32_t unit_chunk_offset(uint32_t m, uint32_t kb) { return m * 128u + (((kb & 7u) ^ (m & 7u)) << 4); }

// the sixteen code bytes of scale block kb of w1 (mat 0) or w3 (mat 1) row i, from the page start
S14_HD size_t mxfp4_up_chunk_offset(uint32_t mat, uint32_t i, uint32_t kb, uint32_t hidden) {
    const uint32_t m = (i & 63u) + mat * 64u;
    return ((size_t)(i >> 6) * (hidden >> 8) + (kb >> 3)) * kUnitBytes + unit_chunk_offset(m, kb);
}
// ... of w2 row n
S14_HD size_t mxfp4_down_chunk_offset(uint32_t n, uint32_t kb, uint32_t hidden, uint32_t inter) {
    return mxfp4_down_offset(hidden, inter) + ((size_t)(n >> 7) * (inter >> 8) + (kb >> 3)) * kUnitBytes +
           unit_chunk_offset(n & 127u, kb);
}
S14_HD uint32_t atom_code_offset(uint32_t m, uint32_t kb) { return (m & 31u) * 16u + (m >> 5) * 4u + (kb & 3u); }
// the scale code of block kb of w1 / w3 row i
S14_HD size_t mxfp4_up_scale_offset(uint32_t mat, uint32_t i, uint32_t kb, uint32_t hidden, uint32_t inter) {
    const uint32_t m = (i & 63u) + mat * 64u;
    return mxfp4_s13_offset(hidden, inter) + ((size_t)(i >> 6) * (hidden >> 7) + (kb >> 2)) * kAtomBytes +
           atom_code_offset(m, kb);
}
// ... of w2 row n
S14_HD size_t mxfp4_down_scale_offset(uint32_t n, uint32_t kb, uint32_t hidden, uint32_t inter) {
    return mxfp4_s2_offset(hidden, inter) + ((size_t)(n >> 7) * (inter >> 7) + (kb >> 2)) * kAtomBytes +
           atom_code_offset(n & 127u, kb);
}

}  // namespace s14

#endif
