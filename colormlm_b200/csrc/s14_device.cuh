// Device helpers shared by the kernel files of the S14 MoE path.
#ifndef S14_DEVICE_CUH
#define S14_DEVICE_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "s14_internal.h"

namespace s14 {

// ---------------------------------------------------------------- decode ----

// Eight E2M1 codes of one 32-bit word (low nibble first) -> four f16x2 words.
__device__ __forceinline__ void e2m1x8_to_h2x4(uint32_t w, uint32_t &h0, uint32_t &h1,
                                               uint32_t &h2, uint32_t &h3) {
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3)
        : "r"(w));
}

// Four E4M3 codes of one 32-bit word -> two f16x2 words.
__device__ __forceinline__ void e4m3x4_to_h2x2(uint32_t w, uint32_t &h0, uint32_t &h1) {
    asm("{\n"
        ".reg .b16 lo, hi;\n"
        "mov.b32 {lo, hi}, %2;\n"
        "cvt.rn.f16x2.e4m3x2 %0, lo;\n"
        "cvt.rn.f16x2.e4m3x2 %1, hi;\n"
        "}\n"
        : "=r"(h0), "=r"(h1)
        : "r"(w));
}

__device__ __forceinline__ float2 h2_to_f2(uint32_t h) {
    __half2 v;
    *reinterpret_cast<uint32_t *>(&v) = h;
    return __half22float2(v);
}

// 2^(code-127) as a double: exact for every code 0..254.
__device__ __forceinline__ double ue8m0_to_f64(uint32_t code) {
    return __hiloint2double((int)((code + 896u) << 20), 0);
}

// 2^(code-127) as a float; code 0 is the subnormal 2^-127.
__device__ __forceinline__ float ue8m0_to_f32(uint32_t code) {
    return __uint_as_float(code == 0u ? 0x00400000u : (code << 23));
}

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The reference's SwiGLU (examples/s14_vulkan_numeric.rs:1543-1556) in F32 with
// separate operations.  expf is evaluated in double and rounded once, which
// reproduces a correctly rounded expf.
__device__ __forceinline__ float swiglu_limit_f32(float gate, float up) {
    const float g = fminf(gate, 10.0f);
    const float u = fminf(fmaxf(up, -10.0f), 10.0f);
    const float e = (float)exp(-(double)g);
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), u);
}

// An expert's score from its logit (the double-accumulated dot product, rounded to F32 first):
// sigmoid or sqrt(softplus), evaluated in double and rounded once.
__device__ __forceinline__ float router_score_f32(double logit_sum, uint32_t score_fn) {
    const double l = (double)(float)logit_sum;
    const double sc = (score_fn == S14_SCORE_SIGMOID) ? 1.0 / (1.0 + exp(-l)) : sqrt(l > 20.0 ? l : log1p(exp(l)));
    return (float)sc;
}

__device__ __forceinline__ const JobTable &table_of(const JobTable *dev, const JobTable &param) {
    return dev ? *dev : param;
}

struct PageView {
    const uint8_t *w1, *w3, *w2, *s1, *s3, *s2;
};

// Byte order inside an MXFP4 expert page (w1 | w3 | w2 | s13 | s2).  The unit of work of the
// tcgen05 kernel is a slice of 64 intermediate elements of one expert: the 64 rows of w1 and of
// w3 that produce them (one 128-row MMA tile) and the 64 columns of w2 that consume them.
//   w1, w3  [inter, hidden/2] bytes, row-major, as the checkpoint has them.
//   w2      by slice s and row tile rt: 128 rows x 32 B (the 64 codes of the slice), 4 KB per
//           (s, rt), row tiles of a slice next to each other -- a slice's columns are one
//           contiguous run of hidden * 32 bytes.
//   s13     the scale codes of w1 and w3 by slice s and K-atom a (four scale blocks): 512 B in
//           the order tensor memory takes them, MMA row m = the slice's w1 row m (m < 64) or w3
//           row m - 64: byte (m % 32) * 16 + (m / 32) * 4 + block % 4.
//   s2      the scale codes of w2 by slice pair p and row tile rt: 512 B, row r of the tile at
//           (r % 32) * 16 + (r / 32) * 4, blocks 4p..4p+3 (slice 2p: 0 and 1, slice 2p+1: 2 and 3).
// hidden and inter are multiples of 128.  The sixteen code bytes (one scale block) of w2 row n:
__device__ __forceinline__ size_t w2_block_offset(uint32_t n, uint32_t kb, uint32_t hidden) {
    return (((size_t)(kb >> 1) * (hidden >> 7) + (n >> 7)) * 128u + (n & 127u)) * 32u + (kb & 1u) * 16u;
}
// the scale code of row i, block kb of w1 (mat 0) or w3 (mat 1), inside s13
__device__ __forceinline__ size_t up_scale_offset(uint32_t mat, uint32_t i, uint32_t kb, uint32_t hidden) {
    const uint32_t m = (i & 63u) + mat * 64u;
    return ((size_t)(i >> 6) * (hidden >> 7) + (kb >> 2)) * 512u + (m & 31u) * 16u + (m >> 5) * 4u + (kb & 3u);
}
// the scale code of row n, block kb of w2, inside s2
__device__ __forceinline__ size_t down_scale_offset(uint32_t n, uint32_t kb, uint32_t hidden) {
    const uint32_t r = n & 127u;
    return ((size_t)(kb >> 2) * (hidden >> 7) + (n >> 7)) * 512u + (r & 31u) * 16u + (r >> 5) * 4u + (kb & 3u);
}

__device__ __forceinline__ PageView page_view(const uint8_t *page, uint32_t kind, uint32_t hidden,
                                              uint32_t inter) {
    PageView v;
    const size_t elems = (size_t)hidden * inter;
    if (kind == S14_PAGE_MXFP4) {
        const size_t wb = elems >> 1, sb = elems >> 5;
        v.w1 = page;
        v.w3 = page + wb;
        v.w2 = page + 2 * wb;
        v.s1 = page + 3 * wb;
        v.s3 = v.s1 + sb;
        v.s2 = v.s3 + sb;
    } else {
        const size_t sb = (size_t)((inter + 127u) >> 7) * ((hidden + 127u) >> 7);
        v.w1 = page;
        v.w3 = page + elems;
        v.w2 = page + 2 * elems;
        v.s1 = page + 3 * elems;
        v.s3 = v.s1 + sb;
        v.s2 = v.s3 + sb;
    }
    return v;
}

}  // namespace s14

#endif
