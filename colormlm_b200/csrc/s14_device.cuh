// Device helpers shared by the kernel files of the S14 MoE path.
#ifndef S14_DEVICE_CUH
#define S14_DEVICE_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "s14_internal.h"
#include "s14_page_layout.h"

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
// reproduces a correctly rounded expf.  The F32 quotient g / (1 + e) is taken in double and rounded
// to F32: with 53 >= 2 * 24 + 2 bits the second rounding changes nothing, so this is the correctly
// rounded F32 division; unlike the F32 division, the double one never leaves its inline path for
// operands of F32 range (the F32 one calls a subroutine whenever 1 + e is huge or infinite, which a
// strongly negative gate makes it, and that subroutine's first call in a layer cost the tensor-core
// layer kernel up to a microsecond of instruction fetch while the weights stream).
__device__ __forceinline__ float swiglu_limit_f32(float gate, float up) {
    const float g = fminf(gate, 10.0f);
    const float u = fminf(fmaxf(up, -10.0f), 10.0f);
    const float e = (float)exp(-(double)g);
    const float q = (float)((double)g / (double)__fadd_rn(1.0f, e));
    return __fmul_rn(q, u);
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

// An expert page as the kernels see it.  FP8 pages are the six tensors one after the other
// (w1 | w3 | w2 | s1 | s3 | s2, weights [N, K] bytes, one UE8M0 code per 128 x 128 block).  MXFP4
// pages are read through the offset functions of s14_page_layout.h from `base`.
struct PageView {
    const uint8_t *base;
    const uint8_t *w1, *w3, *w2, *s1, *s3, *s2;  // FP8 pages only
};

__device__ __forceinline__ PageView page_view(const uint8_t *page, uint32_t kind, uint32_t hidden,
                                              uint32_t inter) {
    PageView v;
    v.base = page;
    const size_t elems = (size_t)hidden * inter;
    const size_t sb = (size_t)((inter + 127u) >> 7) * ((hidden + 127u) >> 7);
    v.w1 = page;
    v.w3 = page + elems;
    v.w2 = page + 2 * elems;
    v.s1 = page + 3 * elems;
    v.s3 = v.s1 + sb;
    v.s2 = v.s3 + sb;
    (void)kind;
    return v;
}

}  // namespace s14

#endif
