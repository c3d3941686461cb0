// tcgen05 / mbarrier / bulk-copy helpers and the digit arithmetic shared by the tensor-core kernels
// of the S14 MoE path (the one-token layer kernel and the grouped block kernels).
#ifndef S14_UMMA_CUH
#define S14_UMMA_CUH

#include "s14_device.cuh"

namespace s14 {
namespace {

constexpr uint32_t kSpin = 1u << 17;        // tries (a microsecond each at most) before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Plain bulk copy global -> this CTA's shared memory; both addresses and the size are multiples
// of 16.  Completion is counted in bytes on the mbarrier.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// The same copy for page bytes that are read once: the lines go first when the L2 needs room, so that
// they do not displace what was fetched ahead (the next layer's shared expert).
__device__ __forceinline__ void bulk_copy_stream(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar,
                                                 unsigned long long policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ unsigned long long l2_policy_evict_first() {
    unsigned long long p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// Asks the L2 for bytes of this GPU's memory that a later copy will read (size a multiple of 16).
__device__ __forceinline__ void l2_prefetch(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// One bounded hardware wait: returns when the phase completes or after about a microsecond.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.b32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the phase did not complete in kSpin tries (each suspends the thread
// for a microsecond at most, so about 0.1 s) or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
#pragma unroll 1
    for (uint32_t i = 0; i < kSpin; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// Named barriers, plain and with a vote.  Every thread of the group executes them, whatever it has
// seen, so a group never splits in front of a barrier; and every one starts by bringing the warp
// back together, because a lane that has been polling or issuing on its own may still be behind its
// warp, and a warp counts as arrived as soon as some of its lanes get there.  1: the 128 epilogue
// threads; 2: the 256 tile threads; 3: the 512 threads that share the token.
template <int ID, int N>
__device__ __forceinline__ bool named_all(bool ok) {
    uint32_t r;
    __syncwarp();
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "setp.ne.b32 p, %1, 0;\n"
        "barrier.cta.red.and.pred q, %2, %3, p;\n"
        "selp.b32 %0, 1, 0, q;\n}"
        : "=r"(r)
        : "r"((uint32_t)ok), "n"(ID), "n"(N)
        : "memory");
    return r != 0;
}
template <int ID, int N>
__device__ __forceinline__ void named_sync() {
    __syncwarp();
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(N) : "memory");
}
__device__ __forceinline__ bool epi_all(bool ok) { return named_all<1, 128>(ok); }
__device__ __forceinline__ bool load_all(bool ok) { return named_all<2, 256>(ok); }
__device__ __forceinline__ bool token_all(bool ok) { return named_all<3, 512>(ok); }
__device__ __forceinline__ void epi_sync() { named_sync<1, 128>(); }
__device__ __forceinline__ void load_sync() { named_sync<2, 256>(); }
__device__ __forceinline__ void token_sync() { named_sync<3, 512>(); }
// Shared-memory matrix descriptor of sm_100: start address, leading and stride byte offsets in
// 16-byte units, descriptor version 1, layout (0 = no swizzle, 2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo16, uint32_t sbo16, uint32_t layout) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)(lbo16 & 0x3FFFu) << 16) |
           ((uint64_t)(sbo16 & 0x3FFFu) << 32) | ((uint64_t)1 << 46) | ((uint64_t)(layout & 7u) << 61);
}
__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void tmem_copy_scales(uint32_t tmem, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// Sixteen accumulator columns of the warp's 32 lanes; the values may be used after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }


__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// E2M1 codes of the eight balanced base-8 digits of q (|q| <= 2^23), one code per byte: digit j in
// byte j of c03 (j < 4) or byte j - 4 of c47.  With the bias 4 * (8^8 - 1) / 7 added, the balanced
// digits are the plain base-8 digits minus 4, so no carry runs through them; the top digit may
// reach +4.  The 3-bit fields are spread to nibbles and looked up four at a time with prmt.
__device__ __forceinline__ void digit_code_bytes(int q, uint32_t &c03, uint32_t &c47) {
    const uint32_t qb = (uint32_t)(q + 0x924924);  // in [0, 8^8 + 8^7)
    uint32_t x = qb & 0xFFFFFFu;
    x = (x & 0x00000FFFu) | ((x & 0x00FFF000u) << 4);
    x = (x & 0x003F003Fu) | ((x & 0x0FC00FC0u) << 2);
    x = (x & 0x07070707u) | ((x & 0x38383838u) << 1);  // digit value j (0..7) in nibble j
    // codes of -4, -3, -2, -1 | 0, 1, 2, 3 by digit value
    c03 = prmt(0x0A0C0D0Eu, 0x05040200u, x);
    c47 = prmt(0x0A0C0D0Eu, 0x05040200u, x >> 16);
    if (qb >> 24) c47 = (c47 & 0x00FFFFFFu) | 0x06000000u;  // top digit +4
}
// Four code bytes (each < 16) -> four nibbles in the low 16 bits of byte lanes 0 and 2 of the result
// (use with pack_pairs).
__device__ __forceinline__ uint32_t pair_nibbles(uint32_t c) { return c | (c >> 4); }
// nibbles of eight codes: a = pair_nibbles of codes 0-3, b = of codes 4-7
__device__ __forceinline__ uint32_t pack_pairs(uint32_t a, uint32_t b) { return prmt(a, b, 0x6420u); }
// E2M1 codes of the eight digits of q, digit j in bits 4j .. 4j+3.
__device__ __forceinline__ uint32_t digit_codes(int q) {
    uint32_t c03, c47;
    digit_code_bytes(q, c03, c47);
    return pack_pairs(pair_nibbles(c03), pair_nibbles(c47));
}
// v * 2^(23-E) = hi + lo * 2^-24 with integers |hi|, |lo| <= 2^23 (|v| < 2^E).
__device__ __forceinline__ void split_hi_lo(float v, float up, int &hi, int &lo) {
    const float t = v * up;  // exact: a power of two
    hi = __float2int_rn(t);
    const float rem = __fsub_rn(t, (float)hi);  // exact
    lo = __float2int_rn(rem * 16777216.0f);
}
__device__ __forceinline__ void digit_codes16(float v, float up, uint32_t &hi_w, uint32_t &lo_w) {
    int hi, lo;
    split_hi_lo(v, up, hi, lo);
    hi_w = digit_codes(hi);
    lo_w = digit_codes(lo);
}
// Transposes four registers of four bytes: out k = byte k of r0, r1, r2, r3.
__device__ __forceinline__ void transpose4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&o)[4]) {
    const uint32_t t0 = prmt(r0, r1, 0x5140u), t1 = prmt(r0, r1, 0x7362u);
    const uint32_t t2 = prmt(r2, r3, 0x5140u), t3 = prmt(r2, r3, 0x7362u);
    o[0] = prmt(t0, t2, 0x5410u);
    o[1] = prmt(t0, t2, 0x7632u);
    o[2] = prmt(t1, t3, 0x5410u);
    o[3] = prmt(t1, t3, 0x7632u);
}
// The exponent E of a scale block from its largest magnitude: bm < 2^E, clamped to [-80, 127] (row
// 8 of a block carries the scale 2^(E-47), whose UE8M0 code must not fall below zero).
__device__ __forceinline__ int block_exponent(float bm) {
    int E = -80;
    if (bm > 0.0f) E = min(max((int)((__float_as_uint(bm) >> 23) & 0xFFu) - 126, -80), 127);
    return E;
}

// Writes the sixteen digit rows of elements 8g .. 8g+7 of a vector into a digit tile (2 KB per 256
// elements: sixteen rows of 128 bytes, the 16-byte chunk of scale block kb at position
// (kb % 8) ^ (row % 8)) and, for the first thread of a scale block, the block's exponent.  Thread g
// owns one 32-bit word of every digit row; the four lanes of a scale block agree on its exponent,
// so whole warps call this together.
__device__ __forceinline__ void digits_of8(const float (&xs)[8], uint32_t g, uint8_t *sB, uint8_t *sE) {
    float bm = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) bm = fmaxf(bm, fabsf(xs[i]));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
    const int E = block_exponent(bm);
    const float up = __uint_as_float((uint32_t)(150 - E) << 23);  // 2^(23-E)
    // Four elements at a time: their code bytes [element][hi digits 0-3, hi 4-7, lo 0-3, lo 4-7] are
    // transposed to [digit row][element] and squeezed to nibbles; the two halves of a row's word are
    // joined at the end.
    uint32_t half[2][16];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t c[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int hi, lo;
            split_hi_lo(xs[h * 4 + i], up, hi, lo);
            digit_code_bytes(hi, c[i][0], c[i][1]);
            digit_code_bytes(lo, c[i][2], c[i][3]);
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {  // four digit rows at a time
            uint32_t a[4];
            transpose4(c[0][q4], c[1][q4], c[2][q4], c[3][q4], a);
#pragma unroll
            for (int k = 0; k < 4; ++k) half[h][q4 * 4 + k] = pair_nibbles(a[k]);
        }
    }
    // word of digit row j: the codes of elements 0..7 in nibbles 0..7
    uint32_t words[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) words[j] = pack_pairs(half[0][j], half[1][j]);
    const uint32_t kb = g >> 2;
    uint8_t *chunk = sB + (kb >> 3) * 2048u + (g & 3u) * 4u;
#pragma unroll
    for (uint32_t j = 0; j < 16; ++j)
        *reinterpret_cast<uint32_t *>(chunk + j * 128u + (((kb & 7u) ^ (j & 7u)) << 4)) = words[j];
    if ((g & 3u) == 0u) sE[kb] = (uint8_t)(E + 100);  // the block's exponent, biased
}

// The scale codes of the sixteen digit rows of a vector of K elements, written to tensor memory by
// the warp that owns lane quadrant `quad` (every quadrant holds all of them); the warp takes the
// groups of four atoms g0, g0 + gstep, ...  Column 4a of lane l holds the codes of N-row l for scale
// blocks 4a..4a+3: digit row l < 8 of a block with exponent E has the code 127 + E - 23 + 3l, row
// 8 + l the code 127 + E - 47 + 3l; columns 4a+1..4a+3 belong to N-rows 32 and up, which a 16-column
// MMA does not use.  sE holds E + 100 per block.
__device__ __forceinline__ void store_digit_scales(uint32_t tmem_sfb, const uint8_t *sE, uint32_t K, uint32_t quad,
                                                   uint32_t g0, uint32_t gstep, uint32_t lane) {
    const uint32_t groups = K >> 9;  // groups of four atoms (512 K-elements, 16 blocks)
    const int shift = lane < 8u ? 4 + 3 * (int)lane : 3 * (int)(lane & 7u) - 20;
    const uint32_t bias = 0x01010101u * (uint32_t)shift;  // no byte borrows: E + 100 >= 20
    const uint32_t base = tmem_sfb + ((quad * 32u) << 16);
    const uint32_t one = 0x7F7F7F7Fu;
#pragma unroll 1
    for (uint32_t g = g0; g < groups; g += gstep) {
        const uint4 e = *reinterpret_cast<const uint4 *>(sE + g * 16u);
        const uint32_t w0 = lane < 16u ? e.x + bias : one, w1 = lane < 16u ? e.y + bias : one;
        const uint32_t w2 = lane < 16u ? e.z + bias : one, w3 = lane < 16u ? e.w + bias : one;
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%5,%5,%5,%2,%5,%5,%5,%3,%5,%5,%5,%4,%5,%5,%5};"
            ::"r"(base + g * 16u), "r"(w0), "r"(w1), "r"(w2), "r"(w3), "r"(one)
            : "memory");
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_gpu(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ ulonglong2 ld_relaxed_gpu2(const void *p) {
    ulonglong2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu2(void *p, unsigned long long a, unsigned long long b) {
    asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire(const unsigned int *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Instruction descriptor of kind::mxf4.block_scale: A and B E2M1 (format 1), both K-major, UE8M0
// scales, M = 128, N = n (a multiple of 16).
__device__ __forceinline__ constexpr uint32_t umma_idesc_mxf4(uint32_t n) {
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);
}

}  // namespace
}  // namespace s14

#endif
