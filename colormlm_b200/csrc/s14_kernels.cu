// sm_100a kernels of the S14 MoE expert hot path.
//
// Two summation orders are implemented for every matvec (see S14_ACCUM_* in
// include/polaris_s14_cuda.h):
//   pairwise  - a warp owns an output row, its lanes split K in 16-byte pieces
//               (128-bit coalesced loads), decode E2M1 / E4M3 with the hardware
//               cvt to f16x2, multiply-accumulate in F32 inside one scale block,
//               then carry block sums, lane sums and the final value in F64;
//   reference - a thread owns an output row and walks k in ascending order with
//               the reference's separate multiply / multiply / add per element
//               (examples/s14_vulkan_numeric.rs:1669-1714), bit-identical to it.
// The elementwise steps (limit-10 SwiGLU, route mix, ordered accumulate) use
// separate F32 multiplies and adds in both modes, as the reference does.
#include "s14_device.cuh"

namespace s14 {

// F32 dot of 32 E2M1 codes (one 16-byte piece = one scale block) with 32
// activations held in registers; two independent even/odd chains on the packed
// F32x2 pipe.
__device__ __forceinline__ float dot32_e2m1(const uint4 &q, const float *__restrict__ xr) {
    float2 acc = make_float2(0.f, 0.f);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t h0, h1, h2, h3;
        e2m1x8_to_h2x4(w[i], h0, h1, h2, h3);
        acc = __ffma2_rn(h2_to_f2(h0), make_float2(xr[i * 8 + 0], xr[i * 8 + 1]), acc);
        acc = __ffma2_rn(h2_to_f2(h1), make_float2(xr[i * 8 + 2], xr[i * 8 + 3]), acc);
        acc = __ffma2_rn(h2_to_f2(h2), make_float2(xr[i * 8 + 4], xr[i * 8 + 5]), acc);
        acc = __ffma2_rn(h2_to_f2(h3), make_float2(xr[i * 8 + 6], xr[i * 8 + 7]), acc);
    }
    return acc.x + acc.y;
}

// F32 dot of 16 E4M3 codes (one 16-byte piece) with 16 activations.
__device__ __forceinline__ float dot16_e4m3(const uint4 &q, const float *__restrict__ xr) {
    float2 acc = make_float2(0.f, 0.f);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t h0, h1;
        e4m3x4_to_h2x2(w[i], h0, h1);
        acc = __ffma2_rn(h2_to_f2(h0), make_float2(xr[i * 4 + 0], xr[i * 4 + 1]), acc);
        acc = __ffma2_rn(h2_to_f2(h1), make_float2(xr[i * 4 + 2], xr[i * 4 + 3]), acc);
    }
    return acc.x + acc.y;
}

// ------------------------------------------------- primitive operators ------

// y[n] = sum_k x[k] * e2m1(w[n,k]) * 2^(s[n,k/32]-127); warp per row.
__global__ void __launch_bounds__(256)
k_mxfp4_matvec_pairwise(const float *__restrict__ x, const uint8_t *__restrict__ w,
                        const uint8_t *__restrict__ s, float *__restrict__ y, uint32_t n_rows,
                        uint32_t k) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t groups = k >> 5;
    for (uint32_t n = warp; n < n_rows; n += n_warps) {
        const uint4 *wrow = reinterpret_cast<const uint4 *>(w + (size_t)n * (k >> 1));
        const uint8_t *srow = s + (size_t)n * groups;
        double acc = 0.0;
        for (uint32_t g = lane; g < groups; g += 32u) {
            const uint4 q = ldg_stream(wrow + g);
            float xr[32];
            const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)g * 32u);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 v = __ldg(xp + i);
                xr[i * 4 + 0] = v.x;
                xr[i * 4 + 1] = v.y;
                xr[i * 4 + 2] = v.z;
                xr[i * 4 + 3] = v.w;
            }
            acc += (double)dot32_e2m1(q, xr) * ue8m0_to_f64(__ldg(srow + g));
        }
        acc = warp_sum(acc);
        if (lane == 0) y[n] = (float)acc;
    }
}

// Reference order: thread per row, k ascending, (x*e)*s then add.
__global__ void __launch_bounds__(128)
k_mxfp4_matvec_reference(const float *__restrict__ x, const uint8_t *__restrict__ w,
                         const uint8_t *__restrict__ s, float *__restrict__ y, uint32_t n_rows,
                         uint32_t k) {
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= n_rows) return;
    const uint32_t groups = k >> 5;
    const uint4 *wrow = reinterpret_cast<const uint4 *>(w + (size_t)n * (k >> 1));
    const uint8_t *srow = s + (size_t)n * groups;
    float sum = 0.0f;
    for (uint32_t g = 0; g < groups; ++g) {
        const uint4 q = __ldg(wrow + g);
        const float sc = ue8m0_to_f32(__ldg(srow + g));
        const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
        const float *xg = x + (size_t)g * 32u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t h[4];
            e2m1x8_to_h2x4(wd[i], h[0], h[1], h[2], h[3]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 e = h2_to_f2(h[j]);
                sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(__ldg(xg + i * 8 + j * 2), e.x), sc));
                sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(__ldg(xg + i * 8 + j * 2 + 1), e.y), sc));
            }
        }
    }
    y[n] = sum;
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t code) {
    const __half_raw hr = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code, __NV_E4M3);
    return __half2float(__half(hr));
}

template <bool F32_SCALE>
__device__ __forceinline__ double fp8_block_scale_f64(const void *scale, size_t idx) {
    if (F32_SCALE) return (double)__ldg(reinterpret_cast<const float *>(scale) + idx);
    return ue8m0_to_f64(__ldg(reinterpret_cast<const uint8_t *>(scale) + idx));
}

template <bool F32_SCALE>
__device__ __forceinline__ float fp8_block_scale_f32(const void *scale, size_t idx) {
    if (F32_SCALE) return __ldg(reinterpret_cast<const float *>(scale) + idx);
    return ue8m0_to_f32(__ldg(reinterpret_cast<const uint8_t *>(scale) + idx));
}

// y[t,n] = sum_k x[t,k] * e4m3(w[n,k]) * scale[n/128][k/128]; warp per row, any k,
// NT tokens per weight pass.  Lanes take 16-byte pieces when the row is 16-byte
// aligned and k is a multiple of 16, single bytes otherwise.
template <int NT, bool F32_SCALE>
__global__ void __launch_bounds__(256)
k_fp8_matvec_pairwise(const float *__restrict__ x, const uint8_t *__restrict__ w,
                      const void *__restrict__ scale, float *__restrict__ y, uint32_t n_rows,
                      uint32_t k) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t k_groups = (k + 127u) >> 7;
    const bool vec_ok = ((k & 15u) == 0u) && ((reinterpret_cast<uintptr_t>(w) & 15u) == 0u) &&
                        ((reinterpret_cast<uintptr_t>(x) & 15u) == 0u);
    for (uint32_t n = warp; n < n_rows; n += n_warps) {
        const uint8_t *wrow = w + (size_t)n * k;
        const size_t srow = (size_t)(n >> 7) * k_groups;
        double acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.0;
        if (vec_ok) {
            const uint32_t pieces = k >> 4;
            for (uint32_t p = lane; p < pieces; p += 32u) {
                const uint4 q = ldg_stream(reinterpret_cast<const uint4 *>(wrow) + p);
                const double sc = fp8_block_scale_f64<F32_SCALE>(scale, srow + (p >> 3));
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    float xr[16];
                    const float4 *xp =
                        reinterpret_cast<const float4 *>(x + (size_t)t * k + (size_t)p * 16u);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 v = __ldg(xp + i);
                        xr[i * 4 + 0] = v.x;
                        xr[i * 4 + 1] = v.y;
                        xr[i * 4 + 2] = v.z;
                        xr[i * 4 + 3] = v.w;
                    }
                    acc[t] += (double)dot16_e4m3(q, xr) * sc;
                }
            }
        } else {
            for (uint32_t kk = lane; kk < k; kk += 32u) {
                const double wv = (double)e4m3_to_f32(__ldg(wrow + kk)) *
                                  fp8_block_scale_f64<F32_SCALE>(scale, srow + (kk >> 7));
#pragma unroll
                for (int t = 0; t < NT; ++t) acc[t] += (double)__ldg(x + (size_t)t * k + kk) * wv;
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const double v = warp_sum(acc[t]);
            if (lane == 0) y[(size_t)t * n_rows + n] = (float)v;
        }
    }
}

// The same product for a block of tokens and a matrix of few rows (the 1024 x 4096 projection of
// the decode step, 1 / 4 / 8 tokens): with a warp per row every warp would fetch the activations of
// all tokens for itself (134 MB of L2 reads for 4 MB of weights at 8 tokens).  Here a CTA of sixteen
// warps takes eight rows, two warps per row (the halves of K), the tokens' activations are staged
// once per CTA in shared memory, a 16-byte piece of weights is decoded once for all tokens, and the
// two halves of a row are added through shared memory.  k a multiple of 32, 16-byte aligned operands.
constexpr uint32_t kFp8BlockRows = 8, kFp8BlockThreads = 512;
template <int NT, bool F32_SCALE>
__global__ void __launch_bounds__(kFp8BlockThreads)
k_fp8_matvec_block(const float *__restrict__ x, const uint8_t *__restrict__ w, const void *__restrict__ scale,
                   float *__restrict__ y, uint32_t n_rows, uint32_t k) {
    extern __shared__ __align__(16) float sx[];  // [NT][k]
    __shared__ double red[kFp8BlockRows][NT];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t r = warp & (kFp8BlockRows - 1u), half = warp >> 3;
    const uint32_t n = blockIdx.x * kFp8BlockRows + r;
    // staged as [token][quarter of a piece][piece]: the lanes of a warp, which hold consecutive pieces,
    // then read consecutive 16 bytes (no bank conflicts)
    const uint32_t pieces = k >> 4, per = pieces >> 1;
    for (uint32_t i = threadIdx.x; i < (NT * k) >> 2; i += kFp8BlockThreads) {
        const uint32_t t = i / (k >> 2), j = i % (k >> 2);
        reinterpret_cast<float4 *>(sx)[(size_t)t * (k >> 2) + (j & 3u) * pieces + (j >> 2)] =
            __ldg(reinterpret_cast<const float4 *>(x) + i);
    }
    __syncthreads();
    const uint32_t k_groups = (k + 127u) >> 7;
    double acc[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.0;
    if (n < n_rows) {
        const uint4 *wrow = reinterpret_cast<const uint4 *>(w + (size_t)n * k);
        const size_t srow = (size_t)(n >> 7) * k_groups;
        for (uint32_t p = half * per + lane; p < (half + 1u) * per; p += 32u) {
            const uint4 q = ldg_stream(wrow + p);
            const double sc = fp8_block_scale_f64<F32_SCALE>(scale, srow + (p >> 3));
            const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
            float2 wf[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t h0, h1;
                e4m3x4_to_h2x2(wd[i], h0, h1);
                wf[i * 2] = h2_to_f2(h0);
                wf[i * 2 + 1] = h2_to_f2(h1);
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float4 *xp = reinterpret_cast<const float4 *>(sx) + (size_t)t * (k >> 2) + p;
                float2 part = make_float2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 v = xp[(size_t)i * pieces];
                    part = __ffma2_rn(wf[i * 2], make_float2(v.x, v.y), part);
                    part = __ffma2_rn(wf[i * 2 + 1], make_float2(v.z, v.w), part);
                }
                acc[t] += (double)(part.x + part.y) * sc;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const double v = warp_sum(acc[t]);
        if (lane == 0 && half == 1u) red[r][t] = v;
        acc[t] = v;
    }
    __syncthreads();
    if (lane == 0 && half == 0u && n < n_rows) {
#pragma unroll
        for (int t = 0; t < NT; ++t) y[(size_t)t * n_rows + n] = (float)(acc[t] + red[r][t]);
    }
}

// Reference order: thread per (row, token), k ascending, (x*e)*s then add
// (examples/s14_vulkan_numeric.rs:1698-1714).
template <bool F32_SCALE>
__global__ void __launch_bounds__(128)
k_fp8_matvec_reference(const float *__restrict__ x, const uint8_t *__restrict__ w,
                       const void *__restrict__ scale, float *__restrict__ y, uint32_t n_rows,
                       uint32_t k, uint32_t n_tokens) {
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t t = blockIdx.y;
    if (n >= n_rows || t >= n_tokens) return;
    const uint32_t k_groups = (k + 127u) >> 7;
    const uint8_t *wrow = w + (size_t)n * k;
    const float *xt = x + (size_t)t * k;
    const size_t srow = (size_t)(n >> 7) * k_groups;
    float sum = 0.0f;
    for (uint32_t kg = 0; kg < k_groups; ++kg) {
        const float sc = fp8_block_scale_f32<F32_SCALE>(scale, srow + kg);
        const uint32_t k_end = min(kg * 128u + 128u, k);
        for (uint32_t kk = kg * 128u; kk < k_end; ++kk)
            sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(__ldg(xt + kk), e4m3_to_f32(__ldg(wrow + kk))), sc));
    }
    y[(size_t)t * n_rows + n] = sum;
}

// s14_swiglu_limit.comp:14-20
__global__ void k_swiglu_limit(const float *__restrict__ gate, const float *__restrict__ up,
                               float *__restrict__ y, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = swiglu_limit_f32(gate[i], up[i]);
}

// s14_route_mix.comp:16-20
__global__ void k_route_mix(const float *__restrict__ expert, float *__restrict__ routed, uint32_t n,
                            float weight) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) routed[i] = __fmul_rn(weight, expert[i]);
}

// s14_moe_accumulate.comp:17-21
__global__ void k_moe_accumulate(const float *__restrict__ expert, float *__restrict__ acc,
                                 uint32_t n, float weight) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) acc[i] = __fadd_rn(acc[i], __fmul_rn(weight, expert[i]));
}

// ------------------------------------------------------- fused MoE layer ----
//
// A job is one (expert page, token) pair.  Jobs of the same expert are adjacent
// so that the second and later tokens of an expert find its page in L2.
//   up   : h[job, i]    = swiglu(w1[i,:] . x_t, w3[i,:] . x_t)      i < inter
//   down : d[job, n]    = w2[n,:] . h[job,:]                        n < hidden
//   mix  : y[t, n]      = sum over the token's jobs, in route order, of
//                         weight * d[job, n]  (shared last, weight 1)

// One MXFP4 row against register-resident activations.  KC = K / 1024; lane l
// owns the 32 elements k = j*1024 + l*32 ... of every 1024-wide slice j, which is
// one 16-byte piece and one scale block.
template <int KC>
struct RowFrag {
    uint4 q[KC];
    uint32_t sc[KC];
};

// MAT: 0 = w1, 1 = w3 (rows of [inter, hidden]), 2 = w2 (rows of [hidden, inter]); `other` is the
// matrix's other dimension (inter for w1 / w3 rows of K = hidden, hidden for w2 rows of K = inter).
template <int KC, int MAT>
__device__ __forceinline__ void load_row_mxfp4(RowFrag<KC> &f, const PageView &pv, uint32_t row, uint32_t lane,
                                               uint32_t other) {
#pragma unroll
    for (int j = 0; j < KC; ++j) {
        const uint32_t kb = (uint32_t)j * 32u + lane;
        if (MAT < 2) {
            constexpr uint32_t hidden = KC * 1024;
            f.q[j] = ldg_stream(reinterpret_cast<const uint4 *>(pv.base + mxfp4_up_chunk_offset(MAT, row, kb, hidden)));
            f.sc[j] = __ldg(pv.base + mxfp4_up_scale_offset(MAT, row, kb, hidden, other));
        } else {
            constexpr uint32_t inter = KC * 1024;
            f.q[j] = ldg_stream(reinterpret_cast<const uint4 *>(pv.base + mxfp4_down_chunk_offset(row, kb, other, inter)));
            f.sc[j] = __ldg(pv.base + mxfp4_down_scale_offset(row, kb, other, inter));
        }
    }
}

template <int KC>
__device__ __forceinline__ double dot_row_mxfp4(const RowFrag<KC> &f, const float *__restrict__ xr) {
    double acc = 0.0;
#pragma unroll
    for (int j = 0; j < KC; ++j)
        acc += (double)dot32_e2m1(f.q[j], xr + j * 32) * ue8m0_to_f64(f.sc[j]);
    return acc;
}

// One FP8 row with the same lane-to-k mapping (two 16-byte pieces per slice).
template <int KC>
__device__ __forceinline__ double dot_row_fp8(const uint8_t *w, const uint8_t *s, uint32_t row,
                                              uint32_t lane, const float *__restrict__ xr) {
    const uint8_t *wrow = w + (size_t)row * (KC * 1024);
    const uint8_t *srow = s + (size_t)(row >> 7) * (KC * 8);
    double acc = 0.0;
#pragma unroll
    for (int j = 0; j < KC; ++j) {
        const uint4 *p = reinterpret_cast<const uint4 *>(wrow + j * 1024 + lane * 32);
        const uint4 q0 = __ldg(p), q1 = __ldg(p + 1);
        const float part = dot16_e4m3(q0, xr + j * 32) + dot16_e4m3(q1, xr + j * 32 + 16);
        acc += (double)part * ue8m0_to_f64(__ldg(srow + j * 8 + (lane >> 2)));
    }
    return acc;
}

template <int KC>
__device__ __forceinline__ void load_x_regs(float *xr, const float *__restrict__ x, uint32_t lane) {
#pragma unroll
    for (int j = 0; j < KC; ++j) {
        const float4 *xp = reinterpret_cast<const float4 *>(x + j * 1024 + lane * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 v = xp[i];
            xr[j * 32 + i * 4 + 0] = v.x;
            xr[j * 32 + i * 4 + 1] = v.y;
            xr[j * 32 + i * 4 + 2] = v.z;
            xr[j * 32 + i * 4 + 3] = v.w;
        }
    }
}

// Up phase, pairwise order.  grid = n_tokens * ctas_per_token; the warps of a CTA
// keep their token's x in registers and stride over that token's (job, row) space.
template <int KC>
__global__ void __launch_bounds__(256, 1)
k_expert_up_pairwise(const JobTable *__restrict__ dev_table,
                     const __grid_constant__ JobTable param_table, const float *__restrict__ x,
                     float *__restrict__ h, uint32_t inter, uint32_t ctas_per_token) {
    const JobTable &tab = table_of(dev_table, param_table);
    constexpr uint32_t hidden = KC * 1024;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t token = blockIdx.x / ctas_per_token;
    const uint32_t cta_in_token = blockIdx.x - token * ctas_per_token;
    const uint32_t warp = cta_in_token * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t n_warps = ctas_per_token * (blockDim.x >> 5);
    const uint32_t job0 = tab.token_job_begin[token];
    const uint32_t n_jobs = tab.token_job_begin[token + 1] - job0;
    const uint32_t items = n_jobs * inter;

    float xr[KC * 32];
    load_x_regs<KC>(xr, x + (size_t)token * hidden, lane);

    RowFrag<KC> g0, u0, g1, u1;
    uint32_t it = warp;
    auto issue = [&](RowFrag<KC> &g, RowFrag<KC> &u, uint32_t item) {
        const uint32_t job = job0 + item / inter, row = item % inter;
        const Job jb = tab.jobs[tab.token_jobs[job]];
        if (jb.kind == S14_PAGE_MXFP4) {
            const PageView pv = page_view(jb.page, jb.kind, hidden, inter);
            load_row_mxfp4<KC, 0>(g, pv, row, lane, inter);
            load_row_mxfp4<KC, 1>(u, pv, row, lane, inter);
        }
    };
    auto finish = [&](const RowFrag<KC> &g, const RowFrag<KC> &u, uint32_t item) {
        const uint32_t job = job0 + item / inter, row = item % inter;
        const uint32_t jid = tab.token_jobs[job];
        const Job jb = tab.jobs[jid];
        double gate, up;
        if (jb.kind == S14_PAGE_MXFP4) {
            gate = dot_row_mxfp4<KC>(g, xr);
            up = dot_row_mxfp4<KC>(u, xr);
        } else {
            const PageView pv = page_view(jb.page, jb.kind, hidden, inter);
            gate = dot_row_fp8<KC>(pv.w1, pv.s1, row, lane, xr);
            up = dot_row_fp8<KC>(pv.w3, pv.s3, row, lane, xr);
        }
        gate = warp_sum(gate);
        up = warp_sum(up);
        if (lane == 0) h[(size_t)jid * inter + row] = swiglu_limit_f32((float)gate, (float)up);
    };
    if (it < items) issue(g0, u0, it);
    while (it < items) {
        const uint32_t nx = it + n_warps;
        if (nx < items) issue(g1, u1, nx);
        finish(g0, u0, it);
        it = nx;
        if (it >= items) break;
        const uint32_t nx2 = it + n_warps;
        if (nx2 < items) issue(g0, u0, nx2);
        finish(g1, u1, it);
        it = nx2;
    }
}

// Down phase, pairwise order.  grid = n_jobs * ctas_per_job; a CTA's warps keep the
// job's h in registers and stride over the rows of w2.
template <int KC>
__global__ void __launch_bounds__(256, (KC >= 4 ? 1 : 2))
k_expert_down_pairwise(const JobTable *__restrict__ dev_table,
                       const __grid_constant__ JobTable param_table, const float *__restrict__ h,
                       float *__restrict__ d, uint32_t hidden, uint32_t ctas_per_job) {
    const JobTable &tab = table_of(dev_table, param_table);
    constexpr uint32_t inter = KC * 1024;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t jid = blockIdx.x / ctas_per_job;
    const uint32_t cta_in_job = blockIdx.x - jid * ctas_per_job;
    const uint32_t warp = cta_in_job * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t n_warps = ctas_per_job * (blockDim.x >> 5);
    if (jid >= tab.n_jobs) return;
    const Job jb = tab.jobs[jid];
    const PageView pv = page_view(jb.page, jb.kind, hidden, inter);

    float xr[KC * 32];
    load_x_regs<KC>(xr, h + (size_t)jid * inter, lane);
    float *out = d + (size_t)jb.out_index * hidden;

    if (jb.kind != S14_PAGE_MXFP4) {
        for (uint32_t row = warp; row < hidden; row += n_warps) {
            const double v = warp_sum(dot_row_fp8<KC>(pv.w2, pv.s2, row, lane, xr));
            if (lane == 0) out[row] = (float)v;
        }
        return;
    }
    RowFrag<KC> a0, a1, b0, b1;
    uint32_t row = warp;
    const uint32_t step = n_warps;
    // two rows per stage, two stages in flight
    auto issue2 = [&](RowFrag<KC> &p, RowFrag<KC> &q, uint32_t r) {
        if (r < hidden) load_row_mxfp4<KC, 2>(p, pv, r, lane, hidden);
        if (r + step < hidden) load_row_mxfp4<KC, 2>(q, pv, r + step, lane, hidden);
    };
    auto finish2 = [&](const RowFrag<KC> &p, const RowFrag<KC> &q, uint32_t r) {
        if (r < hidden) {
            const double v = warp_sum(dot_row_mxfp4<KC>(p, xr));
            if (lane == 0) out[r] = (float)v;
        }
        if (r + step < hidden) {
            const double v = warp_sum(dot_row_mxfp4<KC>(q, xr));
            if (lane == 0) out[r + step] = (float)v;
        }
    };
    if (row < hidden) issue2(a0, a1, row);
    while (row < hidden) {
        const uint32_t nx = row + 2 * step;
        if (nx < hidden) issue2(b0, b1, nx);
        finish2(a0, a1, row);
        row = nx;
        if (row >= hidden) break;
        const uint32_t nx2 = row + 2 * step;
        if (nx2 < hidden) issue2(a0, a1, nx2);
        finish2(b0, b1, row);
        row = nx2;
    }
}

// Reference-order dot of one MXFP4 row: sequential k, (x*e)*s, separate add.
// x is read from shared memory (every lane reads the same address: broadcast).
// MAT: 0 = w1, 1 = w3, 2 = w2 of an expert page; k is the row's length.
template <int MAT>
__device__ __forceinline__ float dot_row_mxfp4_reference(const PageView &pv, uint32_t row, uint32_t k, uint32_t hidden,
                                                         uint32_t inter, const float *__restrict__ xs) {
    const uint32_t groups = k >> 5;
    float sum = 0.0f;
    for (uint32_t g4 = 0; g4 < groups; g4 += 4) {
        uint4 q[4];
        uint32_t scw;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            q[j] = __ldg(reinterpret_cast<const uint4 *>(
                pv.base + (MAT < 2 ? mxfp4_up_chunk_offset(MAT, row, g4 + j, hidden)
                                   : mxfp4_down_chunk_offset(row, g4 + j, hidden, inter))));
        scw = __ldg(reinterpret_cast<const uint32_t *>(
            pv.base + (MAT < 2 ? mxfp4_up_scale_offset(MAT, row, g4, hidden, inter)
                               : mxfp4_down_scale_offset(row, g4, hidden, inter))));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float sc = ue8m0_to_f32((scw >> (8 * j)) & 0xffu);
            const uint32_t wd[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
            const float *xg = xs + (size_t)(g4 + j) * 32u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t hh[4];
                e2m1x8_to_h2x4(wd[i], hh[0], hh[1], hh[2], hh[3]);
                const float4 xa = *reinterpret_cast<const float4 *>(xg + i * 8);
                const float4 xb = *reinterpret_cast<const float4 *>(xg + i * 8 + 4);
                const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    const float2 e = h2_to_f2(hh[p]);
                    sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(xv[p * 2], e.x), sc));
                    sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(xv[p * 2 + 1], e.y), sc));
                }
            }
        }
    }
    return sum;
}

__device__ __forceinline__ float dot_row_fp8_reference(const uint8_t *w, const uint8_t *s,
                                                       uint32_t row, uint32_t k,
                                                       const float *__restrict__ xs) {
    const uint32_t k_groups = (k + 127u) >> 7;
    const uint4 *wrow = reinterpret_cast<const uint4 *>(w + (size_t)row * k);
    const uint8_t *srow = s + (size_t)(row >> 7) * k_groups;
    float sum = 0.0f;
    for (uint32_t kg = 0; kg < k_groups; ++kg) {
        const float sc = ue8m0_to_f32(__ldg(srow + kg));
        for (uint32_t p = 0; p < 8; ++p) {
            const uint4 q = __ldg(wrow + kg * 8 + p);
            const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
            const float *xg = xs + kg * 128u + p * 16u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t h0, h1;
                e4m3x4_to_h2x2(wd[i], h0, h1);
                const float4 xa = *reinterpret_cast<const float4 *>(xg + i * 4);
                const float2 e0 = h2_to_f2(h0), e1 = h2_to_f2(h1);
                sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(xa.x, e0.x), sc));
                sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(xa.y, e0.y), sc));
                sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(xa.z, e1.x), sc));
                sum = __fadd_rn(sum, __fmul_rn(__fmul_rn(xa.w, e1.y), sc));
            }
        }
    }
    return sum;
}

// Up phase, reference order: a thread owns gate row i and up row i of one job.
// grid = (ceil(inter/32), n_jobs), block = 32.
__global__ void __launch_bounds__(32)
k_expert_up_reference(const JobTable *__restrict__ dev_table,
                      const __grid_constant__ JobTable param_table, const float *__restrict__ x,
                      float *__restrict__ h, uint32_t hidden, uint32_t inter) {
    extern __shared__ __align__(16) float xs[];
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t jid = blockIdx.y;
    if (jid >= tab.n_jobs) return;
    const Job jb = tab.jobs[jid];
    const float *xt = x + (size_t)jb.token * hidden;
    for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = xt[i];
    __syncthreads();
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= inter) return;
    const PageView pv = page_view(jb.page, jb.kind, hidden, inter);
    float gate, up;
    if (jb.kind == S14_PAGE_MXFP4) {
        gate = dot_row_mxfp4_reference<0>(pv, row, hidden, hidden, inter, xs);
        up = dot_row_mxfp4_reference<1>(pv, row, hidden, hidden, inter, xs);
    } else {
        gate = dot_row_fp8_reference(pv.w1, pv.s1, row, hidden, xs);
        up = dot_row_fp8_reference(pv.w3, pv.s3, row, hidden, xs);
    }
    h[(size_t)jid * inter + row] = swiglu_limit_f32(gate, up);
}

// Down phase, reference order.  grid = (ceil(hidden/32), n_jobs), block = 32.
__global__ void __launch_bounds__(32)
k_expert_down_reference(const JobTable *__restrict__ dev_table,
                        const __grid_constant__ JobTable param_table, const float *__restrict__ h,
                        float *__restrict__ d, uint32_t hidden, uint32_t inter) {
    extern __shared__ __align__(16) float xs[];
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t jid = blockIdx.y;
    if (jid >= tab.n_jobs) return;
    const Job jb = tab.jobs[jid];
    const float *hj = h + (size_t)jid * inter;
    for (uint32_t i = threadIdx.x; i < inter; i += blockDim.x) xs[i] = hj[i];
    __syncthreads();
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= hidden) return;
    const PageView pv = page_view(jb.page, jb.kind, hidden, inter);
    const float v = (jb.kind == S14_PAGE_MXFP4)
                        ? dot_row_mxfp4_reference<2>(pv, row, inter, hidden, inter, xs)
                        : dot_row_fp8_reference(pv.w2, pv.s2, row, inter, xs);
    d[(size_t)jb.out_index * hidden + row] = v;
}

// Ordered mix (examples/s14_vulkan_numeric.rs:936-946): acc = 0; acc += w * d for the
// token's routed jobs in route order; acc += d_shared.  Separate multiply and add.
__global__ void __launch_bounds__(256)
k_moe_mix(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
          const float *__restrict__ d, float *__restrict__ y, uint32_t hidden) {
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t token = blockIdx.y;
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= hidden) return;
    const uint32_t j0 = tab.token_job_begin[token], j1 = tab.token_job_begin[token + 1];
    float acc = 0.0f;
    for (uint32_t j = j0; j < j1; ++j) {
        const uint32_t jid = tab.token_jobs[j];
        const Job jb = tab.jobs[jid];
        const float v = d[(size_t)jb.out_index * hidden + n];
        acc = jb.is_shared ? __fadd_rn(acc, v) : __fadd_rn(acc, __fmul_rn(jb.weight, v));
    }
    y[(size_t)token * hidden + n] = acc;
}

// Ordered mix of gathered per-slot expert outputs (expert-parallel combine): slots [n_routed (+1)]
// [hidden], weights on the device; same operations and order as k_moe_mix.
__global__ void __launch_bounds__(256)
k_mix_slots(const float *__restrict__ slots, const float *__restrict__ weights, uint32_t n_routed,
            int has_shared, float *__restrict__ y, uint32_t hidden) {
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= hidden) return;
    float acc = 0.0f;
    for (uint32_t j = 0; j < n_routed; ++j)
        acc = __fadd_rn(acc, __fmul_rn(weights[j], slots[(size_t)j * hidden + n]));
    if (has_shared) acc = __fadd_rn(acc, slots[(size_t)n_routed * hidden + n]);
    y[n] = acc;
}

// ------------------------------------------------------------- router -------

// One CTA of two warps per (token, expert) row of BF16 weights: logit in double (every product
// f32 x bf16 is exact in double), score and score + bias in F32.  The last CTA to finish
// (a counter in global memory, no waiting) selects the top-k of every token, normalises the
// weights and, for the one-token decode path, writes the job table of the layer.
__device__ __forceinline__ void router_select(const float *scores, const float *select,
                                              uint32_t n_experts, uint32_t top_k, float route_scale,
                                              int32_t *ids_out, float *weights_out, JobTable *table_out,
                                              const uint8_t *const *page_table, const uint8_t *shared_page,
                                              uint32_t shared_kind, uint32_t lane, uint32_t ep_rank,
                                              uint32_t ep_world, uint32_t shared_owner) {
    // key = (order-preserving bits of score + bias, ~expert): the largest key is the largest value,
    // the lowest expert id on ties; one 64-bit shuffle per butterfly step
    unsigned long long key[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t e = i * 32 + lane;
        key[i] = 0ull;
        if (e < n_experts) {
            const uint32_t bits = __float_as_uint(__ldcg(select + e));
            const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
            key[i] = ((unsigned long long)ordered << 32) | (unsigned long long)(0xffffffffu - e);
        }
    }
    int32_t ids[8];
    float picked[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        ids[j] = -1;
        picked[j] = 0.0f;
        if ((uint32_t)j < top_k) {
            unsigned long long best = key[0];
#pragma unroll
            for (int i = 1; i < 8; ++i) best = key[i] > best ? key[i] : best;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
                best = other > best ? other : best;
            }
            const uint32_t e = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (key[i] == best) key[i] = 0ull;  // taken
            ids[j] = (int32_t)e;
            picked[j] = __ldcg(scores + e);
        }
    }
    if (lane != 0) return;
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if ((uint32_t)j < top_k) sum = __fadd_rn(sum, picked[j]);
    // Expert parallel: this rank keeps the jobs of the experts it owns (id mod world == rank) and,
    // if it is the shared expert's owner, the shared job; every job writes the row of its route
    // slot so that the ranks' outputs add up to the full set.
    uint32_t n = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if ((uint32_t)j >= top_k) continue;
        const float w = __fmul_rn(__fdiv_rn(picked[j], sum), route_scale);
        if (ids_out) ids_out[j] = ids[j];
        if (weights_out) weights_out[j] = w;
        if (table_out && ((uint32_t)ids[j] % ep_world) == ep_rank) {
            Job jb;
            jb.page = page_table[ids[j]];
            jb.kind = S14_PAGE_MXFP4;
            jb.token = 0;
            jb.weight = w;
            jb.is_shared = 0;
            jb.out_index = (uint32_t)j;
            table_out->jobs[n] = jb;
            table_out->token_jobs[n] = (uint8_t)n;
            ++n;
        }
    }
    if (table_out) {
        if (shared_page && shared_owner == ep_rank) {
            Job jb;
            jb.page = shared_page;
            jb.kind = shared_kind;
            jb.token = 0;
            jb.weight = 1.0f;
            jb.is_shared = 1;
            jb.out_index = top_k;
            table_out->jobs[n] = jb;
            table_out->token_jobs[n] = (uint8_t)n;
            ++n;
        }
        table_out->n_jobs = n;
        table_out->n_tokens = 1;
        table_out->token_job_begin[0] = 0;
        table_out->token_job_begin[1] = n;
    }
}

__global__ void __launch_bounds__(64)
k_router(const float *__restrict__ x, const uint16_t *__restrict__ wr, const float *__restrict__ bias,
         float *__restrict__ scores, float *__restrict__ select, uint32_t n_experts, uint32_t hidden,
         uint32_t n_tokens, uint32_t score_fn, uint32_t top_k, float route_scale,
         int32_t *__restrict__ ids_out, float *__restrict__ weights_out, JobTable *__restrict__ table_out,
         const uint8_t *const *__restrict__ page_table, const uint8_t *shared_page, uint32_t shared_kind,
         unsigned int *__restrict__ counter, uint32_t ep_rank, uint32_t ep_world, uint32_t shared_owner) {
    __shared__ bool is_last;
    // a dependent launch (the up phase) may start its own prologue now; it reads what this
    // kernel writes only after cudaGridDependencySynchronize()
    cudaTriggerProgrammaticLaunchCompletion();
    __shared__ double half_sum[2];
    const uint32_t lane = threadIdx.x & 31u, half = threadIdx.x >> 5;
    {
        const uint32_t t = blockIdx.x / n_experts, e = blockIdx.x - t * n_experts;
        const uint32_t pieces = hidden >> 4;  // 16-byte pieces (8 weights) per half row
        const uint4 *row = reinterpret_cast<const uint4 *>(wr + (size_t)e * hidden) + half * pieces;
        const float *xt = x + (size_t)t * hidden + (size_t)half * (hidden >> 1);
        double acc0 = 0.0, acc1 = 0.0;
        for (uint32_t p0 = lane; p0 < pieces; p0 += 32u * 8u) {
            uint4 q[8];
            float4 xa[8], xb[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t p = p0 + u * 32u;
                if (p < pieces) {
                    q[u] = __ldg(row + p);
                    xa[u] = __ldg(reinterpret_cast<const float4 *>(xt + p * 8));
                    xb[u] = __ldg(reinterpret_cast<const float4 *>(xt + p * 8 + 4));
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (p0 + u * 32u < pieces) {
                    const uint32_t wd[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
                    const float xv[8] = {xa[u].x, xa[u].y, xa[u].z, xa[u].w, xb[u].x, xb[u].y, xb[u].z, xb[u].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc0 += (double)xv[i * 2] * (double)__uint_as_float(wd[i] << 16);
                        acc1 += (double)xv[i * 2 + 1] * (double)__uint_as_float(wd[i] & 0xffff0000u);
                    }
                }
            }
        }
        const double part = warp_sum(acc0 + acc1);
        if (lane == 0) half_sum[half] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
            const float s = router_score_f32(half_sum[0] + half_sum[1], score_fn);
            scores[(size_t)t * n_experts + e] = s;
            select[(size_t)t * n_experts + e] = __fadd_rn(s, bias ? bias[e] : 0.0f);
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(counter, 1u) == gridDim.x - 1u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (uint32_t t = threadIdx.x >> 5; t < n_tokens; t += blockDim.x >> 5)
        router_select(scores + (size_t)t * n_experts, select + (size_t)t * n_experts, n_experts, top_k,
                      route_scale, ids_out ? ids_out + (size_t)t * top_k : nullptr,
                      weights_out ? weights_out + (size_t)t * top_k : nullptr, table_out, page_table,
                      shared_page, shared_kind, lane, ep_rank, ep_world, shared_owner);
    if (threadIdx.x == 0) *counter = 0u;  // ready for the next launch
}

// --------------------------------------------------------------- LM head ----

// logits[t, v] = sum_k x[t,k] * bf16(W[v,k]); warp per vocabulary row; 8 products
// in F32, carried in F64.
template <int NT>
__global__ void __launch_bounds__(256)
k_head_logits(const float *__restrict__ x, const uint16_t *__restrict__ w, float *__restrict__ out,
              uint32_t n_rows, uint32_t hidden, uint32_t out_stride) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t n_warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t v = warp; v < n_rows; v += n_warps) {
        const uint4 *row = reinterpret_cast<const uint4 *>(w + (size_t)v * hidden);
        double acc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = 0.0;
        // four 16-byte loads of the row in flight per lane (the row is read once, from HBM); the sums
        // are taken in the order of the chunks, as before
        for (uint32_t p0 = lane; p0 < (hidden >> 3); p0 += 128u) {
            uint4 q4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                q4[u] = (p0 + 32u * u < (hidden >> 3)) ? ldg_stream(row + p0 + 32u * u) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t p = p0 + 32u * u;
                if (p >= (hidden >> 3)) break;
                const uint32_t wd[4] = {q4[u].x, q4[u].y, q4[u].z, q4[u].w};
                float wf[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    wf[i * 2] = __uint_as_float(wd[i] << 16);
                    wf[i * 2 + 1] = __uint_as_float(wd[i] & 0xffff0000u);
                }
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float4 xa = __ldg(reinterpret_cast<const float4 *>(x + (size_t)t * hidden + p * 8));
                    const float4 xb = __ldg(reinterpret_cast<const float4 *>(x + (size_t)t * hidden + p * 8 + 4));
                    float2 part = make_float2(0.f, 0.f);
                    part = __ffma2_rn(make_float2(wf[0], wf[1]), make_float2(xa.x, xa.y), part);
                    part = __ffma2_rn(make_float2(wf[2], wf[3]), make_float2(xa.z, xa.w), part);
                    part = __ffma2_rn(make_float2(wf[4], wf[5]), make_float2(xb.x, xb.y), part);
                    part = __ffma2_rn(make_float2(wf[6], wf[7]), make_float2(xb.z, xb.w), part);
                    acc[t] += (double)part.x + (double)part.y;
                }
            }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const double s = warp_sum(acc[t]);
            if (lane == 0) out[(size_t)t * out_stride + v] = (float)s;
        }
    }
}

// greedy argmax, lowest id wins ties, NaN -> -1; single block.
__global__ void __launch_bounds__(1024)
k_greedy_argmax(const float *__restrict__ logits, uint32_t vocab, int64_t *__restrict__ result) {
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    __shared__ int snan;
    if (threadIdx.x == 0) snan = 0;
    __syncthreads();
    float best = -INFINITY;
    uint32_t best_i = 0xffffffffu;
    bool nan = false;
    // four logits per load where the array allows it (a thread meets its indices in ascending order, so
    // "first largest" stays "lowest index" within a thread)
    const bool vec = (vocab & 3u) == 0u && (reinterpret_cast<uintptr_t>(logits) & 15u) == 0u;
    if (vec) {
        for (uint32_t i = threadIdx.x * 4u; i < vocab; i += blockDim.x * 4u) {
            const float4 q = *reinterpret_cast<const float4 *>(logits + i);
            const float vs[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                const float v = vs[k];
                nan |= (v != v);
                if (best_i == 0xffffffffu || v > best) {
                    best = v;
                    best_i = i + k;
                }
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = logits[i];
            nan |= (v != v);
            if (best_i == 0xffffffffu || v > best) {
                best = v;
                best_i = i;
            }
        }
    }
    if (nan) snan = 1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (oi != 0xffffffffu && (best_i == 0xffffffffu || ob > best || (ob == best && oi < best_i))) {
            best = ob;
            best_i = oi;
        }
    }
    if ((threadIdx.x & 31u) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x];
        best_i = si[threadIdx.x];
        if (threadIdx.x >= (blockDim.x >> 5)) best_i = 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (oi != 0xffffffffu && (best_i == 0xffffffffu || ob > best || (ob == best && oi < best_i))) {
                best = ob;
                best_i = oi;
            }
        }
        if (threadIdx.x == 0) *result = snan ? -1 : (int64_t)best_i;
    }
}

// ------------------------------------------------------------- launchers ----

static inline uint32_t ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

cudaError_t launch_mxfp4_matvec(cudaStream_t st, uint32_t mode, int sm_count, const float *x,
                                const uint8_t *w, const uint8_t *s, float *y, uint32_t n, uint32_t k) {
    if (mode == S14_ACCUM_REFERENCE) {
        k_mxfp4_matvec_reference<<<ceil_div(n, 128), 128, 0, st>>>(x, w, s, y, n, k);
    } else {
        const uint32_t blocks = min(ceil_div(n, 8), (uint32_t)sm_count * 8u);
        k_mxfp4_matvec_pairwise<<<blocks, 256, 0, st>>>(x, w, s, y, n, k);
    }
    return cudaGetLastError();
}

// Largest dynamic shared memory k_fp8_matvec_block may ask for on the current device (0: not set).
template <int NT, bool F32S>
static bool fp8_block_smem_ok(size_t bytes) {
    static int configured[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!configured[dev]) {
        configured[dev] = cudaFuncSetAttribute(k_fp8_matvec_block<NT, F32S>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               160 * 1024) == cudaSuccess ? 1 : -1;
    }
    return configured[dev] == 1 && bytes <= 160u * 1024u;
}

template <int NT, bool F32S>
static bool try_fp8_block(cudaStream_t st, int sm_count, const float *x, const uint8_t *w, const void *s, float *y,
                          uint32_t n, uint32_t k) {
    // few rows (a warp per row would leave most SMs with a handful of warps), k in whole scale
    // blocks, 16-byte aligned operands, the tokens' activations fit shared memory
    const size_t bytes = (size_t)NT * k * sizeof(float);
    if (n > (uint32_t)sm_count * 32u || (k & 31u) || ((uintptr_t)w & 15u) || ((uintptr_t)x & 15u)) return false;
    if (!fp8_block_smem_ok<NT, F32S>(bytes)) return false;
    k_fp8_matvec_block<NT, F32S><<<(n + kFp8BlockRows - 1) / kFp8BlockRows, kFp8BlockThreads, bytes, st>>>(x, w, s, y, n, k);
    return true;
}

template <bool F32S>
static void launch_fp8_pairwise_nt(cudaStream_t st, int sm_count, uint32_t blocks, uint32_t nt, const float *x,
                                   const uint8_t *w, const void *s, float *y, uint32_t n, uint32_t k) {
    bool done = false;
    switch (nt) {
    case 1: done = try_fp8_block<1, F32S>(st, sm_count, x, w, s, y, n, k); break;
    case 2: done = try_fp8_block<2, F32S>(st, sm_count, x, w, s, y, n, k); break;
    case 3: done = try_fp8_block<3, F32S>(st, sm_count, x, w, s, y, n, k); break;
    case 4: done = try_fp8_block<4, F32S>(st, sm_count, x, w, s, y, n, k); break;
    case 5: done = try_fp8_block<5, F32S>(st, sm_count, x, w, s, y, n, k); break;
    case 6: done = try_fp8_block<6, F32S>(st, sm_count, x, w, s, y, n, k); break;
    case 7: done = try_fp8_block<7, F32S>(st, sm_count, x, w, s, y, n, k); break;
    default: done = try_fp8_block<8, F32S>(st, sm_count, x, w, s, y, n, k); break;
    }
    if (done) return;
    switch (nt) {
    case 1: k_fp8_matvec_pairwise<1, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    case 2: k_fp8_matvec_pairwise<2, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    case 3: k_fp8_matvec_pairwise<3, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    case 4: k_fp8_matvec_pairwise<4, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    case 5: k_fp8_matvec_pairwise<5, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    case 6: k_fp8_matvec_pairwise<6, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    case 7: k_fp8_matvec_pairwise<7, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    default: k_fp8_matvec_pairwise<8, F32S><<<blocks, 256, 0, st>>>(x, w, s, y, n, k); break;
    }
}

cudaError_t launch_fp8_matvec(cudaStream_t st, uint32_t mode, int sm_count, uint32_t scale_format,
                              uint32_t n_tokens, const float *x, const uint8_t *w, const void *s,
                              float *y, uint32_t n, uint32_t k) {
    if (mode == S14_ACCUM_REFERENCE) {
        dim3 grid(ceil_div(n, 128), n_tokens);
        if (scale_format == S14_SCALE_F32)
            k_fp8_matvec_reference<true><<<grid, 128, 0, st>>>(x, w, s, y, n, k, n_tokens);
        else
            k_fp8_matvec_reference<false><<<grid, 128, 0, st>>>(x, w, s, y, n, k, n_tokens);
    } else {
        const uint32_t blocks = min(ceil_div(n, 8), (uint32_t)sm_count * 8u);
        if (scale_format == S14_SCALE_F32)
            launch_fp8_pairwise_nt<true>(st, sm_count, blocks, n_tokens, x, w, s, y, n, k);
        else
            launch_fp8_pairwise_nt<false>(st, sm_count, blocks, n_tokens, x, w, s, y, n, k);
    }
    return cudaGetLastError();
}

cudaError_t launch_swiglu_limit(cudaStream_t st, const float *gate, const float *up, float *y,
                                uint32_t n) {
    k_swiglu_limit<<<ceil_div(n, 256), 256, 0, st>>>(gate, up, y, n);
    return cudaGetLastError();
}

cudaError_t launch_route_mix(cudaStream_t st, const float *expert, float *routed, uint32_t n,
                             float weight) {
    k_route_mix<<<ceil_div(n, 256), 256, 0, st>>>(expert, routed, n, weight);
    return cudaGetLastError();
}

cudaError_t launch_moe_accumulate(cudaStream_t st, const float *expert, float *acc, uint32_t n,
                                  float weight) {
    k_moe_accumulate<<<ceil_div(n, 256), 256, 0, st>>>(expert, acc, n, weight);
    return cudaGetLastError();
}

template <int KC>
static void launch_up_pairwise(cudaStream_t st, const JobTable *dev, const JobTable &param,
                               const float *x, float *h, uint32_t inter, uint32_t n_tokens,
                               uint32_t ctas_per_token) {
    k_expert_up_pairwise<KC><<<n_tokens * ctas_per_token, 256, 0, st>>>(dev, param, x, h, inter,
                                                                        ctas_per_token);
}

template <int KC>
static void launch_down_pairwise(cudaStream_t st, const JobTable *dev, const JobTable &param,
                                 const float *h, float *d, uint32_t hidden, uint32_t n_jobs,
                                 uint32_t ctas_per_job) {
    k_expert_down_pairwise<KC><<<n_jobs * ctas_per_job, 256, 0, st>>>(dev, param, h, d, hidden,
                                                                      ctas_per_job);
}

// which implementation the calling thread's last launch_moe_layer chose (S14_LAYER_PATH_*)
static thread_local uint32_t t_last_layer_path = 0;
uint32_t last_layer_path() { return t_last_layer_path; }

int launch_moe_layer(cudaStream_t st, uint32_t mode, int sm_count, const JobTable *dev_table,
                     const JobTable &param_table, uint32_t n_tokens, uint32_t n_jobs_max,
                     uint32_t hidden, uint32_t inter, const float *x, float *h, float *d, float *y,
                     cudaError_t *err, const KernelMarks *km, bool all_mxfp4, unsigned int *counters,
                     const UmmaScratch *umma, const FusedRouter *router, const EpExchange *ep) {
    int launches = 0;
    *err = cudaSuccess;
    t_last_layer_path = 0;
    const bool tensor_path = mode != S14_ACCUM_REFERENCE && all_mxfp4 && counters && umma &&
                             umma_layer_ok(sm_count, n_tokens, n_jobs_max, hidden, inter);
    if (ep && ep->world > 1u && !(tensor_path && router && umma_router_ok(sm_count, router->n_experts))) {
        *err = cudaErrorNotSupported;  // the exchange over peer memory is part of the tensor-core layer kernel
        return launches;
    }
    if (router && !(tensor_path && umma_router_ok(sm_count, router->n_experts))) {
        // the routes come from a kernel of their own, which fills the device job table
        s14_router_desc r = {};
        r.x = x;
        r.router_weight_bf16 = router->weight;
        r.bias = router->bias;
        r.n_experts = router->n_experts;
        r.hidden = hidden;
        r.n_tokens = 1;
        r.score_fn = router->score_fn;
        r.top_k = router->top_k;
        r.route_scale = router->route_scale;
        r.ids_out = router->ids_out;
        r.weights_out = router->weights_out;
        launches += launch_router(st, r, router->scores, router->select, router->table_out, router->page_table,
                                  router->shared_page, router->shared_kind, counters, err, km, router->ep_rank,
                                  router->ep_world, router->shared_owner);
        if (*err != cudaSuccess) return launches;
        dev_table = router->table_out;
        router = nullptr;
        t_last_layer_path |= S14_LAYER_PATH_ROUTER_KERNEL;
    } else if (router && km) {
        cudaEventRecord(km->ev[0], st);
    }
    if (km) cudaEventRecord(km->ev[1], st);
    // A block of several tokens whose routes the caller gives (a verify block of up to eight tokens):
    // the tensor-core kernel takes one token per launch, so the block is one launch per token, each
    // with the token's own jobs in its mix order.  Launches follow one another in the stream (each a
    // programmatic dependent of the one before), a page that several tokens of the block use (the
    // shared expert always) is read from HBM by the first and found in the L2 by the others, and every
    // token's result is, bit for bit, that of its own one-token call.
    const bool block_on_tensor_path = mode != S14_ACCUM_REFERENCE && all_mxfp4 && counters && umma && n_tokens > 1u &&
                                      !router && !ep && !dev_table && y &&
                                      umma_layer_ok(sm_count, 1u, S14_EXPERTS_PER_TOKEN + 1u, hidden, inter);
    if (block_on_tensor_path) {
        bool fits = true;
        for (uint32_t t = 0; t < n_tokens; ++t)
            fits = fits && param_table.token_job_begin[t + 1] - param_table.token_job_begin[t] <= S14_EXPERTS_PER_TOKEN + 1u &&
                   param_table.token_job_begin[t + 1] > param_table.token_job_begin[t];
        if (fits) {
            for (uint32_t t = 0; t < n_tokens && *err == cudaSuccess; ++t) {
                JobTable one = {};
                const uint32_t b = param_table.token_job_begin[t], e = param_table.token_job_begin[t + 1];
                one.n_jobs = e - b;
                one.n_tokens = 1;
                one.token_job_begin[0] = 0;
                one.token_job_begin[1] = e - b;
                for (uint32_t i = b; i < e; ++i) {
                    Job jb = param_table.jobs[param_table.token_jobs[i]];
                    jb.token = 0;
                    jb.out_index = i - b;
                    one.jobs[i - b] = jb;
                    one.token_jobs[i - b] = (uint8_t)(i - b);
                }
                *err = launch_moe_layer_umma(st, sm_count, nullptr, one, x + (size_t)t * hidden, d, y + (size_t)t * hidden,
                                             umma->tiles, counters, umma->status, hidden, inter, nullptr, nullptr,
                                             umma->trace);
                launches += 1;
            }
            if (km) {
                cudaEventRecord(km->ev[2], st);
                cudaEventRecord(km->ev[3], st);
                cudaEventRecord(km->ev[4], st);
            }
            t_last_layer_path |= S14_LAYER_PATH_TENSOR_PER_TOKEN;
            return launches;
        }
    }
    if (mode == S14_ACCUM_REFERENCE) {
        dim3 gu(ceil_div(inter, 32), n_jobs_max), gd(ceil_div(hidden, 32), n_jobs_max);
        k_expert_up_reference<<<gu, 32, hidden * sizeof(float), st>>>(dev_table, param_table, x, h,
                                                                      hidden, inter);
        if (km) cudaEventRecord(km->ev[2], st);
        k_expert_down_reference<<<gd, 32, inter * sizeof(float), st>>>(dev_table, param_table, h, d,
                                                                       hidden, inter);
        launches += 2;
        t_last_layer_path |= S14_LAYER_PATH_REFERENCE;
    } else if (tensor_path) {
        *err = launch_moe_layer_umma(st, sm_count, dev_table, param_table, x, d, y, umma->tiles, counters,
                                     umma->status, hidden, inter, router, ep, umma->trace);
        launches += 1;
        t_last_layer_path |= S14_LAYER_PATH_TENSOR;
        if (km) {  // one kernel runs both phases and the mix: its time is booked as the up phase
            cudaEventRecord(km->ev[2], st);
            cudaEventRecord(km->ev[3], st);
            cudaEventRecord(km->ev[4], st);
        }
        return launches;
    } else {
        const uint32_t ctas_per_token = max(1u, (uint32_t)sm_count / n_tokens);
        switch (hidden >> 10) {
        case 1: launch_up_pairwise<1>(st, dev_table, param_table, x, h, inter, n_tokens, ctas_per_token); break;
        case 2: launch_up_pairwise<2>(st, dev_table, param_table, x, h, inter, n_tokens, ctas_per_token); break;
        default: launch_up_pairwise<4>(st, dev_table, param_table, x, h, inter, n_tokens, ctas_per_token); break;
        }
        if (km) cudaEventRecord(km->ev[2], st);
        const uint32_t ctas_per_job = max(1u, ceil_div(2u * (uint32_t)sm_count, n_jobs_max));
        switch (inter >> 10) {
        case 1: launch_down_pairwise<1>(st, dev_table, param_table, h, d, hidden, n_jobs_max, ctas_per_job); break;
        case 2: launch_down_pairwise<2>(st, dev_table, param_table, h, d, hidden, n_jobs_max, ctas_per_job); break;
        default: launch_down_pairwise<4>(st, dev_table, param_table, h, d, hidden, n_jobs_max, ctas_per_job); break;
        }
        launches += 2;
        t_last_layer_path |= S14_LAYER_PATH_F32;
    }
    if (km) cudaEventRecord(km->ev[3], st);
    if (!y) return launches;  // the caller mixes (expert-parallel combine)
    dim3 gm(ceil_div(hidden, 256), n_tokens);
    k_moe_mix<<<gm, 256, 0, st>>>(dev_table, param_table, d, y, hidden);
    if (km) cudaEventRecord(km->ev[4], st);
    launches += 1;
    *err = cudaGetLastError();
    return launches;
}

int launch_router(cudaStream_t st, const s14_router_desc &r, float *scores, float *select,
                  JobTable *table_out, const uint8_t *const *page_table, const uint8_t *shared_page,
                  uint32_t shared_kind, unsigned int *counter, cudaError_t *err, const KernelMarks *km,
                  uint32_t ep_rank, uint32_t ep_world, uint32_t shared_owner) {
    const uint32_t warps = r.n_experts * r.n_tokens;
    if (km) cudaEventRecord(km->ev[0], st);
    k_router<<<warps, 64, 0, st>>>(r.x, r.router_weight_bf16, r.bias, scores, select,
                                                r.n_experts, r.hidden, r.n_tokens, r.score_fn, r.top_k,
                                                r.route_scale, r.ids_out, r.weights_out, table_out,
                                                page_table, shared_page, shared_kind, counter, ep_rank,
                                                ep_world, shared_owner);
    *err = cudaGetLastError();
    return 1;
}

__global__ void __launch_bounds__(256)
k_stack_step(const float *__restrict__ x, const float *__restrict__ y, float *out, float *y_copy, uint32_t n,
             uint32_t residual) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = y[i];
    if (y_copy) y_copy[i] = v;
    out[i] = residual ? __fadd_rn(x[i], v) : v;
}

// ---- the router for many tokens ----
// Scores: a CTA holds the BF16 rows of eight experts in shared memory and walks a tile of 32 tokens,
// one warp per token at a time: logit in double (every product f32 x bf16 is exact in double), score
// and score + bias in F32 -- the arithmetic of k_router.
constexpr uint32_t kRbTokens = 32;
template <uint32_t kRbExperts, uint32_t kRbPerWarp>
__global__ void __launch_bounds__(256)
k_router_scores_batch(const float *__restrict__ x, const uint16_t *__restrict__ wr, const float *__restrict__ bias,
                      float *__restrict__ scores, float *__restrict__ select, uint32_t n_experts, uint32_t hidden,
                      uint32_t n_tokens, uint32_t score_fn) {
    extern __shared__ __align__(16) uint16_t s_w[];  // [kRbExperts][hidden]
    const uint32_t e0 = blockIdx.x * kRbExperts, t0 = blockIdx.y * kRbTokens;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t pieces = hidden >> 3;  // 16-byte pieces (8 weights) per row
    for (uint32_t i = threadIdx.x; i < kRbExperts * pieces; i += blockDim.x) {
        const uint32_t e = i / pieces, p = i - e * pieces;
        uint4 q = make_uint4(0u, 0u, 0u, 0u);
        if (e0 + e < n_experts) q = __ldg(reinterpret_cast<const uint4 *>(wr + (size_t)(e0 + e) * hidden) + p);
        reinterpret_cast<uint4 *>(s_w)[i] = q;
    }
    __syncthreads();
    // A warp takes kRbPerWarp tokens at a time, a weight's conversion to double serving all of them.  (Measured for
    // 370 tokens x 256 experts with eight experts per CTA: 165 us with one token per warp, 159 with four - the FP64
    // FMAs of the vector pipe bound it, not the conversions -, which is why large blocks take k_router_scores_dmma;
    // small blocks run this kernel with two experts per CTA and one token per warp.)
    for (uint32_t tb = t0 + warp * kRbPerWarp; tb < t0 + kRbTokens && tb < n_tokens; tb += 8u * kRbPerWarp) {
        double acc[kRbPerWarp][kRbExperts];
#pragma unroll
        for (uint32_t j = 0; j < kRbPerWarp; ++j)
#pragma unroll
            for (uint32_t e = 0; e < kRbExperts; ++e) acc[j][e] = 0.0;
        for (uint32_t p = lane; p < pieces; p += 32u) {
            double xv[kRbPerWarp][8];
#pragma unroll
            for (uint32_t j = 0; j < kRbPerWarp; ++j) {
                // (a token past the block's end reads the last token again; its result is not written)
                const float *xt = x + (size_t)min(tb + j, n_tokens - 1u) * hidden;
                const float4 xa = __ldg(reinterpret_cast<const float4 *>(xt + p * 8u));
                const float4 xb = __ldg(reinterpret_cast<const float4 *>(xt + p * 8u + 4u));
                xv[j][0] = xa.x, xv[j][1] = xa.y, xv[j][2] = xa.z, xv[j][3] = xa.w;
                xv[j][4] = xb.x, xv[j][5] = xb.y, xv[j][6] = xb.z, xv[j][7] = xb.w;
            }
#pragma unroll
            for (uint32_t e = 0; e < kRbExperts; ++e) {
                const uint4 q = reinterpret_cast<const uint4 *>(s_w + (size_t)e * hidden)[p];
                const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
                double w[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    w[i * 2] = (double)__uint_as_float(wd[i] << 16);
                    w[i * 2 + 1] = (double)__uint_as_float(wd[i] & 0xffff0000u);
                }
#pragma unroll
                for (uint32_t j = 0; j < kRbPerWarp; ++j) {
                    double a0 = 0.0, a1 = 0.0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        a0 += xv[j][i * 2] * w[i * 2];
                        a1 += xv[j][i * 2 + 1] * w[i * 2 + 1];
                    }
                    acc[j][e] += a0 + a1;
                }
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < kRbPerWarp; ++j) {
#pragma unroll
            for (uint32_t e = 0; e < kRbExperts; ++e) {
                const double sum = warp_sum(acc[j][e]);
                if (lane == 0 && e0 + e < n_experts && tb + j < n_tokens) {
                    const float sc = router_score_f32(sum, score_fn);
                    scores[(size_t)(tb + j) * n_experts + e0 + e] = sc;
                    select[(size_t)(tb + j) * n_experts + e0 + e] = __fadd_rn(sc, bias ? bias[e0 + e] : 0.0f);
                }
            }
        }
    }
}

// The same scores on the FP64 tensor path (B200 runs FP64 FMAs of the vector pipe at a sixteenth of
// the FP32 rate, and a block of hundreds of tokens needs 0.4 G of them): a CTA takes 32 tokens x 16
// experts, stages 256 elements of K at a time in shared memory as doubles (every f32 and bf16 value is
// exact in double, every product of the two exact, the accumulation in double as before, in another order),
// and its eight warps run mma.m8n8k4.f64 on 8 tokens x 8 experts each.
constexpr uint32_t kRdTokens = 32, kRdExperts = 16, kRdK = 256, kRdPitch = kRdK + 4;  // pitch: rows 32 bytes apart mod 128
__global__ void __launch_bounds__(256)
k_router_scores_dmma(const float *__restrict__ x, const uint16_t *__restrict__ wr, const float *__restrict__ bias,
                     float *__restrict__ scores, float *__restrict__ select, uint32_t n_experts, uint32_t hidden,
                     uint32_t n_tokens, uint32_t score_fn) {
    extern __shared__ __align__(16) double s_d[];
    double *sx = s_d;                           // [kRdTokens][kRdPitch]
    double *sw = s_d + kRdTokens * kRdPitch;    // [kRdExperts][kRdPitch]
    const uint32_t e0 = blockIdx.x * kRdExperts, t0 = blockIdx.y * kRdTokens;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t tg = warp & 3u, eg = warp >> 2;
    double c0 = 0.0, c1 = 0.0;
    for (uint32_t k0 = 0; k0 < hidden; k0 += kRdK) {
        __syncthreads();
#pragma unroll
        for (uint32_t i = 0; i < kRdTokens * kRdK / 4u / 256u; ++i) {
            const uint32_t idx = tid + 256u * i, t = idx / (kRdK / 4u), f4 = idx % (kRdK / 4u);
            // (a token past the block's end reads the last token again; its scores are not written)
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x + (size_t)min(t0 + t, n_tokens - 1u) * hidden + k0) + f4);
            double *d = sx + t * kRdPitch + f4 * 4u;
            *reinterpret_cast<double2 *>(d) = make_double2((double)v.x, (double)v.y);
            *reinterpret_cast<double2 *>(d + 2) = make_double2((double)v.z, (double)v.w);
        }
#pragma unroll
        for (uint32_t i = 0; i < kRdExperts * kRdK / 8u / 256u; ++i) {
            const uint32_t idx = tid + 256u * i, e = idx / (kRdK / 8u), p8 = idx % (kRdK / 8u);
            const uint4 q = __ldg(reinterpret_cast<const uint4 *>(wr + (size_t)min(e0 + e, n_experts - 1u) * hidden + k0) + p8);
            const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
            double *d = sw + e * kRdPitch + p8 * 8u;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<double2 *>(d + 2 * j) =
                    make_double2((double)__uint_as_float(wd[j] << 16), (double)__uint_as_float(wd[j] & 0xffff0000u));
        }
        __syncthreads();
        // A (8 tokens x 4 k, row major): lane holds (row lane / 4, column lane % 4); B (4 k x 8 experts, column
        // major): lane holds (row lane % 4, column lane / 4), i.e. the expert's row at the same k
        const double *pa = sx + (tg * 8u + (lane >> 2)) * kRdPitch + (lane & 3u);
        const double *pb = sw + (eg * 8u + (lane >> 2)) * kRdPitch + (lane & 3u);
#pragma unroll 8
        for (uint32_t k = 0; k < kRdK; k += 4u) {
            const double a = pa[k], b = pb[k];
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                         : "+d"(c0), "+d"(c1)
                         : "d"(a), "d"(b));
        }
    }
    // C (8 x 8): lane holds row lane / 4, columns 2 (lane % 4) and 2 (lane % 4) + 1
    const uint32_t t = t0 + tg * 8u + (lane >> 2), e = e0 + eg * 8u + (lane & 3u) * 2u;
    if (t < n_tokens) {
        if (e < n_experts) {
            const float sc = router_score_f32(c0, score_fn);
            scores[(size_t)t * n_experts + e] = sc;
            select[(size_t)t * n_experts + e] = __fadd_rn(sc, bias ? bias[e] : 0.0f);
        }
        if (e + 1u < n_experts) {
            const float sc = router_score_f32(c1, score_fn);
            scores[(size_t)t * n_experts + e + 1u] = sc;
            select[(size_t)t * n_experts + e + 1u] = __fadd_rn(sc, bias ? bias[e + 1u] : 0.0f);
        }
    }
}

// One warp per token picks the routes from the scores.
__global__ void __launch_bounds__(256)
k_router_select_batch(const float *__restrict__ scores, const float *__restrict__ select, uint32_t n_experts, uint32_t n_tokens,
                      uint32_t top_k, float route_scale, int32_t *__restrict__ ids_out, float *__restrict__ weights_out) {
    const uint32_t t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    router_select(scores + (size_t)t * n_experts, select + (size_t)t * n_experts, n_experts, top_k, route_scale,
                  ids_out + (size_t)t * top_k, weights_out + (size_t)t * top_k, nullptr, nullptr, nullptr, 0, threadIdx.x & 31u, 0,
                  1, 0);
}

int launch_router_batch(cudaStream_t st, const s14_router_desc &r, float *scores, float *select, cudaError_t *err) {
    // few tokens: two experts per CTA on the vector pipe, so that the grid covers the SMs; many: the FP64 tensor path
    static bool attr_set[64] = {};
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return 0;
    const size_t smem_d = (size_t)(kRdTokens + kRdExperts) * kRdPitch * sizeof(double);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        *err = cudaFuncSetAttribute(k_router_scores_dmma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_d);
        if (*err != cudaSuccess) return 0;
        attr_set[dev] = true;
    }
    if (r.n_tokens <= kRbTokens) {
        const dim3 grid(ceil_div(r.n_experts, 2u), ceil_div(r.n_tokens, kRbTokens));
        k_router_scores_batch<2, 1><<<grid, 256, (size_t)2u * r.hidden * sizeof(uint16_t), st>>>(
            r.x, r.router_weight_bf16, r.bias, scores, select, r.n_experts, r.hidden, r.n_tokens, r.score_fn);
    } else {
        const dim3 grid(ceil_div(r.n_experts, kRdExperts), ceil_div(r.n_tokens, kRdTokens));
        k_router_scores_dmma<<<grid, 256, smem_d, st>>>(r.x, r.router_weight_bf16, r.bias, scores, select, r.n_experts, r.hidden,
                                                       r.n_tokens, r.score_fn);
    }
    k_router_select_batch<<<ceil_div(r.n_tokens, 8), 256, 0, st>>>(scores, select, r.n_experts, r.n_tokens, r.top_k,
                                                                  r.route_scale, r.ids_out, r.weights_out);
    *err = cudaGetLastError();
    return 2;
}

cudaError_t launch_stack_step(cudaStream_t st, const float *x, const float *y, float *out, float *y_copy,
                              uint32_t n, bool residual) {
    k_stack_step<<<ceil_div(n, 256), 256, 0, st>>>(x, y, out, y_copy, n, residual ? 1u : 0u);
    return cudaGetLastError();
}

cudaError_t launch_mix_slots(cudaStream_t st, const float *slots, const float *weights, uint32_t n_routed,
                             int has_shared, float *y, uint32_t hidden) {
    k_mix_slots<<<ceil_div(hidden, 256), 256, 0, st>>>(slots, weights, n_routed, has_shared, y, hidden);
    return cudaGetLastError();
}

cudaError_t launch_head_logits(cudaStream_t st, int sm_count, const float *x, uint32_t n_tokens,
                               const uint16_t *w, uint32_t n_rows, uint32_t hidden, float *out,
                               uint32_t out_stride) {
    const uint32_t blocks = min(ceil_div(n_rows, 8), (uint32_t)sm_count * 8u);
    switch (n_tokens) {
    case 1: k_head_logits<1><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    case 2: k_head_logits<2><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    case 3: k_head_logits<3><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    case 4: k_head_logits<4><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    case 5: k_head_logits<5><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    case 6: k_head_logits<6><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    case 7: k_head_logits<7><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    default: k_head_logits<8><<<blocks, 256, 0, st>>>(x, w, out, n_rows, hidden, out_stride); break;
    }
    return cudaGetLastError();
}

cudaError_t launch_greedy_argmax(cudaStream_t st, const float *logits, uint32_t vocab,
                                 int64_t *result) {
    k_greedy_argmax<<<1, 1024, 0, st>>>(logits, vocab, result);
    return cudaGetLastError();
}

}  // namespace s14
