// The steps on either side of the MoE inside one layer: hyper-connection reduce (hc_pre) and expand
// (hc_post), RMSNorm, the head's reduce and the hash route of the first layers.  Reference:
//   fast16/research/polaris_meridian_v1/local_s14_primitives/hc.py:19-148
//   fast16/research/polaris_meridian_v1/local_s14_primitives/final_head.py:43-110
//   fast16/research/polaris_meridian_v1/s14_first_real_token/executor.py:638-668
// The Python code computes in F32 and leaves the order of its long sums and its exp to torch's CPU
// kernels.  Here the long sums (mean of squares, the dot products with hc_fn and with the router
// rows) are accumulated in double and rounded to F32 once, exp is evaluated in double and rounded
// once, and everything else follows the Python expressions operation by operation in F32 with
// separate multiplies and adds (no FMA), the sums over the four streams in stream order - the
// arithmetic of the CPU restatement the tests compare with.
// A token's state is hc = 4 streams of `hidden` values, F32 or BF16 (the reference's state is BF16
// [1, 1, 4, 4096]); results are rounded to the streams' type where the Python code casts back.
#include <cuda_bf16.h>

#include "s14_device.cuh"

namespace s14 {

namespace {

constexpr uint32_t kHc = 4;
constexpr uint32_t kMixMax = (2 + kHc) * kHc;

template <bool kBf16>
__device__ __forceinline__ float stream_ld(const void *p, size_t i) {
    if constexpr (kBf16) return __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t *>(p) + i) << 16);
    else return __ldg(reinterpret_cast<const float *>(p) + i);
}
template <bool kBf16>
__device__ __forceinline__ void stream_st(void *p, size_t i, float v) {
    if constexpr (kBf16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float *>(p)[i] = v;
}

// sum of v over the CTA's 256 threads (every thread gets it); red: 8 doubles of shared memory
__device__ __forceinline__ double block_sum_256(double v, double *red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31u) == 0u) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double s = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w];
    return s;
}

__device__ __forceinline__ float sigmoid_f32(float v) { return (float)(1.0 / (1.0 + exp(-(double)v))); }

// CTA (m, t): the dot product of token t's flattened streams with row m of fn, in double, rounded to
// F32; CTA (0, t) also writes the mean of the squares.  256 threads.
template <bool kBf16>
__global__ void __launch_bounds__(256)
k_hc_mixes(const void *__restrict__ x, const float *__restrict__ fn, uint32_t n, float *__restrict__ dots,
           float *__restrict__ mean_sq, uint32_t n_mix) {
    __shared__ double red[8];
    const uint32_t m = blockIdx.x, t = blockIdx.y;
    const float4 *row = reinterpret_cast<const float4 *>(fn + (size_t)m * n);
    double acc = 0.0, ss = 0.0;
    // four elements per thread and step, four steps' loads in flight (n is a multiple of 1024)
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < (n >> 2); i += 256u) {
        float v[4];
        if constexpr (kBf16) {
            const uint2 q = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(x) + (size_t)t * n) + i);
            v[0] = __uint_as_float(q.x << 16), v[1] = __uint_as_float(q.x & 0xffff0000u);
            v[2] = __uint_as_float(q.y << 16), v[3] = __uint_as_float(q.y & 0xffff0000u);
        } else {
            const float4 q = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + (size_t)t * n) + i);
            v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
        }
        const float4 w = __ldg(row + i);
        const float wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const double d = (double)v[k];
            acc += d * (double)wv[k];
            ss += d * d;
        }
    }
    const double dot = block_sum_256(acc, red);
    if (m == 0u) {
        const double s2 = block_sum_256(ss, red);
        if (threadIdx.x == 0) mean_sq[t] = (float)(s2 / (double)n);
    }
    if (threadIdx.x == 0) dots[(size_t)t * n_mix + m] = (float)dot;
}

// hc.py:19-84 by one warp: 24 logits -> pre [4], post [4], comb [4][4], F32 in the reference's order.  Lane
// l < 16 owns comb[l / 4][l % 4]; a row's or column's four values are fetched with shuffles and added in
// index order, as the Python sums do; lanes 0-3 also make pre and post.  All 32 lanes call it.
__device__ __forceinline__ void split_sinkhorn_warp(const float *mixes, const float *scale, const float *base, uint32_t iters,
                                                    float eps, uint32_t lane, float &pre, float &post, float &comb) {
    const uint32_t l = lane & 15u, i = l >> 2, j = l & 3u, h = lane & 3u;
    pre = __fadd_rn(sigmoid_f32(__fadd_rn(__fmul_rn(mixes[h], scale[0]), base[h])), eps);
    post = __fmul_rn(2.0f, sigmoid_f32(__fadd_rn(__fmul_rn(mixes[kHc + h], scale[1]), base[kHc + h])));
    float c = __fadd_rn(__fmul_rn(mixes[2 * kHc + l], scale[2]), base[2 * kHc + l]);
    auto row_sum = [&](float v, bool is_max) {
        const float r0 = __shfl_sync(0xffffffffu, v, i * 4u), r1 = __shfl_sync(0xffffffffu, v, i * 4u + 1u);
        const float r2 = __shfl_sync(0xffffffffu, v, i * 4u + 2u), r3 = __shfl_sync(0xffffffffu, v, i * 4u + 3u);
        if (is_max) return fmaxf(fmaxf(fmaxf(r0, r1), r2), r3);
        return __fadd_rn(__fadd_rn(__fadd_rn(r0, r1), r2), r3);
    };
    auto col_sum = [&](float v) {
        const float r0 = __shfl_sync(0xffffffffu, v, j), r1 = __shfl_sync(0xffffffffu, v, 4u + j);
        const float r2 = __shfl_sync(0xffffffffu, v, 8u + j), r3 = __shfl_sync(0xffffffffu, v, 12u + j);
        return __fadd_rn(__fadd_rn(__fadd_rn(r0, r1), r2), r3);
    };
    // stable row softmax, + eps
    c = (float)exp((double)__fsub_rn(c, row_sum(c, true)));
    c = __fadd_rn(__fdiv_rn(c, row_sum(c, false)), eps);
#pragma unroll 1
    for (uint32_t it = 0; it < iters; ++it) {
        if (it) c = __fdiv_rn(c, __fadd_rn(row_sum(c, false), eps));
        c = __fdiv_rn(c, __fadd_rn(col_sum(c), eps));
    }
    comb = c;
}

// One CTA per token: the coefficients from the dots (one warp), then reduced[d] = sum_h pre[h] x[h][d].
// kHead: the head's reduce (final_head.py:43-81): hc logits, pre = sigmoid(mix * scale + base) + eps only.
template <bool kBf16, bool kHead>
__global__ void __launch_bounds__(256)
k_hc_reduce(const void *__restrict__ x, const float *__restrict__ dots, const float *__restrict__ mean_sq,
            const float *__restrict__ scale, const float *__restrict__ base, uint32_t hidden, float norm_eps, uint32_t iters,
            float hc_eps, void *__restrict__ reduced, float *__restrict__ post_out, float *__restrict__ comb_out,
            float *__restrict__ pre_out) {
    __shared__ float s_pre[kHc], s_mix[kMixMax];
    const uint32_t t = blockIdx.x, lane = threadIdx.x & 31u;
    constexpr uint32_t n_mix = kHead ? kHc : kMixMax;
    if (threadIdx.x < 32u) {
        const float rs = (float)(1.0 / sqrt((double)__fadd_rn(mean_sq[t], norm_eps)));
        if (lane < n_mix) s_mix[lane] = __fmul_rn(dots[(size_t)t * n_mix + lane], rs);
        __syncwarp();
        float pre;
        if constexpr (kHead) {
            const uint32_t h = lane & 3u;
            pre = __fadd_rn(sigmoid_f32(__fadd_rn(__fmul_rn(s_mix[h], scale[0]), base[h])), hc_eps);
        } else {
            float post, comb;
            split_sinkhorn_warp(s_mix, scale, base, iters, hc_eps, lane, pre, post, comb);
            if (lane < kHc) post_out[(size_t)t * kHc + lane] = post;
            if (lane < kHc * kHc) comb_out[(size_t)t * kHc * kHc + lane] = comb;
        }
        if (lane < kHc) {
            s_pre[lane] = pre;
            if (pre_out) pre_out[(size_t)t * kHc + lane] = pre;
        }
    }
    __syncthreads();
    const size_t x0 = (size_t)t * kHc * hidden;
    for (uint32_t d = threadIdx.x; d < hidden; d += 256u) {
        float acc = __fmul_rn(s_pre[0], stream_ld<kBf16>(x, x0 + d));
#pragma unroll
        for (uint32_t h = 1; h < kHc; ++h) acc = __fadd_rn(acc, __fmul_rn(s_pre[h], stream_ld<kBf16>(x, x0 + (size_t)h * hidden + d)));
        stream_st<kBf16>(reduced, (size_t)t * hidden + d, acc);
    }
}

// hc.py:127-148: merged[t][o][d] = post[o] * branch[d] + sum_h comb[h][o] * residual[h][d].
template <bool kBf16>
__global__ void __launch_bounds__(256)
k_hc_post(const void *__restrict__ branch, const void *__restrict__ residual, const float *__restrict__ post,
          const float *__restrict__ comb, uint32_t hidden, void *__restrict__ merged) {
    const uint32_t d = blockIdx.x * 256u + threadIdx.x, t = blockIdx.y;
    if (d >= hidden) return;
    float r[kHc], c[kHc * kHc], p[kHc];
#pragma unroll
    for (uint32_t h = 0; h < kHc; ++h) {
        r[h] = stream_ld<kBf16>(residual, ((size_t)t * kHc + h) * hidden + d);
        p[h] = __ldg(post + (size_t)t * kHc + h);
    }
#pragma unroll
    for (uint32_t i = 0; i < kHc * kHc; ++i) c[i] = __ldg(comb + (size_t)t * kHc * kHc + i);
    const float b = stream_ld<kBf16>(branch, (size_t)t * hidden + d);
#pragma unroll
    for (uint32_t o = 0; o < kHc; ++o) {
        float s = __fmul_rn(c[o], r[0]);
#pragma unroll
        for (uint32_t h = 1; h < kHc; ++h) s = __fadd_rn(s, __fmul_rn(c[h * kHc + o], r[h]));
        stream_st<kBf16>(merged, ((size_t)t * kHc + o) * hidden + d, __fadd_rn(__fmul_rn(p[o], b), s));
    }
}

// final_head.py:84-110: out = w * (x * rsqrt(mean(x^2) + eps)); one CTA per token.
template <bool kBf16>
__global__ void __launch_bounds__(256)
k_rms_norm(const void *__restrict__ x, const float *__restrict__ w, uint32_t hidden, float eps, void *__restrict__ out) {
    __shared__ double red[8];
    const uint32_t t = blockIdx.x;
    double ss = 0.0;
    for (uint32_t i = threadIdx.x; i < hidden; i += 256u) {
        const double v = (double)stream_ld<kBf16>(x, (size_t)t * hidden + i);
        ss += v * v;
    }
    const float ms = (float)(block_sum_256(ss, red) / (double)hidden);
    const float rs = (float)(1.0 / sqrt((double)__fadd_rn(ms, eps)));
    for (uint32_t i = threadIdx.x; i < hidden; i += 256u)
        stream_st<kBf16>(out, (size_t)t * hidden + i, __fmul_rn(__ldg(w + i), __fmul_rn(stream_ld<kBf16>(x, (size_t)t * hidden + i), rs)));
}

// executor.py:638-668 for the hash-routed layers: the ids are the token's row of tid2eid, the weights the
// router's scores of those experts, normalised and scaled.  One CTA per token, warp j scores expert j.
__global__ void __launch_bounds__(256)
k_router_hash(const float *__restrict__ x, const uint16_t *__restrict__ wr, const long long *__restrict__ tid2eid,
              uint32_t n_experts, uint32_t hidden, uint32_t top_k, uint32_t score_fn, float route_scale,
              int32_t *__restrict__ ids_out, float *__restrict__ weights_out) {
    __shared__ float s_sc[8];
    const uint32_t t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (warp < top_k) {
        const long long e = tid2eid[(size_t)t * top_k + warp];
        double acc = 0.0;
        if (e >= 0 && (unsigned long long)e < n_experts) {
            const uint16_t *row = wr + (size_t)e * hidden;
            for (uint32_t k = lane; k < hidden; k += 32u)
                acc += (double)__ldg(x + (size_t)t * hidden + k) * (double)__uint_as_float((uint32_t)__ldg(row + k) << 16);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            s_sc[warp] = router_score_f32(acc, score_fn);
            ids_out[(size_t)t * top_k + warp] = (int32_t)e;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (uint32_t j = 0; j < top_k; ++j) sum = __fadd_rn(sum, s_sc[j]);
        for (uint32_t j = 0; j < top_k; ++j) weights_out[(size_t)t * top_k + j] = __fmul_rn(__fdiv_rn(s_sc[j], sum), route_scale);
    }
}

__global__ void __launch_bounds__(256) k_bf16_to_f32(const uint16_t *__restrict__ in, float *__restrict__ out, uint32_t n) {
    const uint32_t i = blockIdx.x * 256u + threadIdx.x;
    if (i < n) out[i] = __uint_as_float((uint32_t)__ldg(in + i) << 16);
}
__global__ void __launch_bounds__(256) k_f32_to_bf16(const float *__restrict__ in, __nv_bfloat16 *__restrict__ out, uint32_t n) {
    const uint32_t i = blockIdx.x * 256u + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(__ldg(in + i));
}

}  // namespace

cudaError_t launch_bf16_to_f32(cudaStream_t st, const uint16_t *in, float *out, uint32_t n) {
    k_bf16_to_f32<<<(n + 255u) / 256u, 256, 0, st>>>(in, out, n);
    return cudaGetLastError();
}
cudaError_t launch_f32_to_bf16(cudaStream_t st, const float *in, uint16_t *out, uint32_t n) {
    k_f32_to_bf16<<<(n + 255u) / 256u, 256, 0, st>>>(in, reinterpret_cast<__nv_bfloat16 *>(out), n);
    return cudaGetLastError();
}

// dots: [n_tokens, 24] scratch, mean_sq: [n_tokens] scratch.  Returns the number of kernels launched.
int launch_hc_pre(cudaStream_t st, bool bf16, bool head, uint32_t n_tokens, uint32_t hidden, const void *x, const float *fn,
                  const float *scale, const float *base, float norm_eps, uint32_t iters, float hc_eps, float *dots, float *mean_sq,
                  void *reduced, float *post, float *comb, float *pre, cudaError_t *err) {
    const uint32_t n_mix = head ? kHc : kMixMax, n = kHc * hidden;
    const dim3 grid(n_mix, n_tokens);
    if (bf16) k_hc_mixes<true><<<grid, 256, 0, st>>>(x, fn, n, dots, mean_sq, n_mix);
    else k_hc_mixes<false><<<grid, 256, 0, st>>>(x, fn, n, dots, mean_sq, n_mix);
    if (bf16 && head) k_hc_reduce<true, true><<<n_tokens, 256, 0, st>>>(x, dots, mean_sq, scale, base, hidden, norm_eps, iters, hc_eps, reduced, post, comb, pre);
    else if (bf16) k_hc_reduce<true, false><<<n_tokens, 256, 0, st>>>(x, dots, mean_sq, scale, base, hidden, norm_eps, iters, hc_eps, reduced, post, comb, pre);
    else if (head) k_hc_reduce<false, true><<<n_tokens, 256, 0, st>>>(x, dots, mean_sq, scale, base, hidden, norm_eps, iters, hc_eps, reduced, post, comb, pre);
    else k_hc_reduce<false, false><<<n_tokens, 256, 0, st>>>(x, dots, mean_sq, scale, base, hidden, norm_eps, iters, hc_eps, reduced, post, comb, pre);
    *err = cudaGetLastError();
    return 2;
}

cudaError_t launch_hc_post(cudaStream_t st, bool bf16, uint32_t n_tokens, uint32_t hidden, const void *branch, const void *residual,
                           const float *post, const float *comb, void *merged) {
    const dim3 grid((hidden + 255u) / 256u, n_tokens);
    if (bf16) k_hc_post<true><<<grid, 256, 0, st>>>(branch, residual, post, comb, hidden, merged);
    else k_hc_post<false><<<grid, 256, 0, st>>>(branch, residual, post, comb, hidden, merged);
    return cudaGetLastError();
}

cudaError_t launch_rms_norm(cudaStream_t st, bool bf16, uint32_t n_tokens, uint32_t hidden, const void *x, const float *w, float eps,
                            void *out) {
    if (bf16) k_rms_norm<true><<<n_tokens, 256, 0, st>>>(x, w, hidden, eps, out);
    else k_rms_norm<false><<<n_tokens, 256, 0, st>>>(x, w, hidden, eps, out);
    return cudaGetLastError();
}

cudaError_t launch_router_hash(cudaStream_t st, const s14_router_desc &r, const int64_t *tid2eid) {
    k_router_hash<<<r.n_tokens, 256, 0, st>>>(r.x, r.router_weight_bf16, reinterpret_cast<const long long *>(tid2eid), r.n_experts,
                                             r.hidden, r.top_k, r.score_fn, r.route_scale, r.ids_out, r.weights_out);
    return cudaGetLastError();
}

}  // namespace s14
