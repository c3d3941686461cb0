// Pairwise-order up and down phases of the fused MoE layer for MXFP4 pages, built around
// the warp-level f16 tensor-core dot product (mma.sync m16n8k16, F32 accumulate).
//
// Why tensor cores in a matvec: measured on B200 the F32 path needs a half-to-float
// widening (2 FMA-pipe slots per element) plus a multiply-add per element, which alone
// takes longer than streaming the weights from HBM.  Feeding the decoded f16x2 words
// straight into an MMA removes both; the only per-element work left is the hardware
// E2M1 -> f16x2 conversion (one instruction per byte).
//
// Exactness: the activation vector is split into three f16 limbs (11 + 11 + 2 bits, each
// limb pre-scaled by 2^11 / 2^22 so that it stays in f16 range after the token is
// normalised by a power of two); E2M1 values are exact in f16 and every product
// f16 x f16 is exact in the F32 accumulator.  One scale block (32 elements) is two MMAs;
// its result is multiplied by the block's power-of-two scale in F32, eight blocks are
// summed in F32 and carried on in F64.  The summation order differs from the reference's
// sequential F32 order, which is what S14_ACCUM_PAIRWISE means.
//
// Data movement: every warp owns 16 MMA rows (up phase: 8 gate rows of w1 and the 8 up
// rows of w3 with the same indices; down phase: 16 rows of w2) and streams them through a
// private cp.async ring in shared memory (16-byte coalesced copies, XOR-swizzled 128-byte
// rows), four stages of 256 K-elements deep, so that loads in flight do not depend on
// registers.  ldmatrix hands each lane the four bytes of its MMA fragment.
#include "s14_device.cuh"

namespace s14 {

namespace {

constexpr int kStages = 4;         // cp.async ring depth per warp
constexpr int kStageGroups = 8;    // scale blocks (32 elements) per stage: 128 B per row
constexpr int kTileRows = 16;      // MMA rows per warp tile
constexpr int kWarps = 8;          // warps per CTA
constexpr int kStageBytes = kTileRows * 128;          // weights of one warp stage
constexpr int kScaleStageBytes = kTileRows * 8;       // scale bytes of one warp stage
constexpr int kWarpSmem = kStages * (kStageBytes + kScaleStageBytes);

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                            uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory image of one token's activations as three f16 limbs: limb[j][k], each limb
// row padded by 64 bytes so that the three rows start in different banks.
__device__ __forceinline__ uint32_t limb_pitch_bytes(uint32_t k) { return k * 2u + 64u; }

// x = 2^e * (l1 + l2 * 2^-11 + l3 * 2^-22) exactly, |x| * 2^-e < 2.  Returns e.
__device__ int build_limbs(const float *__restrict__ x, uint32_t k, uint8_t *limbs, float *red) {
    float m = 0.0f;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) m = fmaxf(m, fabsf(x[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
    int e = 0;
    if (m > 0.0f && m < INFINITY) {
        frexpf(m, &e);  // m = f * 2^e, f in [0.5, 1)
        e = max(e, -100);
    }
    const float down = ldexpf(1.0f, -e);
    const uint32_t pitch = limb_pitch_bytes(k);
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        const float v = x[i] * down;  // exact: power of two, |v| < 1
        const __half l1 = __float2half_rn(v);
        const float r1 = (v - __half2float(l1)) * 2048.0f;  // exact
        const __half l2 = __float2half_rn(r1);
        const float r2 = (r1 - __half2float(l2)) * 2048.0f;  // exact, at most 2 bits
        const __half l3 = __float2half_rn(r2);
        reinterpret_cast<__half *>(limbs)[i] = l1;
        reinterpret_cast<__half *>(limbs + pitch)[i] = l2;
        reinterpret_cast<__half *>(limbs + 2 * pitch)[i] = l3;
    }
    __syncthreads();
    return e;
}

// Streams the 16 rows of one warp tile through the warp's ring and accumulates, per lane,
// the MMA output fragment (rows g and g+8, columns 2t and 2t+1 = limbs) in F64.
// row_ptr(m) gives the global address of MMA row m's packed codes, scale_ptr(m) its scale row.
struct TileRows {
    const uint8_t *w[2];   // base of MMA rows 0-7 and 8-15
    const uint8_t *s[2];
    uint32_t row0[2];      // first matrix row of each half
    uint32_t row_bytes;    // K / 2
    uint32_t scale_bytes;  // K / 32
};

__device__ __forceinline__ void issue_stage(const TileRows &tr, uint32_t stage_k, uint32_t wbuf,
                                            uint32_t sbuf, uint32_t lane) {
    // 16 rows x 128 B = 128 chunks of 16 B, four per lane; eight consecutive lanes cover one row
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t q = i * 32 + lane, m = q >> 3, c = q & 7u;
        const uint8_t *src = tr.w[m >> 3] + (size_t)(tr.row0[m >> 3] + (m & 7u)) * tr.row_bytes +
                             (size_t)stage_k * 128u + c * 16u;
        cp_async16(wbuf + m * 128u + ((c ^ (m & 7u)) << 4), src);
    }
    if (lane < 16) {
        const uint32_t m = lane;
        const uint8_t *src = tr.s[m >> 3] + (size_t)(tr.row0[m >> 3] + (m & 7u)) * tr.scale_bytes +
                             (size_t)stage_k * 8u;
        cp_async8(sbuf + m * 8u, src);
    }
}

__device__ __forceinline__ float scale_f32(uint32_t code) {
    return __uint_as_float(code ? (code << 23) : 0x00400000u);
}

__device__ __forceinline__ void compute_stage(uint32_t wbuf, const uint8_t *sbuf_gen,
                                              const uint8_t *limbs, uint32_t pitch, uint32_t k0,
                                              uint32_t lane, double (&acc)[4]) {
    const uint32_t g = lane >> 2, t = lane & 3u;
    // the eight scale codes of rows g and g+8 for this stage
    const uint2 sg = *reinterpret_cast<const uint2 *>(sbuf_gen + g * 8u);
    const uint2 sh = *reinterpret_cast<const uint2 *>(sbuf_gen + (g + 8u) * 8u);
    float part[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t mat = lane >> 3, r = lane & 7u;
    const uint32_t lm_row = r + ((mat & 1u) << 3);
    const uint32_t lm_base = wbuf + lm_row * 128u;
    const bool has_b = g < 3;
    const uint8_t *bptr = limbs + (has_b ? g : 0u) * pitch + (size_t)(k0 + t * 8u) * 2u;
#pragma unroll
    for (int cp = 0; cp < kStageGroups; cp += 2) {
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4(lm_base + ((((uint32_t)cp + (mat >> 1)) ^ (lm_row & 7u)) << 4), r0, r1, r2, r3);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int c = cp + half;
            const uint32_t lo = half ? r2 : r0, hi = half ? r3 : r1;
            uint4 b = make_uint4(0u, 0u, 0u, 0u);
            if (has_b) b = *reinterpret_cast<const uint4 *>(bptr + c * 64);
            uint32_t a0, a2, a0b, a2b, a1, a3, a1b, a3b;
            e2m1x8_to_h2x4(lo, a0, a2, a0b, a2b);
            e2m1x8_to_h2x4(hi, a1, a3, a1b, a3b);
            float cfrag[4] = {0.f, 0.f, 0.f, 0.f};
            mma_f16(cfrag, a0, a1, a2, a3, b.x, b.y);
            mma_f16(cfrag, a0b, a1b, a2b, a3b, b.z, b.w);
            const uint32_t cg = (c < 4 ? (sg.x >> (8 * c)) : (sg.y >> (8 * (c - 4)))) & 0xffu;
            const uint32_t ch = (c < 4 ? (sh.x >> (8 * c)) : (sh.y >> (8 * (c - 4)))) & 0xffu;
            const float fg = scale_f32(cg), fh = scale_f32(ch);
            part[0] = fmaf(cfrag[0], fg, part[0]);
            part[1] = fmaf(cfrag[1], fg, part[1]);
            part[2] = fmaf(cfrag[2], fh, part[2]);
            part[3] = fmaf(cfrag[3], fh, part[3]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += (double)part[i];
}

// Runs `n_tiles` tiles of this warp (tile ids first, first + stride, ...) as one flat
// cp.async pipeline; `setup(tile, tr)` fills the row pointers, `finish(tile, v_lo, v_hi)` gets
// the finished values of rows g (v_lo) and g+8 (v_hi) on the lanes with t == 0.
template <class Setup, class Finish>
__device__ __forceinline__ void run_tiles(uint32_t first, uint32_t stride, uint32_t total_tiles,
                                          uint32_t k, const uint8_t *limbs, int x_exp, uint8_t *ring,
                                          uint32_t lane, Setup setup, Finish finish) {
    if (first >= total_tiles) return;
    const uint32_t n_tiles = (total_tiles - first + stride - 1) / stride;
    const uint32_t stages_per_tile = k >> 8;
    const uint32_t total = n_tiles * stages_per_tile;
    const uint32_t pitch = limb_pitch_bytes(k);
    const uint32_t ring_w = smem_u32(ring);
    const uint32_t ring_s = ring_w + kStages * kStageBytes;
    const uint8_t *ring_s_gen = ring + kStages * kStageBytes;

    TileRows tr_issue;
    uint32_t issue_tile = 0xffffffffu;
    auto issue = [&](uint32_t f) {
        if (f < total) {
            const uint32_t ti = f / stages_per_tile, st = f - ti * stages_per_tile;
            if (ti != issue_tile) {
                setup(first + ti * stride, tr_issue);
                issue_tile = ti;
            }
            const uint32_t slot = f % kStages;
            issue_stage(tr_issue, st, ring_w + slot * kStageBytes, ring_s + slot * kScaleStageBytes, lane);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int f = 0; f < kStages - 1; ++f) issue(f);
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    for (uint32_t f = 0; f < total; ++f) {
        cp_async_wait<kStages - 2>();
        __syncwarp();
        const uint32_t ti = f / stages_per_tile, st = f - ti * stages_per_tile;
        const uint32_t slot = f % kStages;
        compute_stage(ring_w + slot * kStageBytes, ring_s_gen + slot * kScaleStageBytes, limbs, pitch,
                      st << 8, lane, acc);
        __syncwarp();
        issue(f + kStages - 1);
        if (st + 1 == stages_per_tile) {
            // columns: t == 0 holds limbs 0 and 1, t == 1 holds limb 2 (and an unused column)
            const double l2_lo = __shfl_down_sync(0xffffffffu, acc[0], 1);
            const double l2_hi = __shfl_down_sync(0xffffffffu, acc[2], 1);
            const double sc = ldexp(1.0, x_exp);
            const double v_lo = (acc[0] + acc[1] * (1.0 / 2048.0) + l2_lo * (1.0 / 4194304.0)) * sc;
            const double v_hi = (acc[2] + acc[3] * (1.0 / 2048.0) + l2_hi * (1.0 / 4194304.0)) * sc;
            finish(first + ti * stride, v_lo, v_hi);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0;
        }
    }
    cp_async_wait<0>();
}

}  // namespace

// Up phase.  grid = n_tokens * ctas_per_token, block = 256, dynamic smem =
// 8 * kWarpSmem + 3 * limb pitch.  Tiles of 8 row pairs of the token's jobs, which must all be
// MXFP4 pages (the launcher routes layers with an FP8 page to the F32 kernels).
__global__ void __launch_bounds__(256, 2)
k_expert_up_mma(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
                const float *__restrict__ x, float *__restrict__ h, uint32_t hidden, uint32_t inter,
                uint32_t ctas_per_token) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[kWarps];
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t token = blockIdx.x / ctas_per_token;
    const uint32_t cta_in_token = blockIdx.x - token * ctas_per_token;
    uint8_t *limbs = smem + kWarps * kWarpSmem;
    const int x_exp = build_limbs(x + (size_t)token * hidden, hidden, limbs, red);

    const uint32_t job0 = tab.token_job_begin[token];
    const uint32_t n_jobs = tab.token_job_begin[token + 1] - job0;
    const uint32_t tiles_per_job = inter >> 3;
    const uint32_t total_tiles = n_jobs * tiles_per_job;
    const uint32_t first = cta_in_token * kWarps + warp, stride = ctas_per_token * kWarps;
    const uint32_t g = lane >> 2, t = lane & 3u;

    auto setup = [&](uint32_t tile, TileRows &tr) {
        const uint32_t jid = tab.token_jobs[job0 + tile / tiles_per_job];
        const Job jb = tab.jobs[jid];
        const PageView pv = page_view(jb.page, S14_PAGE_MXFP4, hidden, inter);
        const uint32_t n0 = (tile % tiles_per_job) << 3;
        tr.w[0] = pv.w1;
        tr.w[1] = pv.w3;
        tr.s[0] = pv.s1;
        tr.s[1] = pv.s3;
        tr.row0[0] = tr.row0[1] = n0;
        tr.row_bytes = hidden >> 1;
        tr.scale_bytes = hidden >> 5;
    };
    auto finish = [&](uint32_t tile, double gate, double up) {
        if (t == 0) {
            const uint32_t jid = tab.token_jobs[job0 + tile / tiles_per_job];
            const uint32_t n0 = (tile % tiles_per_job) << 3;
            h[(size_t)jid * inter + n0 + g] = swiglu_limit_f32((float)gate, (float)up);
        }
    };
    run_tiles(first, stride, total_tiles, hidden, limbs, x_exp, smem + warp * kWarpSmem, lane, setup, finish);
}

// Down phase.  grid = n_jobs * ctas_per_job; a CTA keeps the limbs of its job's hidden vector.
__global__ void __launch_bounds__(256, 2)
k_expert_down_mma(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
                  const float *__restrict__ h, float *__restrict__ d, uint32_t hidden, uint32_t inter,
                  uint32_t ctas_per_job) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[kWarps];
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t jid = blockIdx.x / ctas_per_job;
    const uint32_t cta_in_job = blockIdx.x - jid * ctas_per_job;
    if (jid >= tab.n_jobs) return;
    const Job jb = tab.jobs[jid];
    if (jb.kind != S14_PAGE_MXFP4) return;
    uint8_t *limbs = smem + kWarps * kWarpSmem;
    const int x_exp = build_limbs(h + (size_t)jid * inter, inter, limbs, red);
    const PageView pv = page_view(jb.page, S14_PAGE_MXFP4, hidden, inter);
    const uint32_t total_tiles = hidden >> 4;
    const uint32_t first = cta_in_job * kWarps + warp, stride = ctas_per_job * kWarps;
    const uint32_t g = lane >> 2, t = lane & 3u;
    float *out = d + (size_t)jid * hidden;
    auto setup = [&](uint32_t tile, TileRows &tr) {
        tr.w[0] = tr.w[1] = pv.w2;
        tr.s[0] = tr.s[1] = pv.s2;
        tr.row0[0] = tile << 4;
        tr.row0[1] = (tile << 4) + 8u;
        tr.row_bytes = inter >> 1;
        tr.scale_bytes = inter >> 5;
    };
    auto finish = [&](uint32_t tile, double lo, double hi) {
        if (t == 0) {
            out[(tile << 4) + g] = (float)lo;
            out[(tile << 4) + 8u + g] = (float)hi;
        }
    };
    run_tiles(first, stride, total_tiles, inter, limbs, x_exp, smem + warp * kWarpSmem, lane, setup, finish);
}

static size_t mma_smem_bytes(uint32_t k) { return (size_t)kWarps * kWarpSmem + 3u * (k * 2u + 64u); }

cudaError_t launch_up_mma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                          const float *x, float *h, uint32_t hidden, uint32_t inter, uint32_t n_tokens) {
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(k_expert_up_mma, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)mma_smem_bytes(4096));
        cudaFuncSetAttribute(k_expert_down_mma, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)mma_smem_bytes(4096));
        configured = true;
    }
    const uint32_t ctas_per_token = max(1u, 2u * (uint32_t)sm_count / n_tokens);
    k_expert_up_mma<<<n_tokens * ctas_per_token, 256, mma_smem_bytes(hidden), st>>>(
        dev, param, x, h, hidden, inter, ctas_per_token);
    return cudaGetLastError();
}

cudaError_t launch_down_mma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                            const float *h, float *d, uint32_t hidden, uint32_t inter, uint32_t n_jobs) {
    const uint32_t ctas_per_job = max(1u, (2u * (uint32_t)sm_count + n_jobs - 1) / n_jobs);
    k_expert_down_mma<<<n_jobs * ctas_per_job, 256, mma_smem_bytes(inter), st>>>(
        dev, param, h, d, hidden, inter, ctas_per_job);
    return cudaGetLastError();
}

}  // namespace s14
