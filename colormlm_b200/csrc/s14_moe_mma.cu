// Pairwise-order up and down phases of the fused MoE layer for MXFP4 pages, built around
// the warp-level f16 tensor-core dot product (mma.sync m16n8k16, F32 accumulate).
//
// Why tensor cores in a matvec: measured on B200, the F32 path needs a half-to-float
// widening (2 FMA-pipe slots per element) plus a multiply-add per element, which alone
// takes longer than streaming the weights from HBM.  Feeding the decoded f16x2 words
// straight into an MMA removes both; the per-element work left is the hardware
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
// Data movement: one CTA per SM.  A warp streams tiles of 16 MMA rows (up phase: 8 gate
// rows of w1 and the 8 up rows of w3 with the same indices; down phase: 16 rows of w2)
// through a private cp.async ring in shared memory (16-byte coalesced copies,
// XOR-swizzled 128-byte rows, stages of 256 K-elements), so that loads in flight do not
// depend on registers; ldmatrix hands each lane the four bytes of its MMA fragment.  When a
// CTA has few tiles, its (tile, stage) list is cut into equal runs for the warps and the
// partial sums of a tile meet in shared memory in a fixed order.
#include "s14_device.cuh"


namespace s14 {

namespace {

constexpr int kStages = 4;                        // cp.async ring depth per warp
constexpr int kMaxWarps = 16;                     // warps per CTA (one CTA per SM)
constexpr int kStageBytes = 16 * 128;             // 16 rows x 128 B of codes
constexpr int kScaleRaw = 16 * 8;                 // 16 rows x 8 scale codes
constexpr int kConvPitch = 80;                    // bytes per row of converted scales (8 x (f, f) + pad)
constexpr int kConvBytes = 16 * kConvPitch;
constexpr int kWarpSmem = kStages * (kStageBytes + kScaleRaw) + kConvBytes;
constexpr int kSplitTiles = 16;                   // at most this many tiles per CTA are cut into runs
constexpr int kMaxSeg = 3;                        // runs that can touch one tile
constexpr int kPartBytes = kSplitTiles * kMaxSeg * 16 * 8;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                            uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// d = a * b + c; not volatile so that independent MMAs can be interleaved by the scheduler.
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1, float c0, float c1,
                                        float c2, float c3) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

// Shared-memory image of one token's activations: three f16 limb rows and one row of zeros
// (the B fragment of the five unused MMA columns), each padded by 64 bytes.
__device__ __forceinline__ uint32_t limb_pitch_bytes(uint32_t k) { return k * 2u + 64u; }

// x = 2^e * (l1 + l2 * 2^-11 + l3 * 2^-22) exactly, |x| * 2^-e < 1.  Returns e.  The caller
// synchronises the CTA before the limbs are read.
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
        const float v = x[i] * down;  // exact: power of two
        const __half l1 = __float2half_rn(v);
        const float r1 = (v - __half2float(l1)) * 2048.0f;  // exact
        const __half l2 = __float2half_rn(r1);
        const float r2 = (r1 - __half2float(l2)) * 2048.0f;  // exact, at most 2 bits
        const __half l3 = __float2half_rn(r2);
        reinterpret_cast<__half *>(limbs)[i] = l1;
        reinterpret_cast<__half *>(limbs + pitch)[i] = l2;
        reinterpret_cast<__half *>(limbs + 2 * pitch)[i] = l3;
        reinterpret_cast<uint16_t *>(limbs + 3 * pitch)[i] = 0;
    }
    return e;
}

// Rows of one tile: MMA rows 0-7 are rows r0.. of matrix (w0, s0), rows 8-15 rows r1.. of (w1, s1).
struct TileRows {
    const uint8_t *w0, *w1, *s0, *s1;
    uint32_t r0, r1;
};

// Per-lane source pointers of a tile (stage 0) and destination offsets inside a ring slot: the 16
// rows x 128 B of a stage are 128 pieces of 16 B, four per lane, eight consecutive lanes per row.
struct LaneCopy {
    const uint8_t *src[4];
    const uint8_t *ssrc;  // scale codes, lanes 0-15
    uint32_t dst[4];
};

__device__ __forceinline__ void lane_copy_init(LaneCopy &lc, uint32_t lane) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t m = i * 4 + (lane >> 3), c = lane & 7u;
        lc.dst[i] = m * 128u + ((c ^ (m & 7u)) << 4);
    }
}

__device__ __forceinline__ void lane_copy_tile(LaneCopy &lc, const TileRows &tr, uint32_t row_bytes,
                                               uint32_t scale_bytes, uint32_t lane) {
    const uint32_t sub = lane >> 3, c = lane & 7u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // i < 2: MMA rows 0-7, else rows 8-15
        const uint8_t *base = (i < 2) ? tr.w0 : tr.w1;
        const uint32_t row = ((i < 2) ? tr.r0 : tr.r1) + ((i & 1) * 4 + sub);
        lc.src[i] = base + (size_t)row * row_bytes + c * 16u;
    }
    const uint8_t *sbase = (lane < 8) ? tr.s0 : tr.s1;
    lc.ssrc = sbase + scale_word_offset(((lane < 8) ? tr.r0 : tr.r1) + (lane & 7u), 0, scale_bytes << 5);
}

__device__ __forceinline__ void issue_stage(const LaneCopy &lc, uint32_t stage_k, uint32_t wbuf, uint32_t sbuf,
                                            uint32_t lane) {
#pragma unroll
    for (int i = 0; i < 4; ++i) cp_async16(wbuf + lc.dst[i], lc.src[i] + stage_k * 128u);
    if (lane < 16) {  // eight codes of a row: two words, one per atom
        cp_async4(sbuf + lane * 8u, lc.ssrc + stage_k * 1024u);
        cp_async4(sbuf + lane * 8u + 4u, lc.ssrc + stage_k * 1024u + 512u);
    }
}

// The 128 scale codes of a stage -> (f, f) pairs of 2^(code-127) in the warp's conversion area.
__device__ __forceinline__ void convert_scales(const uint8_t *raw, uint8_t *conv, uint32_t lane) {
    const uint32_t w = reinterpret_cast<const uint32_t *>(raw)[lane];  // row lane/2, codes (lane&1)*4..
    uint32_t b[4];
    b[0] = (w & 0xffu) << 23;
    b[1] = (w << 15) & 0x7f800000u;
    b[2] = (w << 7) & 0x7f800000u;
    b[3] = (w >> 1) & 0x7f800000u;
    if (((w - 0x01010101u) & ~w & 0x80808080u) != 0u) {  // code 0 is the subnormal 2^-127
#pragma unroll
        for (int i = 0; i < 4; ++i) b[i] = b[i] ? b[i] : 0x00400000u;
    }
    uint4 *dst = reinterpret_cast<uint4 *>(conv + (lane >> 1) * kConvPitch + (lane & 1u) * 32u);
    dst[0] = make_uint4(b[0], b[0], b[1], b[1]);
    dst[1] = make_uint4(b[2], b[2], b[3], b[3]);
}

// One stage = eight scale blocks of the warp's 16 rows.  Four blocks at a time: two ldmatrix.x4,
// four B fragments, eight MMAs (four independent chains of two), then the scale multiply.
__device__ __forceinline__ void compute_stage(uint32_t wbuf, const uint8_t *conv, const uint8_t *bptr,
                                              uint32_t lane, double (&acc)[4]) {
    const uint32_t g = lane >> 2;
    float2 p_lo = make_float2(0.f, 0.f), p_hi = make_float2(0.f, 0.f);
    const uint32_t mat = lane >> 3, r = lane & 7u;
    const uint32_t lm_row = r + ((mat & 1u) << 3);
    const uint32_t lm_base = wbuf + lm_row * 128u;
    const uint8_t *cg = conv + g * kConvPitch, *ch = conv + (g + 8u) * kConvPitch;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        uint32_t raw[8];
        ldmatrix_x4(lm_base + ((((uint32_t)(4 * hh) + (mat >> 1)) ^ (lm_row & 7u)) << 4), raw[0], raw[1],
                    raw[2], raw[3]);
        ldmatrix_x4(lm_base + ((((uint32_t)(4 * hh + 2) + (mat >> 1)) ^ (lm_row & 7u)) << 4), raw[4], raw[5],
                    raw[6], raw[7]);
        uint4 b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const uint4 *>(bptr + (4 * hh + j) * 64);
        const float4 sg0 = *reinterpret_cast<const float4 *>(cg + hh * 32);
        const float4 sg1 = *reinterpret_cast<const float4 *>(cg + hh * 32 + 16);
        const float4 sh0 = *reinterpret_cast<const float4 *>(ch + hh * 32);
        const float4 sh1 = *reinterpret_cast<const float4 *>(ch + hh * 32 + 16);
        float c[4][4];
        uint32_t a[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // a[j][0..3]: row g bytes 0..3 of block j; a[j][4..7]: row g+8
            e2m1x8_to_h2x4(raw[j * 2], a[j][0], a[j][1], a[j][2], a[j][3]);
            e2m1x8_to_h2x4(raw[j * 2 + 1], a[j][4], a[j][5], a[j][6], a[j][7]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            mma_f16(c[j], a[j][0], a[j][4], a[j][1], a[j][5], b[j].x, b[j].y, 0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            mma_f16(c[j], a[j][2], a[j][6], a[j][3], a[j][7], b[j].z, b[j].w, c[j][0], c[j][1], c[j][2],
                    c[j][3]);
        p_lo = __ffma2_rn(make_float2(c[0][0], c[0][1]), make_float2(sg0.x, sg0.y), p_lo);
        p_hi = __ffma2_rn(make_float2(c[0][2], c[0][3]), make_float2(sh0.x, sh0.y), p_hi);
        p_lo = __ffma2_rn(make_float2(c[1][0], c[1][1]), make_float2(sg0.z, sg0.w), p_lo);
        p_hi = __ffma2_rn(make_float2(c[1][2], c[1][3]), make_float2(sh0.z, sh0.w), p_hi);
        p_lo = __ffma2_rn(make_float2(c[2][0], c[2][1]), make_float2(sg1.x, sg1.y), p_lo);
        p_hi = __ffma2_rn(make_float2(c[2][2], c[2][3]), make_float2(sh1.x, sh1.y), p_hi);
        p_lo = __ffma2_rn(make_float2(c[3][0], c[3][1]), make_float2(sg1.z, sg1.w), p_lo);
        p_hi = __ffma2_rn(make_float2(c[3][2], c[3][3]), make_float2(sh1.z, sh1.w), p_hi);
    }
    acc[0] += (double)p_lo.x;
    acc[1] += (double)p_lo.y;
    acc[2] += (double)p_hi.x;
    acc[3] += (double)p_hi.y;
}

// The tiles of one CTA: tile ids first, first + stride, ..., n of them, each `spt` stages long.
// Short lists are cut into equal runs of stages for the warps (a tile then has up to kMaxSeg
// partial sums); long lists are dealt out tile by tile.
struct WorkList {
    uint32_t first, stride, n, spt;
    bool split;
    uint32_t warps_used, total;  // runs (split mode) or warps, and flat length
};

__device__ __forceinline__ WorkList make_work(uint32_t first, uint32_t stride, uint32_t total_tiles,
                                              uint32_t spt, uint32_t n_warps) {
    WorkList wl;
    wl.first = first;
    wl.stride = stride;
    wl.spt = spt;
    wl.n = first < total_tiles ? (total_tiles - first + stride - 1) / stride : 0u;
    wl.split = wl.n <= (uint32_t)kSplitTiles;
    wl.total = wl.n * spt;
    const uint32_t min_run = (spt + 1u) >> 1;
    wl.warps_used = wl.split ? max(1u, min(n_warps, wl.total / max(1u, min_run))) : n_warps;
    return wl;
}

// Warp that owns flat stage f0 in split mode.
__device__ __forceinline__ uint32_t run_of(const WorkList &wl, uint32_t f0) {
    return (uint32_t)((((uint64_t)f0 + 1) * wl.warps_used + wl.total - 1) / wl.total) - 1u;
}
__device__ __forceinline__ uint32_t run_begin(const WorkList &wl, uint32_t w) {
    return (uint32_t)(((uint64_t)w * wl.total) / wl.warps_used);
}
// True when one run covers the whole tile, so its result was stored directly.
__device__ __forceinline__ bool tile_is_whole(const WorkList &wl, uint32_t tl) {
    const uint32_t f0 = tl * wl.spt, w = run_of(wl, f0);
    return run_begin(wl, w) <= f0 && run_begin(wl, w + 1) >= f0 + wl.spt;
}

// Runs this warp's share of the work list as one flat cp.async pipeline.  `setup(tile, tr)`
// fills the row pointers of a global tile id; finished sums of rows g (lo) and g+8 (hi) are
// handed, on the lanes with t == 0, to `emit(tile_local, seg, whole, lo, hi)`.
// `before_compute()` runs on every warp of the CTA after the first copies are in flight and
// before any activation limb is read (the down phase builds its limbs there).
template <class Setup, class Emit, class Before>
__device__ __forceinline__ void run_tiles(const WorkList &wl, uint32_t warp, uint32_t k, const uint8_t *limbs,
                                          uint8_t *ring, uint32_t lane, Setup setup, Emit emit,
                                          Before before_compute) {
    const uint32_t spt = wl.spt;
    uint32_t count = 0, tl0 = 0, st0 = 0, tl_step = 1;  // stages to run, first local tile and stage, tile step
    if (wl.split) {
        if (warp < wl.warps_used) {
            const uint32_t f_lo = run_begin(wl, warp), f_hi = run_begin(wl, warp + 1);
            count = f_hi - f_lo;
            tl0 = f_lo / spt;
            st0 = f_lo - tl0 * spt;
        }
    } else if (warp < wl.n) {
        count = ((wl.n - warp + wl.warps_used - 1) / wl.warps_used) * spt;
        tl0 = warp;
        tl_step = wl.warps_used;
    }
    const uint32_t row_bytes = k >> 1, scale_bytes = k >> 5;
    const uint32_t pitch = limb_pitch_bytes(k);
    const uint32_t ring_w = smem_u32(ring);
    const uint32_t ring_s = ring_w + kStages * kStageBytes;
    const uint8_t *ring_s_gen = ring + kStages * kStageBytes;
    uint8_t *conv = ring + kStages * (kStageBytes + kScaleRaw);
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint8_t *bbase = limbs + (g < 3 ? g : 3u) * pitch + (size_t)(t * 8u) * 2u;

    // producer side: next stage to copy
    LaneCopy lc;
    lane_copy_init(lc, lane);
    uint32_t i_left = count, i_tl = tl0, i_st = st0, i_slot = 0;
    bool i_new_tile = true;
    auto issue = [&]() {
        if (i_left) {
            if (i_new_tile) {
                TileRows tr;
                setup(wl.first + i_tl * wl.stride, tr);
                lane_copy_tile(lc, tr, row_bytes, scale_bytes, lane);
                i_new_tile = false;
            }
            issue_stage(lc, i_st, ring_w + i_slot * kStageBytes, ring_s + i_slot * kScaleRaw, lane);
            --i_left;
            i_slot = (i_slot + 1 == kStages) ? 0 : i_slot + 1;
            if (++i_st == spt) {
                i_st = 0;
                i_tl += tl_step;
                i_new_tile = true;
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) issue();
    before_compute();
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    uint32_t slot = 0, tl = tl0, st = st0;
    for (uint32_t left = count; left; --left) {
        cp_async_wait<kStages - 2>();
        __syncwarp();
        convert_scales(ring_s_gen + slot * kScaleRaw, conv, lane);
        __syncwarp();
        compute_stage(ring_w + slot * kStageBytes, conv, bbase + (size_t)(st << 8) * 2u, lane, acc);
        __syncwarp();
        issue();
        slot = (slot + 1 == kStages) ? 0 : slot + 1;
        ++st;
        if (st == spt || left == 1) {
            // columns: t == 0 holds limbs 0 and 1, t == 1 holds limb 2 (and an unused column)
            const double l2_lo = __shfl_down_sync(0xffffffffu, acc[0], 1);
            const double l2_hi = __shfl_down_sync(0xffffffffu, acc[2], 1);
            const double v_lo = acc[0] + acc[1] * (1.0 / 2048.0) + l2_lo * (1.0 / 4194304.0);
            const double v_hi = acc[2] + acc[3] * (1.0 / 2048.0) + l2_hi * (1.0 / 4194304.0);
            uint32_t seg = 0;
            bool whole = true;
            if (wl.split) {
                seg = warp - run_of(wl, tl * spt);
                whole = tile_is_whole(wl, tl);
            }
            if (t == 0) emit(tl, seg, whole, v_lo, v_hi);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.0;
            if (st == spt) {
                st = 0;
                tl += tl_step;
            }
        }
    }
    cp_async_wait<0>();
}

__device__ __forceinline__ uint8_t *smem_limbs(uint8_t *smem, uint32_t n_warps) {
    return smem + n_warps * kWarpSmem + kPartBytes;
}
__device__ __forceinline__ double *smem_parts(uint8_t *smem, uint32_t n_warps) {
    return reinterpret_cast<double *>(smem + n_warps * kWarpSmem);
}

}  // namespace

// Up phase.  grid = n_tokens * ctas_per_token, block = 32 * warps, dynamic smem =
// warps * kWarpSmem + kPartBytes + 4 * limb pitch.  Tiles of 8 row pairs of the token's jobs,
// which must all be MXFP4 pages (the launcher routes layers with an FP8 page to the F32 kernels).
__global__ void __launch_bounds__(512, 1)
k_expert_up_mma(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
                const float *__restrict__ x, float *__restrict__ h, uint32_t hidden, uint32_t inter,
                uint32_t ctas_per_token) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[kMaxWarps];
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const uint32_t token = blockIdx.x / ctas_per_token;
    const uint32_t cta_in_token = blockIdx.x - token * ctas_per_token;
    uint8_t *limbs = smem_limbs(smem, n_warps);
    double *parts = smem_parts(smem, n_warps);
    for (uint32_t i = threadIdx.x; i < kPartBytes / 8; i += blockDim.x) parts[i] = 0.0;
    const int x_exp = build_limbs(x + (size_t)token * hidden, hidden, limbs, red);
    __syncthreads();
    // When launched as a programmatic dependent of the router, everything above overlapped with
    // it; the job table is read only after the router has completed.  The down kernel may queue
    // behind this one from here on (its CTAs start as ours retire and prefetch their weights).
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();

    const uint32_t job0 = tab.token_job_begin[token];
    const uint32_t n_jobs = tab.token_job_begin[token + 1] - job0;
    const uint32_t tiles_per_job = inter >> 3;
    const WorkList wl = make_work(cta_in_token, ctas_per_token, n_jobs * tiles_per_job, hidden >> 8, n_warps);
    const double sc = ldexp(1.0, x_exp);
    const uint32_t g = lane >> 2;

    auto setup = [&](uint32_t tile, TileRows &tr) {
        const uint32_t jid = tab.token_jobs[job0 + tile / tiles_per_job];
        const PageView pv = page_view(tab.jobs[jid].page, S14_PAGE_MXFP4, hidden, inter);
        tr.w0 = pv.w1;
        tr.w1 = pv.w3;
        tr.s0 = pv.s1;
        tr.s1 = pv.s3;
        tr.r0 = tr.r1 = (tile % tiles_per_job) << 3;
    };
    auto store = [&](uint32_t tile, uint32_t row, double gate, double up) {
        const uint32_t jid = tab.token_jobs[job0 + tile / tiles_per_job];
        h[(size_t)jid * inter + ((tile % tiles_per_job) << 3) + row] =
            swiglu_limit_f32((float)(gate * sc), (float)(up * sc));
    };
    auto emit = [&](uint32_t tl, uint32_t seg, bool whole, double lo, double hi) {
        if (whole) {
            store(wl.first + tl * wl.stride, g, lo, hi);
        } else {
            double *p = parts + ((size_t)tl * kMaxSeg + seg) * 16;
            p[g] = lo;
            p[g + 8] = hi;
        }
    };
    run_tiles(wl, warp, hidden, limbs, smem + warp * kWarpSmem, lane, setup, emit, [] {});
    if (!wl.split) return;
    __syncthreads();
    // tiles whose stages were shared between warps: add the partial sums in run order
    for (uint32_t i = threadIdx.x; i < wl.n * 8u; i += blockDim.x) {
        const uint32_t tl = i >> 3, row = i & 7u;
        if (tile_is_whole(wl, tl)) continue;
        const double *p = parts + (size_t)tl * kMaxSeg * 16;
        double gate = 0.0, up = 0.0;
#pragma unroll
        for (int s = 0; s < kMaxSeg; ++s) {
            gate += p[s * 16 + row];
            up += p[s * 16 + 8 + row];
        }
        store(wl.first + tl * wl.stride, row, gate, up);
    }
}

// Down phase and mix.  grid = n_jobs * ctas_per_job; a CTA keeps the limbs of its job's hidden
// vector and owns the row tiles cta_in_job, cta_in_job + ctas_per_job, ... of that job.
__global__ void __launch_bounds__(512, 1)
k_expert_down_mma(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
                  const float *__restrict__ h, float *__restrict__ d, float *__restrict__ y,
                  unsigned int *__restrict__ counters, uint32_t hidden, uint32_t inter,
                  uint32_t ctas_per_job) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[kMaxWarps];
    __shared__ bool is_last;
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const uint32_t jid = blockIdx.x / ctas_per_job;
    const uint32_t cta_in_job = blockIdx.x - jid * ctas_per_job;
    if (jid >= tab.n_jobs) return;
    const Job jb = tab.jobs[jid];
    if (jb.kind != S14_PAGE_MXFP4) return;
    uint8_t *limbs = smem_limbs(smem, n_warps);
    double *parts = smem_parts(smem, n_warps);
    for (uint32_t i = threadIdx.x; i < kPartBytes / 8; i += blockDim.x) parts[i] = 0.0;
    const PageView pv = page_view(jb.page, S14_PAGE_MXFP4, hidden, inter);
    const WorkList wl = make_work(cta_in_job, ctas_per_job, hidden >> 4, inter >> 8, n_warps);
    double sc = 1.0;
    // The weight copies start before the up phase has finished (programmatic dependent launch);
    // the hidden vector is read, and split into limbs, only after it has.
    auto before = [&] {
        cudaGridDependencySynchronize();
        const int x_exp = build_limbs(h + (size_t)jid * inter, inter, limbs, red);
        __syncthreads();
        sc = ldexp(1.0, x_exp);
    };
    const uint32_t g = lane >> 2;
    float *out = d + (size_t)jb.out_index * hidden;
    auto setup = [&](uint32_t tile, TileRows &tr) {
        tr.w0 = tr.w1 = pv.w2;
        tr.s0 = tr.s1 = pv.s2;
        tr.r0 = tile << 4;
        tr.r1 = (tile << 4) + 8u;
    };
    auto emit = [&](uint32_t tl, uint32_t seg, bool whole, double lo, double hi) {
        if (whole) {
            const uint32_t tile = wl.first + tl * wl.stride;
            out[(tile << 4) + g] = (float)(lo * sc);
            out[(tile << 4) + 8u + g] = (float)(hi * sc);
        } else {
            double *p = parts + ((size_t)tl * kMaxSeg + seg) * 16;
            p[g] = lo;
            p[g + 8] = hi;
        }
    };
    run_tiles(wl, warp, inter, limbs, smem + warp * kWarpSmem, lane, setup, emit, before);
    if (wl.split) {
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < wl.n * 16u; i += blockDim.x) {
            const uint32_t tl = i >> 4, row = i & 15u;
            if (tile_is_whole(wl, tl)) continue;
            const double *p = parts + (size_t)tl * kMaxSeg * 16;
            double v = 0.0;
#pragma unroll
            for (int s = 0; s < kMaxSeg; ++s) v += p[s * 16 + row];
            out[((wl.first + tl * wl.stride) << 4) + row] = (float)(v * sc);
        }
    }
    if (!y) return;  // the caller mixes (expert-parallel combine)
    // Ordered mix (examples/s14_vulkan_numeric.rs:936-946) by the last CTA of this token to finish
    // this slice of rows: acc = 0; acc += w * d for the routed jobs in route order; acc += d_shared.
    __threadfence();
    __syncthreads();
    const uint32_t j0 = tab.token_job_begin[jb.token], j1 = tab.token_job_begin[jb.token + 1];
    unsigned int *counter = counters + 1u + jb.token * 160u + cta_in_job;
    if (threadIdx.x == 0) is_last = atomicAdd(counter, 1u) == (j1 - j0) - 1u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (uint32_t i = threadIdx.x; i < wl.n * 16u; i += blockDim.x) {
        const uint32_t n = ((wl.first + (i >> 4) * wl.stride) << 4) + (i & 15u);
        float acc = 0.0f;
        for (uint32_t j = j0; j < j1; ++j) {
            const uint32_t other = tab.token_jobs[j];
            const float v = __ldcg(d + (size_t)tab.jobs[other].out_index * hidden + n);
            acc = tab.jobs[other].is_shared ? __fadd_rn(acc, v)
                                            : __fadd_rn(acc, __fmul_rn(tab.jobs[other].weight, v));
        }
        y[(size_t)jb.token * hidden + n] = acc;
    }
    if (threadIdx.x == 0) *counter = 0u;  // ready for the next launch
}

static size_t mma_smem_bytes(uint32_t warps, uint32_t k) {
    return (size_t)warps * kWarpSmem + kPartBytes + 4u * (k * 2u + 64u);
}

static void configure_once() {
    static bool configured = false;
    if (configured) return;
    const int most = (int)mma_smem_bytes(kMaxWarps, 4096);
    cudaFuncSetAttribute(k_expert_up_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    cudaFuncSetAttribute(k_expert_down_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    configured = true;
}

template <class Kernel, class... Args>
static cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

cudaError_t launch_up_mma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                          const float *x, float *h, uint32_t hidden, uint32_t inter, uint32_t n_tokens,
                          bool after_router) {
    configure_once();
    const uint32_t ctas_per_token = max(1u, (uint32_t)sm_count / n_tokens);
    return launch_pdl(k_expert_up_mma, dim3(n_tokens * ctas_per_token), dim3(kMaxWarps * 32),
                      mma_smem_bytes(kMaxWarps, hidden), st, after_router, dev, param, x, h, hidden, inter,
                      ctas_per_token);
}

cudaError_t launch_down_mma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                            const float *h, float *d, float *y, unsigned int *counters, uint32_t hidden,
                            uint32_t inter, uint32_t n_jobs) {
    configure_once();
    const uint32_t ctas_per_job = max(1u, (uint32_t)sm_count / n_jobs);
    return launch_pdl(k_expert_down_mma, dim3(n_jobs * ctas_per_job), dim3(kMaxWarps * 32),
                      mma_smem_bytes(kMaxWarps, inter), st, true, dev, param, h, d, y, counters, hidden, inter,
                      ctas_per_job);
}

}  // namespace s14
