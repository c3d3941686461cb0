// Pairwise-order up and down phases of a one-token MoE layer on the fifth-generation tensor
// cores: tcgen05.mma kind::mxf4.block_scale consumes the page bytes as they are (packed E2M1,
// one UE8M0 scale per 32 elements along K), so no thread decodes or scales a weight.
//
// The matvec as a block-scaled MMA.  A = 128 weight rows x 64 K-elements per instruction, staged
// in shared memory K-major with the 128-byte swizzle; its scales go to tensor memory with
// tcgen05.cp.  B = the activation vector, written once per CTA as eight balanced base-8 digit
// rows: within a scale block of 32 elements with largest magnitude < 2^E (E >= -100), every element is
// q * 2^(E-23) with |q| <= 2^23 (rounded to nearest when it has more bits below the block's top
// bit), q = sum_j d_j 8^j with d_j in [-4, 4] -- all of them E2M1 values -- and digit row j carries
// the UE8M0 scale 2^(E-23+3j).  Accumulator column j therefore holds the exact digit-j share of
// the dot product in F32; the eight columns are added in F64 and rounded once.  Measured against
// a double-precision sum on B200: relative RMSE 1.5e-7, all of it from the 23-bit quantisation of
// elements far below their block's largest one.  Columns 8-15 of the 16-column MMA are zero rows.
//
// Work split.  A unit is one 128-row x 256-K stage (16 KB of codes + 1 KB of scales).  The units
// of the launch, ordered job, row tile, K (up phase: w1 and w3 alternate, two accumulators),
// are cut into gridDim.x equal runs, one CTA per SM.  A run that ends inside a tile leaves F64
// partial sums in global scratch; whichever CTA arrives last at the tile's counter adds the
// partials in K order and finishes the rows (no CTA waits for another).  Roles inside a CTA:
// four producer warps (cp.async into an 8-stage ring, completion through mbarriers), one MMA
// thread, four epilogue warps (tcgen05.ld, F64 sums, SwiGLU or the ordered mix).  Every mbarrier
// wait is bounded; a wait that runs out raises the CTA's abort flag, the status word is set and
// the CTA drains its copies, frees its tensor memory and returns.
#include "s14_device.cuh"

namespace s14 {

namespace {

constexpr uint32_t kRing = 8;                  // stages, accumulators and scale slots in flight per CTA
constexpr uint32_t kStageA = 128 * 128;        // 128 rows x 128 B of codes
constexpr uint32_t kStageSf = 2 * 512;         // two scale atoms (128 rows x 4 blocks each)
constexpr uint32_t kEpiGroup = 128;            // two epilogue groups of four warps (even / odd units of a tile)
constexpr uint32_t kMmaWarp0 = 8;              // warps 8 and 9: one issuing thread each (even / odd units of the run)
constexpr uint32_t kProdWarp0 = 10;            // warps 10..13 copy
constexpr uint32_t kProdThreads = 128;
constexpr uint32_t kThreads = 512;               // warps 14 and 15 only help with the digits
constexpr uint32_t kTmemCols = 512;            // [0,128): 8 accumulators x 16; [128,192): weight scales; [192,512): digit scales
constexpr uint32_t kSfaCol0 = 128, kSfbCol0 = 192;
constexpr uint32_t kDigitSlots = 2;            // activation vectors a CTA's run can need
constexpr uint32_t kMaxBlocks = 160;           // scale blocks per activation vector (K <= 5120)
constexpr uint32_t kMaxK = (kTmemCols - kSfbCol0) / kDigitSlots / 4 * 128;  // digit scales of both slots fit tensor memory
constexpr uint32_t kSpin = 1u << 17;           // tries before a wait gives up
constexpr uint32_t kMaxTiles = 2048;           // tile counters per phase
constexpr uint32_t kUpCounter0 = 1, kDownCounter0 = 1 + kMaxTiles, kMixCounter0 = 1 + 2 * kMaxTiles;
constexpr uint32_t kHReadyCounter0 = kMixCounter0 + kMaxTokens * 64;  // finished up tiles per job
constexpr uint32_t kExitCounter = kHReadyCounter0 + kMaxJobs;          // CTAs that have left the kernel
static_assert(kExitCounter < 8192, "a context allocates 8192 arrival counters");
constexpr uint32_t kSpinGlobal = 1u << 20;     // polls (100 ns apart) of another CTA's progress before giving up
constexpr uint32_t kMaxRowTiles = 64;             // mix counters: [token][row tile]

// Bar indices in the static barrier array: stage filled, unit multiplied, accumulator read,
// digit scales in tensor memory, both issuing threads finished.
constexpr uint32_t kBarFull = 0, kBarDone = kRing, kBarAccFree = 2 * kRing, kBarDigitsUp = 3 * kRing,
                   kBarDigitsDown = 3 * kRing + 1, kBarFin = 3 * kRing + 2, kBars = 3 * kRing + 3;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrives once the calling thread's earlier cp.async copies have landed.
__device__ __forceinline__ void mbar_arrive_after_copies(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
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
    for (uint32_t i = 0; i < kSpin; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// Named barriers of the epilogue: 1 = the 128 threads of group A, 2 = both groups.
__device__ __forceinline__ void group_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
__device__ __forceinline__ bool epi_bar_and(bool v) {
    uint32_t r;
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "setp.ne.b32 q, %1, 0;\n"
        "bar.red.and.pred p, 2, 256, q;\n"
        "selp.b32 %0, 1, 0, p;\n}"
        : "=r"(r)
        : "r"((uint32_t)v)
        : "memory");
    return r != 0;
}

// Position of a unit: tile t (job j, row tile rt) and unit w of the tile.
struct UnitCursor {
    uint32_t t, w, j, rt;
};
__device__ __forceinline__ UnitCursor cursor_at(uint32_t u, uint32_t upt, uint32_t tpj) {
    UnitCursor c;
    c.t = u / upt;
    c.w = u - c.t * upt;
    c.j = c.t / tpj;
    c.rt = c.t - c.j * tpj;
    return c;
}
__device__ __forceinline__ void cursor_advance(UnitCursor &c, uint32_t step, uint32_t upt, uint32_t tpj) {
    c.w += step;
    while (c.w >= upt) {
        c.w -= upt;
        ++c.t;
        if (++c.rt == tpj) {
            c.rt = 0;
            ++c.j;
        }
    }
}

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
__device__ __forceinline__ void tmem_ld8(uint32_t addr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

#ifdef S14_UMMA_TRACE
__device__ unsigned long long g_umma_trace[2][160][12];
__device__ __forceinline__ void trace_mark(bool up, uint32_t k) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_umma_trace[up ? 1 : 0][blockIdx.x][k] = t;
}
#define TRACE(k) trace_mark(true, k)
__device__ long long g_umma_cyc[2][160][8];
#define CYC_DECL(n) long long cyc_[n] = {}; long long cyc_t_ = clock64()
#define CYC_LAP(k) do { const long long now_ = clock64(); cyc_[k] += now_ - cyc_t_; cyc_t_ = now_; } while (0)
#define CYC_STORE(base, n) do { for (int q_ = 0; q_ < (n); ++q_) g_umma_cyc[1][blockIdx.x][(base) + q_] = cyc_[q_]; } while (0)
#else
#define TRACE(k) ((void)0)
#define CYC_DECL(n) ((void)0)
#define CYC_LAP(k) ((void)0)
#define CYC_STORE(base, n) ((void)0)
#endif

// Instruction descriptor: A and B E2M1 (format 1), both K-major, N = 16, UE8M0 scales, M = 128.
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);

// Writes the eight digit rows of v[0..K) and their scale atoms.  A thread owns eight consecutive
// elements, i.e. one 32-bit word of every digit row; the four lanes of a scale block agree on its
// exponent E (largest magnitude < 2^E, clamped to [-100, 128]).  With the bias 4 * (8^8 - 1) / 7
// added, the balanced digits of q are the plain base-8 digits minus 4, so no carry runs through
// them.  Rows 8-15 of the tile are zeroed by the caller; the blocks' exponents go to sE, from which
// store_digit_scales writes the digit rows' scale codes into tensor memory.
__device__ void build_digits(const float *v0, const float *v1, uint32_t n_vec, uint32_t K,
                             uint8_t *sB, uint32_t b_stride, uint8_t *sE, uint32_t tid,
                             uint32_t n_threads) {
    const uint32_t per_vec = K >> 3;
    for (uint32_t item = tid; item < n_vec * per_vec; item += n_threads) {
        const uint32_t slot = item >= per_vec ? 1u : 0u, g = item - slot * per_vec;
        const float *v = slot ? v1 : v0;
        // read through L2: a hidden vector was written by other CTAs of this launch
        const float4 p0 = __ldcg(reinterpret_cast<const float4 *>(v) + 2u * g);
        const float4 p1 = __ldcg(reinterpret_cast<const float4 *>(v) + 2u * g + 1u);
        const float xs[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        float bm = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) bm = fmaxf(bm, fabsf(xs[i]));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
        bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));
        int E = -100;
        if (bm > 0.0f) E = min(max((int)((__float_as_uint(bm) >> 23) & 0xFFu) - 126, -100), 127);
        const float up = __uint_as_float((uint32_t)(150 - E) << 23);  // 2^(23-E)
        uint32_t words[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t qb = (uint32_t)(__float2int_rn(xs[i] * up) + 0x924924);  // in [0, 8^8 + 8^7) for finite input
#pragma unroll
            for (int j = 0; j < 7; ++j)  // E2M1 codes of -4..3 by digit value 0..7
                words[j] |= ((0x5420ACDEu >> (((qb >> (3 * j)) & 7u) << 2)) & 0xFu) << (4 * i);
            const uint32_t top = qb >> 21;  // 0..8 -> -4..4
            words[7] |= (top > 7u ? 6u : ((0x5420ACDEu >> (top << 2)) & 0xFu)) << (4 * i);
        }
        const uint32_t kb = g >> 2;
        uint8_t *chunk = sB + slot * b_stride + (kb >> 3) * 2048u + (g & 3u) * 4u;
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j)
            *reinterpret_cast<uint32_t *>(chunk + j * 128u + (((kb & 7u) ^ j) << 4)) = words[j];
        if ((g & 3u) == 0u) sE[slot * kMaxBlocks + kb] = (uint8_t)(E + 100);  // the block's exponent, biased
    }
}

// The scale codes of the digit rows, written to tensor memory by the eight epilogue warps (each
// lane quadrant takes every atom; warps 0-3 the even groups of four atoms, warps 4-7 the odd ones).
// Column 4a of lane l holds the codes of N-row l for scale blocks 4a..4a+3: digit row l < 8 of a
// block with exponent E has the code 127 + E - 23 + 3l; rows 8-15 are zero rows, columns 4a+1..4a+3
// belong to N-rows 32 and up, which a 16-column MMA does not read.
__device__ __forceinline__ void store_digit_scales(uint32_t tmem_sfb, const uint8_t *sE, uint32_t n_slots, uint32_t K,
                                                   uint32_t sfb_cols, uint32_t warp, uint32_t lane) {
    const uint32_t groups = K >> 9;  // groups of four atoms (512 K-elements, 16 blocks)
    const uint32_t bias = 0x01010101u * (4u + 3u * (lane & 7u));
    const uint32_t quad = tmem_sfb + (((warp & 3u) * 32u) << 16);
    for (uint32_t q = warp >> 2; q < n_slots * groups; q += 2u) {
        const uint32_t b = q / groups, g = q - b * groups;
        const uint4 e = *reinterpret_cast<const uint4 *>(sE + b * kMaxBlocks + g * 16u);
        const uint32_t one = 0x7F7F7F7Fu;
        const uint32_t w0 = lane < 8u ? e.x + bias : one, w1 = lane < 8u ? e.y + bias : one;
        const uint32_t w2 = lane < 8u ? e.z + bias : one, w3 = lane < 8u ? e.w + bias : one;
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%5,%5,%5,%2,%5,%5,%5,%3,%5,%5,%5,%4,%5,%5,%5};"
            ::"r"(quad + b * sfb_cols + g * 16u), "r"(w0), "r"(w1), "r"(w2), "r"(w3), "r"(one)
            : "memory");
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// s + e = a + b exactly (Knuth); no operation may be contracted or reordered.
__device__ __forceinline__ void two_sum(float a, float b, float &s, float &e) {
    s = __fadd_rn(a, b);
    const float bb = __fsub_rn(s, a);
    e = __fadd_rn(__fsub_rn(a, __fsub_rn(s, bb)), __fsub_rn(b, bb));
}

// SwiGLU of the pairwise path: the same expression as swiglu_limit_f32 with the F32 library
// exponential (FP64 is scarce on this GPU; the bit-exact order keeps the correctly rounded one).
__device__ __forceinline__ float swiglu_limit_fast(float gate, float up) {
    const float g = fminf(gate, 10.0f);
    const float u = fminf(fmaxf(up, -10.0f), 10.0f);
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

// Shape of one phase: the up phase multiplies [inter, hidden] twice (w1, w3), the down phase
// [hidden, inter] once (w2).
struct PhaseShape {
    uint32_t K, rows, mats, kchunks, upt, tpj;  // upt: units per tile, tpj: tiles per job
    uint32_t b_stride, sfb_cols;                // digit tile (shared memory), its scale columns (tensor memory)
};
__device__ __forceinline__ PhaseShape phase_shape(bool up, uint32_t hidden, uint32_t inter) {
    PhaseShape ps;
    ps.K = up ? hidden : inter;
    ps.rows = up ? inter : hidden;
    ps.mats = up ? 2u : 1u;
    ps.kchunks = ps.K >> 8;
    ps.upt = ps.mats * ps.kchunks;
    ps.tpj = ps.rows >> 7;
    ps.b_stride = ps.kchunks * 2048u;
    ps.sfb_cols = (ps.K >> 7) * 4u;
    return ps;
}
// A CTA's run of a phase: units [u0, u1) of `total`, cut into G equal runs.
struct Run {
    uint64_t total;
    uint32_t G, u0, u1, n, job_first, job_last;
};
__device__ __forceinline__ Run make_run(const PhaseShape &ps, uint32_t n_jobs, uint32_t grid, uint32_t cta) {
    Run r;
    r.total = (uint64_t)n_jobs * ps.tpj * ps.upt;
    // every working CTA gets at least one unit, so each tile's contributors are consecutive CTAs
    r.G = (uint32_t)min((uint64_t)grid, r.total);
    const bool working = cta < r.G;
    r.u0 = working ? (uint32_t)(r.total * cta / r.G) : 0u;
    r.u1 = working ? (uint32_t)(r.total * (cta + 1u) / r.G) : 0u;
    r.n = r.u1 - r.u0;
    // a run is at most one job long (the launcher requires n_jobs <= gridDim.x): two jobs at most
    r.job_first = r.n ? (r.u0 / ps.upt) / ps.tpj : 0u;
    r.job_last = r.n ? ((r.u1 - 1u) / ps.upt) / ps.tpj : 0u;
    return r;
}

__device__ __forceinline__ uint32_t ld_acquire(const unsigned int *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One launch runs the whole layer.  Every CTA streams its run of the up phase and then its run of
// the down phase through one ring; the copies of the down phase do not wait for the hidden
// vectors, only its MMAs do (the vectors of a job are complete when the job's counter says that
// all its up tiles are finished, whichever CTAs finished them).
__global__ void __launch_bounds__(kThreads, 1)
k_moe_layer_umma(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
                 const float *__restrict__ x, float *h, float *d, float *__restrict__ y,
                 double *__restrict__ partials, unsigned int *__restrict__ counters, uint32_t *__restrict__ status,
                 uint32_t hidden, uint32_t inter, uint32_t b_bytes) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[kBars];
    __shared__ double xchg[kEpiGroup];  // group B's sums of a tile, handed to group A
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ uint32_t epi_info[3];
    __shared__ __align__(16) uint8_t sE[kDigitSlots * kMaxBlocks];  // block exponents of the digit tiles

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const bool is_producer = warp >= kProdWarp0 && warp < kProdWarp0 + kProdThreads / 32u;
    if (tid == 0) TRACE(0);
    const PhaseShape PU = phase_shape(true, hidden, inter), PD = phase_shape(false, hidden, inter);
    uint8_t *const sA = smem;
    uint8_t *const sSFA = sA + kRing * kStageA;
    uint8_t *const sB = sSFA + kRing * kStageSf;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](uint32_t i) { return bar0 + i * 8u; };

    // rows 8-15 of every digit tile stay zero
    for (uint32_t i = tid; i < b_bytes >> 4; i += kThreads) reinterpret_cast<uint4 *>(sB)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
        for (uint32_t s = 0; s < kRing; ++s) {
            mbar_init(bar(kBarFull + s), kProdThreads);
            mbar_init(bar(kBarDone + s), 1);
            mbar_init(bar(kBarAccFree + s), kEpiGroup);
        }
        mbar_init(bar(kBarDigitsUp), 2u * kEpiGroup);
        mbar_init(bar(kBarDigitsDown), 2u * kEpiGroup);
        mbar_init(bar(kBarFin), 2);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_slot;
    if (tid == 0) TRACE(1);

    if (dev_table) {
        // One token routed on the device: the token does not depend on the router, so its digits
        // are built while the router runs; the job table is read only afterwards.
        build_digits(x, x, 1, PU.K, sB, PU.b_stride, sE, tid, kThreads);
    }
    cudaGridDependencySynchronize();
    const JobTable &tab = table_of(dev_table, param_table);
    const uint32_t n_jobs = tab.n_jobs, cta = blockIdx.x;
    const Run RU = make_run(PU, n_jobs, gridDim.x, cta), RD = make_run(PD, n_jobs, gridDim.x, cta);
    const uint32_t tok0 = (!dev_table && RU.n) ? tab.jobs[RU.job_first].token : 0u;
    const uint32_t tok1 = (!dev_table && RU.n) ? tab.jobs[RU.job_last].token : 0u;
    const uint32_t up_slots = tok1 != tok0 ? 2u : 1u, down_slots = RD.job_last - RD.job_first + 1u;
    // digit slot of job j: up phase by token, down phase by job
    auto slot_up = [&](uint32_t j) { return tab.jobs[j].token == tok0 ? 0u : 1u; };
    if (!dev_table && RU.n)
        build_digits(x + (size_t)tok0 * hidden, x + (size_t)tok1 * hidden, up_slots, PU.K, sB, PU.b_stride, sE, tid,
                     kThreads);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) TRACE(2);

    unsigned int *const h_ready = counters + kHReadyCounter0;

    if (is_producer) {
        // ---- copies: the run of the up phase, then the run of the down phase, through one ring ----
        const uint32_t pt = tid - kProdWarp0 * 32u, r8 = pt >> 3, cc = pt & 7u;
        const uint32_t dst0 = smem_u32(sA) + r8 * 128u + ((cc ^ (r8 & 7u)) << 4);
        uint32_t i = 0;
        bool ok = true;
        for (uint32_t ph = 0; ph < 2 && ok; ++ph) {
            const PhaseShape &ps = ph ? PD : PU;
            const Run &run = ph ? RD : RU;
            UnitCursor c = cursor_at(run.u0, ps.upt, ps.tpj);
            for (uint32_t l = 0; l < run.n; ++l, ++i) {
                const uint32_t s = i % kRing;
                if (i >= kRing && !mbar_wait(bar(kBarDone + s), ((i / kRing) - 1u) & 1u, &abort_flag)) {
                    ok = false;
                    break;
                }
                const uint32_t ks = ph ? c.w : (c.w >> 1), mat = ph ? 0u : (c.w & 1u);
                const PageView pv = page_view(tab.jobs[c.j].page, S14_PAGE_MXFP4, hidden, inter);
                const uint8_t *wp = ph ? pv.w2 : (mat ? pv.w3 : pv.w1);
                const uint8_t *sp = ph ? pv.s2 : (mat ? pv.s3 : pv.s1);
                const uint8_t *src = wp + (size_t)(c.rt * 128u + r8) * (ps.K >> 1) + ks * 128u + cc * 16u;
                const uint32_t dst = dst0 + s * kStageA;
#pragma unroll
                for (uint32_t i8 = 0; i8 < 8; ++i8) cp_async16(dst + i8 * 2048u, src + (size_t)i8 * 16u * (ps.K >> 1));
                // the unit's two scale atoms are 1 KB of consecutive page bytes, already in tensor-memory order
                if (pt < kStageSf / 16u)
                    cp_async16(smem_u32(sSFA + s * kStageSf) + pt * 16u,
                               sp + scale_word_offset(c.rt * 128u, ks * 2u, ps.K) + pt * 16u);
                mbar_arrive_after_copies(bar(kBarFull + s));
                cursor_advance(c, 1, ps.upt, ps.tpj);
            }
        }
        if (tid == kProdWarp0 * 32u) TRACE(8);
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (tid == kProdWarp0 * 32u) TRACE(9);
    } else if (warp == kMmaWarp0 || warp == kMmaWarp0 + 1u) {
        if (lane == 0 && (RU.n || RD.n)) {
            // ---- MMA issue: two threads take the even and the odd ring indices.  One accumulator per
            // unit: a tile's result is the sum of its units' F32 sums, whichever CTAs computed them. ----
            const uint32_t m = warp - kMmaWarp0;
            const uint64_t a_desc0 = smem_desc(smem_u32(sA), 1, 64, 2), b_desc0 = smem_desc(smem_u32(sB), 1, 64, 2);
            const uint64_t sfa_desc0 = smem_desc(smem_u32(sSFA), 0, 8, 0);
            bool ok = true;
            for (uint32_t ph = 0; ph < 2 && ok; ++ph) {
                const PhaseShape &ps = ph ? PD : PU;
                const Run &run = ph ? RD : RU;
                if (!run.n) continue;
                const uint32_t i0 = ph ? RU.n : 0u;
                // the phase's digit rows are in shared memory, their scales in tensor memory
                ok = mbar_wait(bar(ph ? kBarDigitsDown : kBarDigitsUp), 0, &abort_flag);
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                fence_after();
                const uint32_t l0 = (m ^ i0) & 1u;  // first unit of this phase with ring index parity m
                UnitCursor c = cursor_at(run.u0 + l0, ps.upt, ps.tpj);
                uint32_t slot_t = ~0u, b = 0;
                CYC_DECL(4);
                for (uint32_t l = l0; l < run.n; l += 2) {
                    const uint32_t i = i0 + l;
                    if (c.t != slot_t) {
                        slot_t = c.t;
                        b = ph ? c.j - RD.job_first : slot_up(c.j);
                    }
                    const uint32_t ks = ph ? c.w : (c.w >> 1);
                    const uint32_t s = i % kRing, par = (i / kRing) & 1u;
                    CYC_LAP(0);
                    if (!mbar_wait(bar(kBarFull + s), par, &abort_flag)) { ok = false; break; }
                    if (i == 0) TRACE(3);
                    CYC_LAP(1);
                    if (i >= kRing && !mbar_wait(bar(kBarAccFree + s), par ^ 1u, &abort_flag)) { ok = false; break; }
                    CYC_LAP(2);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    fence_after();
                    const uint32_t sfa_t = tmem + kSfaCol0 + s * 8u, sfb_t = tmem + kSfbCol0 + b * ps.sfb_cols + ks * 8u;
                    const uint64_t sfa_d = sfa_desc0 + s * (kStageSf >> 4);
                    tmem_copy_scales(sfa_t, sfa_d);
                    tmem_copy_scales(sfa_t + 4u, sfa_d + (512u >> 4));
                    const uint64_t ad = a_desc0 + s * (kStageA >> 4), bd = b_desc0 + ((b * ps.b_stride + ks * 2048u) >> 4);
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk) {
                        const uint32_t atom = kk >> 1, sfid = (kk & 1u) * 2u;
                        umma_mxf4(tmem + s * 16u, ad + kk * 2u, bd + kk * 2u, kIdesc | (sfid << 29) | (sfid << 4),
                                  (sfa_t + atom * 4u) | (sfid << 30), (sfb_t + atom * 4u) | (sfid << 30), kk ? 1u : 0u);
                    }
                    umma_commit(bar(kBarDone + s));
                    CYC_LAP(3);
                    cursor_advance(c, 2, ps.upt, ps.tpj);
                }
                if (m == 0 && ph == 0) {
                    CYC_STORE(0, 4);
                    TRACE(4);
                }
            }
            // nothing of this CTA's tensor work is in flight when the tensor memory is freed
            umma_commit(bar(kBarFin));
            mbar_wait(bar(kBarFin), 0, &abort_flag);
            if (m == 0) TRACE(5);
        }
    } else if (warp < 2u * kEpiGroup / 32u && (RU.n || RD.n)) {
        // ---- epilogue.  Group A (warps 0-3) sums the even units of a tile, group B (warps 4-7) the
        // odd ones: in the up phase these are the gate and the up projection. ----
        const uint32_t grp = warp >> 2, row = tid & (kEpiGroup - 1u);
        const uint32_t lane_base = tmem + (((warp & 3u) * 32u) << 16);
        bool ok = true;
        uint32_t i = 0;
        for (uint32_t ph = 0; ph < 2 && ok; ++ph) {
            const PhaseShape &ps = ph ? PD : PU;
            const Run &run = ph ? RD : RU;
            if (!run.n) continue;
            if (!ph) {
                store_digit_scales(tmem + kSfbCol0, sE, up_slots, PU.K, PU.sfb_cols, warp, lane);
                fence_before();
                mbar_arrive(bar(kBarDigitsUp));
            } else {
                // The hidden vectors of this run's jobs: wait until every up tile of them is finished,
                // then write their digit rows (the token's digits are no longer read: every MMA of
                // the up phase has completed before its accumulator was read above).
                if (tid == 0) {
                    for (uint32_t j = RD.job_first; j <= RD.job_last && ok; ++j) {
                        uint32_t tries = 0;
                        while (ld_acquire(h_ready + j) < PU.tpj) {
                            if (++tries > kSpinGlobal || abort_flag) {
                                abort_flag = 1;
                                ok = false;
                                break;
                            }
                            __nanosleep(100);
                        }
                    }
                }
                ok = epi_bar_and(ok);
                if (!ok) break;
                if (tid == 0) TRACE(6);
                build_digits(h + (size_t)RD.job_first * inter, h + (size_t)RD.job_last * inter, down_slots, PD.K, sB,
                             PD.b_stride, sE, tid, 2u * kEpiGroup);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                epi_bar_sync();  // every block exponent is written
                store_digit_scales(tmem + kSfbCol0, sE, down_slots, PD.K, PD.sfb_cols, warp, lane);
                fence_before();
                mbar_arrive(bar(kBarDigitsDown));
            }
            float hi = 0.0f, lo = 0.0f;  // hi + lo: this group's sum over the tile's units, to about 48 bits
            UnitCursor c = cursor_at(run.u0, ps.upt, ps.tpj);
            for (uint32_t l = 0; l < run.n; ++l, ++i) {
                const uint32_t s = i % kRing;
                if ((c.w & 1u) == grp) {
                    ok = __all_sync(0xffffffffu, ok && mbar_wait(bar(kBarDone + s), (i / kRing) & 1u, &abort_flag));
                    if (ok) {
                        fence_after();
                        float a[8];
                        tmem_ld8(lane_base + s * 16u, a);
                        fence_before();
                        mbar_arrive(bar(kBarAccFree + s));
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) {  // low digits first
                            float e;
                            two_sum(hi, a[jj], hi, e);
                            lo = __fadd_rn(lo, e);
                        }
                    }
                }
                const bool tile_ends = c.w + 1u == ps.upt;
                if (!tile_ends && l + 1u != run.n) {
                    cursor_advance(c, 1, ps.upt, ps.tpj);
                    continue;
                }

                // the run's units of tile c.t, [wa, c.w], are summed
                const double v = (double)hi + (double)lo;
                if (grp == 1u) xchg[row] = v;
                if (!epi_bar_and(ok)) {
                    ok = false;
                    break;
                }
                if (grp == 0u) {
                    const uint32_t t = c.t, t_begin = t * ps.upt, j = c.j, rt = c.rt;
                    const uint32_t seg_first = max(run.u0, t_begin), wa = seg_first - t_begin;
                    double v0 = ph ? v + xchg[row] : v, v1 = ph ? 0.0 : xchg[row];
                    bool finish = (wa == 0u && tile_ends);
                    double *const part = partials + (ph ? (size_t)gridDim.x * 2u * 2u * 128u : 0u);
                    if (!finish) {
                        // part of the tile's K range: leave the partial sums, count the arrival
                        const uint32_t slot = (seg_first == run.u0) ? 0u : 1u;
                        double *p = part + (size_t)(cta * 2u + slot) * 2u * 128u + row;
                        p[0] = v0;
                        if (!ph) p[128] = v1;
                        __threadfence();
                        group_bar_sync();
                        if (row == 0) {
                            const uint32_t c_first = (uint32_t)((((uint64_t)t_begin + 1u) * run.G - 1u) / run.total);
                            const uint32_t c_last = (uint32_t)((((uint64_t)t_begin + ps.upt) * run.G - 1u) / run.total);
                            unsigned int *cnt = counters + (ph ? kDownCounter0 : kUpCounter0) + t;
                            const bool last = atomicAdd(cnt, 1u) == c_last - c_first;
                            if (last) *cnt = 0u;  // ready for the next launch
                            epi_info[0] = last ? 1u : 0u;
                            epi_info[1] = c_first;
                            epi_info[2] = c_last;
                        }
                        group_bar_sync();
                        finish = epi_info[0] != 0u;
                        if (finish) {
                            __threadfence();
                            const uint32_t c_first = epi_info[1], c_last = epi_info[2];
                            v0 = 0.0;
                            v1 = 0.0;
                            for (uint32_t cc = c_first; cc <= c_last; ++cc) {  // K order
                                const uint32_t sl = ((uint32_t)(run.total * cc / run.G) >= t_begin) ? 0u : 1u;
                                const double *q = part + (size_t)(cc * 2u + sl) * 2u * 128u + row;
                                v0 += __ldcg(q);
                                if (!ph) v1 += __ldcg(q + 128);
                            }
                        }
                    }
                    if (finish && !ph) {
                        h[(size_t)j * inter + rt * 128u + row] = swiglu_limit_fast((float)v0, (float)v1);
                        __threadfence();
                        group_bar_sync();
                        if (row == 0) atomicAdd(h_ready + j, 1u);  // one more tile of job j's hidden vector
                    } else if (finish) {
                        const uint32_t n = rt * 128u + row, tk = tab.jobs[j].token;
                        d[(size_t)tab.jobs[j].out_index * hidden + n] = (float)v0;
                        if (y) {
                            // Ordered mix (examples/s14_vulkan_numeric.rs:936-946) by whoever finishes the
                            // token's last job of these 128 rows: acc = 0; acc += w * d in route order;
                            // acc += d_shared.
                            const uint32_t j0 = tab.token_job_begin[tk], j1 = tab.token_job_begin[tk + 1u];
                            __threadfence();
                            group_bar_sync();
                            if (row == 0) {
                                unsigned int *cnt = counters + kMixCounter0 + tk * kMaxRowTiles + rt;
                                const bool last = atomicAdd(cnt, 1u) == j1 - j0 - 1u;
                                if (last) *cnt = 0u;
                                epi_info[0] = last ? 1u : 0u;
                            }
                            group_bar_sync();
                            if (epi_info[0]) {
                                __threadfence();
                                float acc = 0.0f;
                                for (uint32_t jj = j0; jj < j1; ++jj) {
                                    const Job &o = tab.jobs[tab.token_jobs[jj]];
                                    const float dv = __ldcg(d + (size_t)o.out_index * hidden + n);
                                    acc = o.is_shared ? __fadd_rn(acc, dv) : __fadd_rn(acc, __fmul_rn(o.weight, dv));
                                }
                                y[(size_t)tk * hidden + n] = acc;
                            }
                        }
                    }
                }
                // xchg and epi_info are rewritten only after every epilogue thread has passed this point
                epi_bar_sync();
                hi = 0.0f;
                lo = 0.0f;
                cursor_advance(c, 1, ps.upt, ps.tpj);
            }
        }
    }

    if (tid == 0) TRACE(7);
    fence_before();
    __syncthreads();
    if (tid == 0) TRACE(10);
    if (tid == 0) {
        if (abort_flag) atomicExch(status, 0x5501u);
        // the last CTA to leave puts the hidden vectors' counters back to zero for the next launch
        __threadfence();
        unsigned int *exit_count = counters + kExitCounter;
        if (atomicAdd(exit_count, 1u) == gridDim.x - 1u) {
            for (uint32_t j = 0; j < n_jobs; ++j) h_ready[j] = 0u;
            *exit_count = 0u;
        }
    }
    if (warp == kMmaWarp0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Bytes of the digit tiles: two hidden vectors in the down phase, one token (two in a block of
// several tokens) in the up phase.
size_t digit_tile_bytes(uint32_t n_tokens, uint32_t hidden, uint32_t inter) {
    const size_t up = (size_t)(n_tokens > 1u ? 2u : 1u) * (hidden >> 8) * 2048u, down = (size_t)2u * (inter >> 8) * 2048u;
    return up > down ? up : down;
}
size_t umma_smem_bytes(uint32_t n_tokens, uint32_t hidden, uint32_t inter) {
    return (size_t)kRing * (kStageA + kStageSf) + digit_tile_bytes(n_tokens, hidden, inter);
}

template <class Kernel, class... Args>
cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
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

constexpr size_t kMaxSmem = 227u * 1024u;  // per CTA, static + dynamic

// Largest dynamic size the kernel may ask for (the limit minus its static part); 0 on failure.
size_t g_dynamic_limit = 0;

void configure_once() {
    static bool configured = false;
    if (configured) return;
    configured = true;
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, k_moe_layer_umma) != cudaSuccess) return;
    const size_t most = kMaxSmem - fa.sharedSizeBytes;
    if (cudaFuncSetAttribute(k_moe_layer_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most) != cudaSuccess) return;
    g_dynamic_limit = most;
}

}  // namespace

size_t umma_partials_bytes(int sm_count) {
    // two phases x (CTA, first or last run) x two accumulators x 128 rows of F64
    return (size_t)2 * sm_count * 2 * 2 * 128 * sizeof(double);
}

bool umma_layer_ok(int sm_count, uint32_t n_tokens, uint32_t n_jobs_max, uint32_t hidden, uint32_t inter) {
    if (n_tokens == 0u || n_tokens > kMaxTokens || n_jobs_max == 0u || (int)n_jobs_max > sm_count) return false;
    if ((hidden & 511u) || (inter & 511u) || hidden < 512u || inter < 512u) return false;
    if (n_jobs_max * (inter >> 7) > kMaxTiles || n_jobs_max * (hidden >> 7) > kMaxTiles) return false;
    if ((hidden >> 7) > kMaxRowTiles || hidden > kMaxK || inter > kMaxK || n_jobs_max > kMaxJobs) return false;
    configure_once();
    return umma_smem_bytes(n_tokens, hidden, inter) <= g_dynamic_limit;
}

cudaError_t launch_moe_layer_umma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                                  uint32_t n_tokens, const float *x, float *h, float *d, float *y, double *partials,
                                  unsigned int *counters, uint32_t *status, uint32_t hidden, uint32_t inter,
                                  bool after_router) {
    configure_once();
    return launch_pdl(k_moe_layer_umma, dim3(sm_count), dim3(kThreads), umma_smem_bytes(n_tokens, hidden, inter), st,
                      after_router, dev, param, x, h, d, y, partials, counters, status, hidden, inter,
                      (uint32_t)digit_tile_bytes(n_tokens, hidden, inter));
}

}  // namespace s14
