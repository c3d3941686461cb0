// The pairwise-order MoE layer of one token on the fifth-generation tensor cores:
// tcgen05.mma kind::mxf4.block_scale consumes the page bytes as they are (packed E2M1, one
// UE8M0 scale per 32 elements along K), so no thread decodes or scales a weight.
//
// The matvec as a block-scaled MMA.  A = 128 weight rows x 64 K-elements per instruction; its
// scales go to tensor memory with tcgen05.cp.  B = the activation vector as eight balanced
// base-8 digit rows: within a scale block of 32 elements with largest magnitude < 2^E
// (E >= -100), every element is q * 2^(E-23) with |q| <= 2^23 (rounded to nearest when it has
// more bits below the block's top bit), q = sum_j d_j 8^j with d_j in [-4, 4] -- all of them
// E2M1 values -- and digit row j carries the UE8M0 scale 2^(E-23+3j).  Accumulator column j
// holds the digit-j share of the dot product in F32; the eight columns are added low digits
// first.  Measured against a double-precision sum on B200: relative RMSE 1.5e-7, nearly all of it
// from the 23-bit quantisation of elements far below their block's largest one.  Columns 8-15 of
// the 16-column MMA are zero rows.
//
// Work split: by slice.  An item is (expert, 64 intermediate elements): the 64 rows of w1 and
// the 64 rows of w3 that produce them form one 128-row MMA tile over K = hidden (up phase, one
// accumulator: lanes 0-63 the gate, 64-127 the up projection), and the 64 columns of w2 that
// consume them are hidden / 128 MMAs of K = 64 (down phase).  The hidden values of a slice never
// leave the CTA: SwiGLU, digits and scales are made from the up accumulator and fed to the down
// MMAs.  Each item leaves its contribution to the expert's output, 4 bytes per row, in global
// scratch; when every item of the layer is done (one counter, bounded polling; the grid is one
// CTA per SM, all resident), every CTA adds up its share of the rows in slice order and applies
// the ordered mix.  Items are handed out in equal numbers, so the result does not depend on how.
// The expert page stores w2 and all scales by slice for this purpose.
//
// Roles inside a CTA: four producer warps (cp.async into a 10-stage ring of 16 KB of codes + 2 KB
// of scales: up units of all items first, then down stages), four MMA-issuing threads, eight
// epilogue warps (tcgen05.ld / tcgen05.st).  Every mbarrier wait and the poll of the item
// counter are bounded; a wait that runs out raises the CTA's abort flag, the status word is set
// and the CTA drains its copies, frees its tensor memory and returns.
#include "s14_device.cuh"

namespace s14 {

namespace {

constexpr uint32_t kRing = 10;                 // stages in flight per CTA (even: an up unit's parity is its slot's)
constexpr uint32_t kStageA = 128 * 128;        // 16 KB of codes: an up unit (128 rows x 256 K) or four down blocks (128 rows x 64 K each)
constexpr uint32_t kStageSf = 4 * 512;         // scale atoms of a stage: two (up unit) or four (down stage)
constexpr uint32_t kEpiGroup = 128;            // two epilogue groups of four warps
constexpr uint32_t kMmaWarp0 = 8;              // warps 8, 9, 14, 15: one issuing thread each (lane 0)
constexpr uint32_t kIssuers = 4;
constexpr uint32_t kProdWarp0 = 10;            // warps 10..13 copy
constexpr uint32_t kProdThreads = 128;
constexpr uint32_t kThreads = 512;
constexpr uint32_t kDRing = 4;                 // down stages whose four accumulators are in flight (one per issuing thread)
constexpr uint32_t kItemSlots = 4;             // items a CTA can hold (digit tiles of their hidden values)
// tensor memory columns
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColD = 0;                  // kDRing x 4 accumulators x 16
constexpr uint32_t kColU = kColD + kDRing * 64;    // 2 issuing threads x 16 (one item at a time)
constexpr uint32_t kColSfa = kColU + 32;       // kIssuers x 16: weight scales of the stage each issuing thread is at
// Scales of digit rows: an atom (four scale blocks) is four columns (N-rows 0-31, 32-63, ...; a 16-row
// operand uses the first).  Scale addresses given to the MMA stay atom-aligned.
constexpr uint32_t kColSfbX = kColSfa + kIssuers * 16;  // hidden / 32: scales of the token's digit rows
constexpr uint32_t kColSfbH = kColSfbX + 128;           // kItemSlots x 4: scales of the hidden values' digit rows
static_assert(kColSfbH + kItemSlots * 4 <= kTmemCols, "tensor memory map");
constexpr uint32_t kMaxHidden = 4096;          // 128 columns of token digit scales
constexpr uint32_t kMaxBlocks = kMaxHidden / 32;
constexpr uint32_t kSpin = 1u << 17;           // tries (a microsecond each at most) before a wait gives up
constexpr uint32_t kSpinGlobal = 1u << 20;     // polls (100 ns apart) of the item counter before giving up
constexpr uint32_t kItemCounter = 1, kExitCounter = 2;  // in the context's counter array ([0] is the router's)
constexpr uint32_t kRouteCounter = 3;          // CTAs whose expert scores are written (routes computed in this kernel)
constexpr uint32_t kRouterSlots = 4;           // experts a CTA scores at most

// Bar indices in the static barrier array.
constexpr uint32_t kBarFull = 0;                      // ring slot filled with an up unit (128 copying threads)
constexpr uint32_t kBarDFull = kRing;                 // ring slot filled with a down stage
constexpr uint32_t kBarDone = 2 * kRing;              // the slot's MMAs have completed (the copies may reuse it)
constexpr uint32_t kBarDFree = 3 * kRing;             // a down stage's accumulators have been read
constexpr uint32_t kBarDDone = kBarDFree + kDRing;    // a down stage's accumulators are complete
constexpr uint32_t kBarUDone = kBarDDone + kDRing;    // an item's up accumulators are complete
constexpr uint32_t kBarUFree = kBarUDone + 1;         // ... have been read
constexpr uint32_t kBarHReady = kBarUFree + 1;        // an item's hidden digits and scales are in place
constexpr uint32_t kBarXReady = kBarHReady + kItemSlots;  // the token's digit scales are in tensor memory
constexpr uint32_t kBarFin = kBarXReady + 1;          // both issuing threads have finished
constexpr uint32_t kBars = kBarFin + 1;

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
// Named barrier 1: the 128 threads of epilogue group A.
__device__ __forceinline__ void group_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
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
// Eight accumulator columns of the warp's 32 lanes; the values may be used after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }


// Instruction descriptor: A and B E2M1 (format 1), both K-major, N = 16, UE8M0 scales, M = 128.
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);

// Writes the eight digit rows of elements 8g .. 8g+7 of a vector and, for the first thread of a
// scale block, the block's exponent.  Thread g of the CTA owns group g, i.e. one 32-bit word of
// every digit row; the four lanes of a scale block agree on its exponent E (largest magnitude
// < 2^E, clamped to [-100, 127]), so whole warps call this together.  With the bias
// 4 * (8^8 - 1) / 7 added, the balanced digits of q are the plain base-8 digits minus 4, so no
// carry runs through them.  Rows 8-15 of the tile are zeroed by the caller; the blocks' exponents
// go to sE, from which store_digit_scales writes the digit rows' scale codes into tensor memory.
__device__ __forceinline__ void digits_of8(const float (&xs)[8], uint32_t g, uint8_t *sB, uint8_t *sE) {
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
    uint8_t *chunk = sB + (kb >> 3) * 2048u + (g & 3u) * 4u;
#pragma unroll
    for (uint32_t j = 0; j < 8; ++j)
        *reinterpret_cast<uint32_t *>(chunk + j * 128u + (((kb & 7u) ^ j) << 4)) = words[j];
    if ((g & 3u) == 0u) sE[kb] = (uint8_t)(E + 100);  // the block's exponent, biased
}

// The scale codes of the digit rows, written to tensor memory by the eight epilogue warps (each
// lane quadrant takes every atom; warps 0-3 the even groups of four atoms, warps 4-7 the odd ones).
// Column 4a of lane l holds the codes of N-row l for scale blocks 4a..4a+3: digit row l < 8 of a
// block with exponent E has the code 127 + E - 23 + 3l; rows 8-15 are zero rows, columns 4a+1..4a+3
// belong to N-rows 32 and up, which a 16-column MMA does not use.
__device__ __forceinline__ void store_digit_scales(uint32_t tmem_sfb, const uint8_t *sE, uint32_t K, uint32_t warp,
                                                   uint32_t lane) {
    const uint32_t groups = K >> 9;  // groups of four atoms (512 K-elements, 16 blocks)
    const uint32_t bias = 0x01010101u * (4u + 3u * (lane & 7u));
    const uint32_t quad = tmem_sfb + (((warp & 3u) * 32u) << 16);
    for (uint32_t g = warp >> 2; g < groups; g += 2u) {
        const uint4 e = *reinterpret_cast<const uint4 *>(sE + g * 16u);
        const uint32_t one = 0x7F7F7F7Fu;
        const uint32_t w0 = lane < 8u ? e.x + bias : one, w1 = lane < 8u ? e.y + bias : one;
        const uint32_t w2 = lane < 8u ? e.z + bias : one, w3 = lane < 8u ? e.w + bias : one;
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%5,%5,%5,%2,%5,%5,%5,%3,%5,%5,%5,%4,%5,%5,%5};"
            ::"r"(quad + g * 16u), "r"(w0), "r"(w1), "r"(w2), "r"(w3), "r"(one)
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


__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire(const unsigned int *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// No-swizzle K-major tile of 8-row x 16-byte core matrices for K = 64 (32 bytes per row): the two
// halves of a row are 128 B apart (leading offset), 8-row groups 256 B apart (stride offset).
__device__ __forceinline__ uint64_t smem_desc_k64(uint32_t addr) { return smem_desc(addr, 8, 16, 0); }

// The routes of the token from the experts' scores, by one warp (the same picks, sums and weights
// as k_router's last block: largest score + bias first, lowest id on ties; weight = score / sum of
// the picked scores x route_scale).  Scores, selection values and page addresses come in one round
// of loads; the picked expert's values come from the lane that holds them.  Lane 0 writes the jobs
// (route order, the shared expert last), the mix and every route's weight; `publish` also writes
// the caller's ids and weights.  Expert parallel: the rank keeps the jobs of the experts it owns and, as the shared
// expert's owner, the shared job; every job writes the row of its route slot.
__device__ void route_select(const FusedRouter &rt, uint32_t lane, bool publish, Job *jobs, uint32_t *n_jobs_out,
                             float *mix_w, uint32_t *mix_job, float *route_w) {
    unsigned long long key[8], pg[8];
    float sc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t e = i * 32 + lane;
        key[i] = 0ull;
        pg[i] = 0ull;
        sc[i] = 0.0f;
        if (e < rt.n_experts) {
            const uint32_t bits = __float_as_uint(__ldcg(rt.select + e));
            sc[i] = __ldcg(rt.scores + e);
            pg[i] = __ldg(reinterpret_cast<const unsigned long long *>(rt.page_table) + e);
            const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
            key[i] = ((unsigned long long)ordered << 32) | (unsigned long long)(0xffffffffu - e);
        }
    }
    int32_t ids[S14_EXPERTS_PER_TOKEN];
    float picked[S14_EXPERTS_PER_TOKEN];
    unsigned long long pages[S14_EXPERTS_PER_TOKEN];
#pragma unroll
    for (int j = 0; j < S14_EXPERTS_PER_TOKEN; ++j) {
        ids[j] = -1;
        picked[j] = 0.0f;
        pages[j] = 0ull;
        if ((uint32_t)j < rt.top_k) {
            unsigned long long best = key[0];
#pragma unroll
            for (int i = 1; i < 8; ++i) best = key[i] > best ? key[i] : best;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
                best = other > best ? other : best;
            }
            const uint32_t e = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
            float my_sc = sc[0];
            unsigned long long my_pg = pg[0];
#pragma unroll
            for (int i = 1; i < 8; ++i) {
                if ((e >> 5) == (uint32_t)i) {
                    my_sc = sc[i];
                    my_pg = pg[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (key[i] == best) key[i] = 0ull;  // taken
            ids[j] = (int32_t)e;
            picked[j] = __shfl_sync(0xffffffffu, my_sc, e & 31u);
            pages[j] = __shfl_sync(0xffffffffu, my_pg, e & 31u);
        }
    }
    if (lane != 0) return;
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < S14_EXPERTS_PER_TOKEN; ++j)
        if ((uint32_t)j < rt.top_k) sum = __fadd_rn(sum, picked[j]);
    uint32_t n = 0;
#pragma unroll
    for (int j = 0; j < S14_EXPERTS_PER_TOKEN; ++j) {
        if ((uint32_t)j >= rt.top_k) continue;
        const float w = __fmul_rn(__fdiv_rn(picked[j], sum), rt.route_scale);
        if (publish && rt.ids_out) rt.ids_out[j] = ids[j];
        if (publish && rt.weights_out) rt.weights_out[j] = w;
        route_w[j] = w;  // every route's weight, also of experts other ranks own
        if (((uint32_t)ids[j] % rt.ep_world) == rt.ep_rank) {
            Job jb;
            jb.page = reinterpret_cast<const uint8_t *>(pages[j]);
            jb.kind = S14_PAGE_MXFP4;
            jb.token = 0;
            jb.weight = w;
            jb.is_shared = 0;
            jb.out_index = (uint32_t)j;
            jobs[n] = jb;
            mix_w[n] = w;
            mix_job[n] = n;
            ++n;
        }
    }
    if (rt.shared_page && rt.shared_owner == rt.ep_rank) {
        Job jb;
        jb.page = rt.shared_page;
        jb.kind = rt.shared_kind;
        jb.token = 0;
        jb.weight = 1.0f;
        jb.is_shared = 1;
        jb.out_index = rt.top_k;
        jobs[n] = jb;
        mix_w[n] = 1.0f;
        mix_job[n] = n | 0x80000000u;
        ++n;
    }
    *n_jobs_out = n;
}

__global__ void __launch_bounds__(kThreads, 1)
k_moe_layer_umma(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
                 const float *__restrict__ x, float *d_out, float *__restrict__ y, float *part,
                 unsigned int *counters, uint32_t *__restrict__ status, uint32_t hidden, uint32_t inter,
                 const __grid_constant__ FusedRouter rt, const __grid_constant__ EpExchange ep) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[kBars];
    __shared__ __align__(16) uint8_t sE[kMaxBlocks];         // block exponents of the token's digits
    __shared__ __align__(16) uint8_t sBh[kItemSlots * 512];  // digit tiles of the items' hidden values (rows 8-15 zero)
    __shared__ float s_up[64];                               // an item's up projection, handed to the gate threads
    __shared__ uint8_t sEh[kItemSlots][2];
    __shared__ float s_mix_w[S14_EXPERTS_PER_TOKEN + 1];        // the mix, in route order: weight (shared expert: 1)
    __shared__ uint32_t s_mix_job[S14_EXPERTS_PER_TOKEN + 1];   //   job, bit 31 set for the shared expert
    __shared__ Job s_jobs[S14_EXPERTS_PER_TOKEN + 1];           // the layer's jobs, from the routes or the caller's table
    __shared__ uint32_t s_n_jobs;
    __shared__ float s_route_w[S14_EXPERTS_PER_TOKEN];         // expert parallel: the weight of every route
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int s_behind;  // expert parallel: a peer's word carries a later step's number

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const bool is_producer = warp >= kProdWarp0 && warp < kProdWarp0 + kProdThreads / 32u;
    const uint32_t KU = hidden >> 8;   // up units of an item (256 K-elements each)
    const uint32_t DS = hidden >> 9;   // down stages of an item (four 128-row tiles each)
    const uint32_t RT = hidden >> 7;   // row tiles of w2
    const uint32_t S = inter >> 6;     // slices of an expert
    uint8_t *const sA = smem;
    uint8_t *const sSF = sA + kRing * kStageA;
    uint8_t *const sBx = sSF + kRing * kStageSf;  // the token's digit tile, 2 KB per 256 K-elements
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](uint32_t i) { return bar0 + i * 8u; };

    // Thread t owns elements 8t .. 8t+7 of the token (hidden <= 8 x kThreads), for the digits and for
    // the router's dot products; the router weights of this CTA's experts (cta, cta + grid, ...) are
    // asked for first, so that they arrive while the CTA sets itself up.
    const bool routes_here = rt.weight != nullptr;
    // expert parallel: the step count picks the slot buffer and the flag value; the last CTA to
    // leave advances it, after every CTA has read it
    const bool ep_on = ep.world > 1u;
    const bool has_x = tid < (hidden >> 3);
    float xs[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    uint4 rq[kRouterSlots];
    if (routes_here) {
#pragma unroll
        for (uint32_t k = 0; k < kRouterSlots; ++k) {
            const uint32_t e = blockIdx.x + k * gridDim.x;
            rq[k] = make_uint4(0u, 0u, 0u, 0u);
            if (has_x && e < rt.n_experts) rq[k] = ldg_stream(reinterpret_cast<const uint4 *>(rt.weight + (size_t)e * hidden) + tid);
        }
    }
    // The kernel is launched as a programmatic dependent of whatever precedes it in the stream: its
    // CTAs may be placed as soon as SMs are free and set themselves up (barriers, tensor memory);
    // everything an earlier kernel may have written (the token, the counters, the step count) is read
    // only after cudaGridDependencySynchronize() below.  In the same way the next launch may be set
    // up from now on.  Weights and page tables are constant during a step.
    cudaTriggerProgrammaticLaunchCompletion();

    // rows 8-15 of the digit tiles stay zero
    for (uint32_t i = tid; i < (KU * 2048u) >> 4; i += kThreads) reinterpret_cast<uint4 *>(sBx)[i] = make_uint4(0u, 0u, 0u, 0u);
    for (uint32_t i = tid; i < sizeof(sBh) / 4u; i += kThreads) reinterpret_cast<uint32_t *>(sBh)[i] = 0u;
    if (tid == 0) {
        for (uint32_t s = 0; s < kRing; ++s) {
            mbar_init(bar(kBarFull + s), kProdThreads);
            mbar_init(bar(kBarDFull + s), kProdThreads);
            mbar_init(bar(kBarDone + s), 1);
        }
        for (uint32_t s = 0; s < kDRing; ++s) {
            mbar_init(bar(kBarDFree + s), kEpiGroup);
            mbar_init(bar(kBarDDone + s), 1);
        }
        mbar_init(bar(kBarUDone), 2);
        mbar_init(bar(kBarUFree), kEpiGroup);
        for (uint32_t s = 0; s < kItemSlots; ++s) mbar_init(bar(kBarHReady + s), kEpiGroup);
        mbar_init(bar(kBarXReady), 2u * kEpiGroup);
        mbar_init(bar(kBarFin), kIssuers);
        abort_flag = 0;
        s_behind = 0;
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

    cudaGridDependencySynchronize();
    const uint32_t ep_step = ep_on ? __ldcg(ep.step) : 0u;
    if (has_x) {
        const float4 p0 = __ldcg(reinterpret_cast<const float4 *>(x) + 2u * tid);
        const float4 p1 = __ldcg(reinterpret_cast<const float4 *>(x) + 2u * tid + 1u);
        xs[0] = p0.x, xs[1] = p0.y, xs[2] = p0.z, xs[3] = p0.w;
        xs[4] = p1.x, xs[5] = p1.y, xs[6] = p1.z, xs[7] = p1.w;
    }

    if (routes_here) {
        // ---- expert scores: logit = x . w in double (warp sums, then the sixteen warps in order),
        // rounded to F32; score and score + bias go to global memory, then the CTA counts itself ----
        double *s_red = reinterpret_cast<double *>(smem);  // [slot][warp]; the ring is not in use yet
#pragma unroll
        for (uint32_t k = 0; k < kRouterSlots; ++k) {
            if (blockIdx.x + k * gridDim.x >= rt.n_experts) break;
            const uint32_t wd[4] = {rq[k].x, rq[k].y, rq[k].z, rq[k].w};
            double acc0 = 0.0, acc1 = 0.0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc0 += (double)xs[i * 2] * (double)__uint_as_float(wd[i] << 16);
                acc1 += (double)xs[i * 2 + 1] * (double)__uint_as_float(wd[i] & 0xffff0000u);
            }
            const double ws = warp_sum(acc0 + acc1);
            if (lane == 0) s_red[k * (kThreads / 32u) + warp] = ws;
        }
        __syncthreads();
        if (tid < kRouterSlots && blockIdx.x + tid * gridDim.x < rt.n_experts) {
            const uint32_t e = blockIdx.x + tid * gridDim.x;
            double sum = 0.0;
            for (uint32_t w = 0; w < kThreads / 32u; ++w) sum += s_red[tid * (kThreads / 32u) + w];
            const float sc = router_score_f32(sum, rt.score_fn);
            rt.scores[e] = sc;
            rt.select[e] = __fadd_rn(sc, rt.bias ? rt.bias[e] : 0.0f);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) atomicAdd(counters + kRouteCounter, 1u);
    }

    // the token's digits (they do not depend on the routes)
    if (has_x) digits_of8(xs, tid, sBx, sE);
    __syncthreads();  // every block exponent is written
    if (warp < 2u * kEpiGroup / 32u) {
        store_digit_scales(tmem + kColSfbX, sE, hidden, warp, lane);
        fence_before();
        mbar_arrive(bar(kBarXReady));
    }
    const uint32_t grid = gridDim.x, cta = blockIdx.x;
    if (routes_here) {
        // every CTA's scores are needed: all CTAs are resident (one per SM), the wait is bounded
        if (tid == 0) {
            uint32_t tries = 0;
            while (ld_acquire(counters + kRouteCounter) < grid) {
                if (++tries > kSpinGlobal) {
                    abort_flag = 1;
                    break;
                }
                __nanosleep(40);
            }
        }
        __syncthreads();
        if (warp == 0 && !abort_flag) route_select(rt, lane, cta == 0, s_jobs, &s_n_jobs, s_mix_w, s_mix_job, s_route_w);
        if (tid == 0 && abort_flag) s_n_jobs = 0;
    } else {
        const JobTable &tab = table_of(dev_table, param_table);
        const uint32_t nj = min(tab.token_job_begin[1] - tab.token_job_begin[0], (uint32_t)S14_EXPERTS_PER_TOKEN + 1u);
        if (tid < min(tab.n_jobs, (uint32_t)S14_EXPERTS_PER_TOKEN + 1u)) s_jobs[tid] = tab.jobs[tid];
        if (tid < nj) {
            const uint32_t jb = tab.token_jobs[tab.token_job_begin[0] + tid];  // the job table may live in global memory
            s_mix_w[tid] = tab.jobs[jb].weight;
            s_mix_job[tid] = jb | (tab.jobs[jb].is_shared ? 0x80000000u : 0u);
        }
        if (tid == 0) s_n_jobs = min(tab.n_jobs, (uint32_t)S14_EXPERTS_PER_TOKEN + 1u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the digit tiles are read by the tensor cores
    __syncthreads();
    const uint32_t n_jobs = s_n_jobs, n_items = n_jobs * S;
    // items are dealt in equal shares; with more CTAs than items the last CTAs have none
    const uint32_t G = min(grid, n_items);
    const uint32_t q0 = cta < G ? (uint32_t)((uint64_t)n_items * cta / G) : 0u;
    const uint32_t q1 = cta < G ? (uint32_t)((uint64_t)n_items * (cta + 1u) / G) : 0u;
    const uint32_t n_it = min(q1 - q0, kItemSlots);  // the launcher keeps the share within kItemSlots
    const uint32_t nU = n_it * KU, nD = n_it * DS;

    if (is_producer && n_it) {
        // ---- copies: the up units of every item, then the down stages of every item ----
        const uint32_t pt = tid - kProdWarp0 * 32u, r8 = pt >> 3, cc = pt & 7u;
        const uint32_t dst_up = smem_u32(sA) + r8 * 128u + ((cc ^ (r8 & 7u)) << 4);
        bool ok = true;
        uint32_t i = 0;
        for (uint32_t l = 0; l < n_it && ok; ++l) {
            const uint32_t q = q0 + l, j = q / S, sl = q - j * S;
            const PageView pv = page_view(s_jobs[j].page, S14_PAGE_MXFP4, hidden, inter);
            // rows r8, r8 + 16, ... of the tile: the first four are w1 rows of the slice, the last four w3 rows
            const uint8_t *src1 = pv.w1 + (size_t)(sl * 64u + r8) * (hidden >> 1) + cc * 16u;
            const uint8_t *src3 = pv.w3 + (size_t)(sl * 64u + r8) * (hidden >> 1) + cc * 16u;
            const uint8_t *sf = pv.s1 + (size_t)sl * RT * 512u + pt * 16u;
            for (uint32_t ks = 0; ks < KU; ++ks, ++i) {
                const uint32_t s = i % kRing;
                if (i >= kRing && !mbar_wait(bar(kBarDone + s), ((i / kRing) - 1u) & 1u, &abort_flag)) {
                    ok = false;
                    break;
                }
                const uint32_t dst = dst_up + s * kStageA;
#pragma unroll
                for (uint32_t i8 = 0; i8 < 4; ++i8) {
                    cp_async16(dst + i8 * 2048u, src1 + (size_t)i8 * 16u * (hidden >> 1) + ks * 128u);
                    cp_async16(dst + (i8 + 4u) * 2048u, src3 + (size_t)i8 * 16u * (hidden >> 1) + ks * 128u);
                }
                // the unit's two scale atoms are 1 KB of consecutive page bytes
                if (pt < 64u) cp_async16(smem_u32(sSF + s * kStageSf) + pt * 16u, sf + (size_t)ks * 1024u);
                mbar_arrive_after_copies(bar(kBarFull + s));
            }
        }
        for (uint32_t l = 0; l < n_it && ok; ++l) {
            const uint32_t q = q0 + l, j = q / S, sl = q - j * S;
            const PageView pv = page_view(s_jobs[j].page, S14_PAGE_MXFP4, hidden, inter);
            const uint8_t *wsrc = pv.w2 + (size_t)sl * RT * 4096u + pt * 16u;        // the slice's columns, 4 KB per row tile
            const uint8_t *sf = pv.s2 + (size_t)(sl >> 1) * RT * 512u + pt * 16u;   // the slice pair's atoms
            for (uint32_t v = 0; v < DS; ++v, ++i) {
                const uint32_t s = i % kRing;
                if (i >= kRing && !mbar_wait(bar(kBarDone + s), ((i / kRing) - 1u) & 1u, &abort_flag)) {
                    ok = false;
                    break;
                }
                const uint32_t dst = smem_u32(sA + s * kStageA);
#pragma unroll
                for (uint32_t i8 = 0; i8 < 8; ++i8) {
                    // piece id: block id / 256, row (id % 256) / 2, half id % 2 -> 8-row x 16-byte core matrices
                    const uint32_t id = pt + i8 * 128u, r = (id & 255u) >> 1;
                    cp_async16(dst + (id >> 8) * 4096u + (r >> 3) * 256u + (id & 1u) * 128u + (r & 7u) * 16u,
                               wsrc + (size_t)v * 16384u + i8 * 2048u);
                }
                cp_async16(smem_u32(sSF + s * kStageSf) + pt * 16u, sf + (size_t)v * 2048u);
                mbar_arrive_after_copies(bar(kBarDFull + s));
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if ((warp == kMmaWarp0 || warp == kMmaWarp0 + 1u || warp >= 14u) && n_it) {
        if (lane == 0) {
            // ---- MMA issue.  Issuing a tcgen05 operation costs the thread 70-90 cycles (measured), more
            // than a 16 KB stage may take once it has up to ten of them, so four threads issue.  Thread 0
            // issues the up units (one accumulator per item, in order); the down stages have
            // accumulators of their own and go round the four threads.  The down stages use ring-slot
            // barriers of their own, so each thread sees every phase of the barriers it waits on. ----
            const uint32_t m = warp < 14u ? warp - kMmaWarp0 : warp - 12u;
            const uint64_t a_up0 = smem_desc(smem_u32(sA), 1, 64, 2), b_x0 = smem_desc(smem_u32(sBx), 1, 64, 2);
            const uint64_t sf_desc0 = smem_desc(smem_u32(sSF), 0, 8, 0);
            const uint32_t sfa_t = tmem + kColSfa + m * 16u;  // a thread's copies and MMAs execute in issue order
            bool ok = true;
            if (m < 2u) {
                // up units: threads 0 and 1 take the even and the odd ones (hidden / 256 is even, so the
                // parity of a unit is the parity of its ring slot) and accumulate into accumulators of their own
                ok = mbar_wait(bar(kBarXReady), 0, &abort_flag);
                for (uint32_t l = 0; l < n_it && ok; ++l) {
                    // the two up accumulators serve one item at a time
                    if (l >= 1u) ok = mbar_wait(bar(kBarUFree), (l - 1u) & 1u, &abort_flag);
                    const uint32_t acc = tmem + kColU + m * 16u;
                    for (uint32_t ks = m; ks < KU && ok; ks += 2u) {
                        const uint32_t i = l * KU + ks, s = i % kRing;
                        ok = mbar_wait(bar(kBarFull + s), (i / kRing) & 1u, &abort_flag);
                        if (!ok) break;
                        fence_after();
                        const uint32_t sfb_t = tmem + kColSfbX + ks * 8u;
                        const uint64_t sfd = sf_desc0 + s * (kStageSf >> 4);
                        tmem_copy_scales(sfa_t, sfd);
                        tmem_copy_scales(sfa_t + 4u, sfd + (512u >> 4));
                        const uint64_t ad = a_up0 + s * (kStageA >> 4), bd = b_x0 + ks * (2048u >> 4);
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) {
                            const uint32_t atom = kk >> 1, sfid = (kk & 1u) * 2u;
                            umma_mxf4(acc, ad + kk * 2u, bd + kk * 2u, kIdesc | (sfid << 29) | (sfid << 4),
                                      (sfa_t + atom * 4u) | (sfid << 30), (sfb_t + atom * 4u) | (sfid << 30),
                                      (ks >= 2u || kk) ? 1u : 0u);
                        }
                        umma_commit(bar(kBarDone + s));
                        if (ks + 2u >= KU) umma_commit(bar(kBarUDone));
                    }
                }
            }
            {
                // Down stage vg sits in ring slot s = (nU + vg) % kRing and belongs to the issuing thread and
                // accumulator set s % 4, so that every slot's barrier has one waiting thread, which sees
                // each of its phases; j counts this thread's down stages (the phases of its own barriers).
                uint32_t j = 0;
                for (uint32_t vg = 0; vg < nD && ok; ++vg) {
                    const uint32_t s = (nU + vg) % kRing;
                    if ((s & 3u) != m) continue;
                    const uint32_t l = vg / DS, sl = (q0 + l) % S, asf = (sl & 1u) * 2u;
                    ok = mbar_wait(bar(kBarHReady + l), 0, &abort_flag);
                    ok = ok && mbar_wait(bar(kBarDFull + s), (vg / kRing) & 1u, &abort_flag);
                    ok = ok && (j == 0u || mbar_wait(bar(kBarDFree + m), (j - 1u) & 1u, &abort_flag));
                    if (!ok) break;
                    ++j;
                    fence_after();
                    const uint64_t sfd = sf_desc0 + s * (kStageSf >> 4);
                    const uint64_t bd = smem_desc_k64(smem_u32(sBh + l * 512u));
                    const uint64_t ad = smem_desc_k64(smem_u32(sA + s * kStageA));
#pragma unroll
                    for (uint32_t b = 0; b < 4; ++b) tmem_copy_scales(sfa_t + b * 4u, sfd + b * (512u >> 4));
#pragma unroll
                    for (uint32_t b = 0; b < 4; ++b)
                        umma_mxf4(tmem + kColD + m * 64u + b * 16u, ad + b * (4096u >> 4), bd, kIdesc | (asf << 29),
                                  (sfa_t + b * 4u) | (asf << 30), tmem + kColSfbH + l * 4u, 0u);
                    umma_commit(bar(kBarDone + s));
                    umma_commit(bar(kBarDDone + m));
                }
            }
            // nothing of this CTA's tensor work is in flight when the tensor memory is freed
            umma_commit(bar(kBarFin));
            mbar_wait(bar(kBarFin), 0, &abort_flag);
        }
    } else if (warp < 2u * kEpiGroup / 32u && n_it) {
        // ---- epilogue: group A (warps 0-3) turns the up accumulators into hidden digits, then both
        // groups read the down accumulators (alternate stages) ----
        const uint32_t grp = warp >> 2, row = tid & (kEpiGroup - 1u);
        const uint32_t lane_base = tmem + (((warp & 3u) * 32u) << 16);
        bool ok = true;
        if (grp == 0u) {
            for (uint32_t l = 0; l < n_it; ++l) {
                const uint32_t q = q0 + l, j = q / S;
                ok = __all_sync(0xffffffffu, ok && mbar_wait(bar(kBarUDone), l & 1u, &abort_flag));
                float v = 0.0f;
                if (ok) {
                    fence_after();
                    uint32_t a[8], b[8];  // even and odd units of the item
                    tmem_ld8(lane_base + kColU, a);
                    tmem_ld8(lane_base + kColU + 16u, b);
                    tmem_ld_wait();
                    fence_before();
                    mbar_arrive(bar(kBarUFree));
                    // Digit columns, low digits first, each column about eight times the one before: plain F32
                    // additions lose a few 2^-24 of the result, below the 23-bit digits of what follows.
                    float sa = 0.0f, sb = 0.0f;
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) {
                        sa = __fadd_rn(sa, __uint_as_float(a[jj]));
                        sb = __fadd_rn(sb, __uint_as_float(b[jj]));
                    }
                    v = __fadd_rn(sa, sb);
                }
                if (row >= 64u) s_up[row - 64u] = v;
                group_bar_sync();
                (void)j;
                if (row < 64u) {
                    // hidden value `row` of the slice -> eight digit nibbles, scale block = warp
                    const float hv = swiglu_limit_fast(v, s_up[row]);
                    float bm = fabsf(hv);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
                    int E = -100;
                    if (bm > 0.0f) E = min(max((int)((__float_as_uint(bm) >> 23) & 0xFFu) - 126, -100), 127);
                    const uint32_t qb = (uint32_t)(__float2int_rn(hv * __uint_as_float((uint32_t)(150 - E) << 23)) + 0x924924);
                    uint32_t word = 0;
#pragma unroll
                    for (int jj = 0; jj < 7; ++jj) word |= ((0x5420ACDEu >> (((qb >> (3 * jj)) & 7u) << 2)) & 0xFu) << (4 * jj);
                    const uint32_t top = qb >> 21;
                    word |= (top > 7u ? 6u : ((0x5420ACDEu >> (top << 2)) & 0xFu)) << 28;
                    const uint32_t other = __shfl_xor_sync(0xffffffffu, word, 1);
                    const uint32_t lo_w = (lane & 1u) ? other : word, hi_w = (lane & 1u) ? word : other;
                    uint8_t *chunk = sBh + l * 512u + warp * 128u + (lane >> 1);  // K half = scale block = warp
#pragma unroll
                    for (uint32_t jj = 0; jj < 4; ++jj) {
                        const uint32_t dj = (lane & 1u) * 4u + jj;  // digit row
                        chunk[dj * 16u] = (uint8_t)(((lo_w >> (4u * dj)) & 0xFu) | (((hi_w >> (4u * dj)) & 0xFu) << 4));
                    }
                    if (lane == 0) sEh[l][warp] = (uint8_t)(E + 100);
                }
                group_bar_sync();
                {
                    // scale codes of the eight digit rows for the slice's two blocks (blocks 2, 3 unused)
                    const uint32_t bias = 4u + 3u * (lane & 7u);
                    const uint32_t w0 = lane < 8u ? ((sEh[l][0] + bias) | ((sEh[l][1] + bias) << 8) | 0x7F7F0000u) : 0x7F7F7F7Fu;
                    const uint32_t one = 0x7F7F7F7Fu;
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%2,%2};" ::"r"(lane_base + kColSfbH + l * 4u),
                                 "r"(w0), "r"(one)
                                 : "memory");
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                fence_before();
                mbar_arrive(bar(kBarHReady + l));
            }
        }
        uint32_t seen_lo = 0, seen_hi = 0;  // down stages of the group's two accumulator sets so far
        for (uint32_t vg = 0; vg < nD; ++vg) {
            const uint32_t acc = ((nU + vg) % kRing) & 3u;  // the stage's issuing thread and accumulator set
            if ((acc & 1u) != grp) continue;                // sets 0, 2: group A; sets 1, 3: group B
            const uint32_t j = (acc & 2u) ? seen_hi++ : seen_lo++;
            const uint32_t l = vg / DS, vloc = vg - l * DS, q = q0 + l;
            // every phase of this barrier is waited for by this group, in order
            ok = __all_sync(0xffffffffu, ok && mbar_wait(bar(kBarDDone + acc), j & 1u, &abort_flag));
            if (!ok) break;
            fence_after();
            uint32_t a[4][8];
#pragma unroll
            for (uint32_t b = 0; b < 4; ++b) tmem_ld8(lane_base + kColD + acc * 64u + b * 16u, a[b]);
            tmem_ld_wait();
            fence_before();
            mbar_arrive(bar(kBarDFree + acc));  // the accumulators are in registers: the next stage may overwrite them
            float out[4];
#pragma unroll
            for (uint32_t b = 0; b < 4; ++b) {  // low digits first; the share is kept as one F32 anyway
                float sum = 0.0f;
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) sum = __fadd_rn(sum, __uint_as_float(a[b][jj]));
                out[b] = sum;
            }
            // the item's share of rows (4 vloc + b) * 128 + row of its expert's output
            float *p = part + (size_t)q * hidden + (size_t)vloc * 512u + row;
#pragma unroll
            for (uint32_t b = 0; b < 4; ++b) p[b * 128u] = out[b];
        }
    }

    // ---- every item's share is in global memory: count the CTA's items, wait for all of them ----
    __threadfence();
    fence_before();
    __syncthreads();
    if (warp == kMmaWarp0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
    if (tid == 0) {
        if (n_it) atomicAdd(counters + kItemCounter, abort_flag ? 0u : n_it);
        uint32_t tries = 0;
        while (!abort_flag && ld_acquire(counters + kItemCounter) < n_items) {
            if (++tries > kSpinGlobal) abort_flag = 1;
            __nanosleep(100);
        }
        if (abort_flag) atomicExch(status, 0x5501u);
    }
    __syncthreads();
    if (!abort_flag) {
        // ---- rows [n0, n1) of this CTA: expert outputs as sums over slices in slice order, then the
        // ordered mix (examples/s14_vulkan_numeric.rs:936-946): acc = 0; acc += w * d in route order;
        // acc += d_shared.  Scratch: the ring's shared memory. ----
        const uint32_t n0 = (uint32_t)((uint64_t)hidden * cta / grid), n1 = (uint32_t)((uint64_t)hidden * (cta + 1u) / grid);
        const uint32_t rows = n1 - n0, chunks = S >> 2;
        // sums as (hi, lo) pairs of F32 with error-free additions: FP64 is scarce on this GPU
        float2 *red = reinterpret_cast<float2 *>(smem);                        // [job][chunk][row]
        float *dj = reinterpret_cast<float *>(smem + (size_t)n_jobs * chunks * rows * 8u);  // [job][row]
        for (uint32_t t0 = tid; t0 < n_jobs * chunks * rows; t0 += 4u * kThreads) {
            float v[4][4];  // four tasks at a time, so that sixteen loads are in flight per thread
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                const uint32_t t = min(t0 + k * kThreads, n_jobs * chunks * rows - 1u);
                const uint32_t r = t % rows, jc = t / rows;  // jc = job * chunks + chunk: four slices of one job
                const float *p = part + (size_t)jc * 4u * hidden + n0 + r;
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) v[k][c] = __ldcg(p + (size_t)c * hidden);
            }
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                const uint32_t t = t0 + k * kThreads;
                float hi = v[k][0], lo = 0.0f, e;
#pragma unroll
                for (uint32_t c = 1; c < 4; ++c) {
                    two_sum(hi, v[k][c], hi, e);
                    lo = __fadd_rn(lo, e);
                }
                if (t < n_jobs * chunks * rows) red[t] = make_float2(hi, lo);
            }
        }
        __syncthreads();
        for (uint32_t t = tid; t < n_jobs * rows; t += kThreads) {
            const uint32_t r = t % rows, j = t / rows;
            float hi = 0.0f, lo = 0.0f, e;
            for (uint32_t c = 0; c < chunks; ++c) {  // slice order
                const float2 pr = red[((size_t)j * chunks + c) * rows + r];
                two_sum(hi, pr.x, hi, e);
                lo = __fadd_rn(lo, __fadd_rn(e, pr.y));
            }
            const float v = __fadd_rn(hi, lo);
            dj[t] = v;
            if (ep_on) {
                // the expert's rows of this CTA go to the route slot's row in every rank's slot buffer,
                // each value with the step's number in one 8-byte store
                const size_t at = ((size_t)(ep_step & 1u) * ep.n_slots + s_jobs[j].out_index) * hidden + n0 + r;
                const unsigned long long word = ((unsigned long long)(ep_step + 1u) << 32) | __float_as_uint(v);
                for (uint32_t p = 0; p < ep.world; ++p) st_relaxed_sys(ep.slots[p] + at, word);
            } else if (!y) {
                d_out[(size_t)s_jobs[j].out_index * hidden + n0 + r] = v;  // the caller mixes
            }
        }
        __syncthreads();
        if (ep_on) {
            // ---- exchange: rows [n0, n1) of every slot arrive in this rank's own buffer from the CTA of
            // the same number on the slot's owner; a thread polls (bounded) one word until it carries
            // this step's number, then the rows are mixed in route order, the shared expert last ----
            if (ep.wait_and_mix) {
                float *sv = dj;  // [slot][row]; the experts' sums are not needed any more
                for (uint32_t t = tid; t < ep.n_slots * rows; t += kThreads) {
                    const uint32_t r = t % rows, jj = t / rows;
                    const unsigned long long *w =
                        ep.slots[ep.rank] + ((size_t)(ep_step & 1u) * ep.n_slots + jj) * hidden + n0 + r;
                    unsigned long long got = ld_relaxed_sys(w);
                    uint32_t tries = 0;
                    // A word with an earlier step's number is waited for.  One with a LATER number means that a
                    // peer gave up on this rank and ran ahead: the words this rank still misses belong to
                    // steps its peers have left behind and would never come, so it reports that, waits for
                    // nothing more in this step and runs at full speed until it is level again.
                    while ((int32_t)((uint32_t)(got >> 32) - (ep_step + 1u)) < 0) {
                        if (s_behind) break;
                        if (++tries > ep.wait_limit || abort_flag) {
                            abort_flag = 1;
                            break;
                        }
                        __nanosleep(100);
                        got = ld_relaxed_sys(w);
                    }
                    if ((int32_t)((uint32_t)(got >> 32) - (ep_step + 1u)) > 0) {
                        s_behind = 1;
                        atomicExch(status, 0x5504u);
                    }
                    sv[t] = __uint_as_float((uint32_t)got);
                }
                __syncthreads();
                if (abort_flag) {
                    if (tid == 0) atomicExch(status, 0x5503u);
                } else if (y && tid < rows) {
                    float acc = 0.0f;
                    for (uint32_t jj = 0; jj < rt.top_k; ++jj)
                        acc = __fadd_rn(acc, __fmul_rn(s_route_w[jj], sv[jj * rows + tid]));
                    if (ep.n_slots > rt.top_k) acc = __fadd_rn(acc, sv[rt.top_k * rows + tid]);
                    y[n0 + tid] = acc;
                }
            }
        } else if (y && tid < rows) {
            float acc = 0.0f;
            for (uint32_t jj = 0; jj < n_jobs; ++jj) {
                const uint32_t jb = s_mix_job[jj];
                const float dv = dj[(size_t)(jb & 0x7FFFFFFFu) * rows + tid];
                acc = (jb >> 31) ? __fadd_rn(acc, dv) : __fadd_rn(acc, __fmul_rn(s_mix_w[jj], dv));
            }
            y[n0 + tid] = acc;
        }
    }
    // the last CTA to leave puts the counters back to zero for the next launch
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(counters + kExitCounter, 1u) == grid - 1u) {
            counters[kItemCounter] = 0u;
            counters[kExitCounter] = 0u;
            counters[kRouteCounter] = 0u;
            if (ep_on) *ep.step = ep_step + 1u;  // every CTA has read the count
        }
    }
}

size_t umma_smem_bytes(uint32_t hidden) { return (size_t)kRing * (kStageA + kStageSf) + (size_t)(hidden >> 8) * 2048u; }

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

size_t umma_partials_bytes() {
    // one F32 per (item, output row): experts of a token x slices x rows, at the largest shape
    return (size_t)(S14_EXPERTS_PER_TOKEN + 1) * (4096 / 64) * kMaxHidden * sizeof(float);
}

bool umma_layer_ok(int sm_count, uint32_t n_tokens, uint32_t n_jobs_max, uint32_t hidden, uint32_t inter) {
    if (n_tokens != 1u || n_jobs_max == 0u || n_jobs_max > S14_EXPERTS_PER_TOKEN + 1u) return false;
    if ((hidden & 511u) || (inter & 511u) || hidden < 512u || inter < 512u || hidden > kMaxHidden || inter > 4096u) return false;
    const uint32_t items = n_jobs_max * (inter >> 6);
    if ((items + (uint32_t)sm_count - 1u) / (uint32_t)sm_count > kItemSlots) return false;
    configure_once();
    // the final sums reuse the ring: [jobs][slices / 4][rows] doubles + [jobs][rows] floats
    const size_t rows = (hidden + sm_count - 1) / sm_count + 1;
    if ((size_t)n_jobs_max * ((inter >> 8) * 8u + 4u) * rows > (size_t)kRing * (kStageA + kStageSf)) return false;
    return umma_smem_bytes(hidden) <= g_dynamic_limit;
}

bool umma_router_ok(int sm_count, uint32_t n_experts) {
    return n_experts > 0u && n_experts <= kRouterSlots * (uint32_t)sm_count;
}

cudaError_t launch_moe_layer_umma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                                  const float *x, float *d, float *y, float *partials, unsigned int *counters,
                                  uint32_t *status, uint32_t hidden, uint32_t inter, bool after_router,
                                  const FusedRouter *router, const EpExchange *ep) {
    configure_once();
    FusedRouter rt = {};
    if (router) rt = *router;
    EpExchange ex = {};
    if (ep) ex = *ep;
    if (ex.world > 1u && !router) return cudaErrorInvalidValue;  // the mix needs every route's weight
    (void)after_router;
    // A programmatic dependent of the previous launch on the single-GPU path.  The expert-parallel
    // paths (exchange inside the kernel, or expert outputs handed to a collective) were measured as
    // ordinary launches only and stay so; the kernel's own dependency calls are then no-ops.
    return launch_pdl(k_moe_layer_umma, dim3(sm_count), dim3(kThreads), umma_smem_bytes(hidden), st, ex.world <= 1u && y != nullptr, dev, param, x, d, y, partials, counters, status, hidden, inter, rt, ex);
}

}  // namespace s14
