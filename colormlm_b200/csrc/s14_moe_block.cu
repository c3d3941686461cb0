// The MoE layer of a BLOCK of tokens (a verify block of up to 8 tokens, a prefill of hundreds) on
// the fifth-generation tensor cores, with the tokens grouped by expert so that an expert's page is
// streamed once for all the tokens routed to it.  Semantics: the reference's per-token layer loop
// (examples/s14_vulkan_numeric.rs:929-947) applied to every token of the block, which is all the
// reference's own prefill does (ssd_inference/src/forward.rs:544-549 walks the tokens one by one).
//
// The contraction is the one of the one-token layer kernel (s14_moe_umma.cu), widened along N:
// tcgen05.mma kind::mxf4.block_scale with A = 128 weight rows x 64 K-elements of page bytes as they
// are, and B = the sixteen balanced base-8 digit rows of EVERY token of a chunk (up to kBlockNt tokens
// that share the expert: N = 16 * tokens).  Accumulator columns 16 t .. 16 t + 15 hold the digit
// shares of token t's dot products; added in double and rounded once they give the double-accumulated
// dot product rounded to F32, so every token's result is bit-identical to what the one-token kernel
// and the double-accumulating CPU restatement give for that token alone.
//
// Five or six launches per layer, all plain stream order (the routed calls run the router's two launches first):
//   k_block_digits   x [T, hidden] -> digit tiles (2 KB per token and 256 elements) + block exponents
//   k_block_group    routes [T, top_k] -> chunks (expert page, <= nt_cap tokens: 2 for small blocks, else 6 or
//                    12); an item index decodes to (chunk, slice or row tile) from the chunk records
//   k_block_gemm<0>  up items (chunk, one or two slices of 64 intermediate elements): w1 | w3 units x the
//                    chunk's token tiles; epilogue: limited SwiGLU, then either the digit tiles of the hidden
//                    values per (token, route) pair (small blocks) or the hidden values themselves, whose
//                    digit tiles a second k_block_digits launch over the pairs lays out (larger blocks)
//   k_block_gemm<1>  down items (chunk, one or two tiles of 128 rows of w2) x the pairs' digit tiles -> the
//                    pairs' expert outputs [pair, hidden] (expert parallel: into every rank's pair buffer)
//   k_block_mix      per token the ordered mix: routes in order, shared expert last (expert parallel: after
//                    every rank's rows have arrived)
// Items are dealt round robin to one persistent CTA per SM, the chunks of one expert next to each
// other, so that the second and later chunks of an expert find its units in the L2.
//
// Roles inside a GEMM CTA: all threads decode the CTA's items of a batch into shared-memory records; one
// copying thread (the units of 17 KB page bytes of a ring stage: plain bulk copies, no multicast), two
// MMA-issuing threads (even and odd stages of an item, accumulators of their own), four epilogue warps, eight
// warps that lay out the digit rows' scale codes of an item in shared memory (tcgen05.cp brings them to
// tensor memory stage by stage, like the weights' scales) and then, for large blocks, fetch the chunk's token
// tiles of every stage (cp.async, 16 bytes a thread; for small blocks a second copying thread brings them by
// bulk copies).  What bounds the kernels is the number of bytes an SM takes in (45-50 GB/s per SM, whether
// from memory or from the L2), so a large block takes TWO slices or row tiles per item: the token tiles of a
// K range are fetched once for two units.  With the official expert arithmetic
// (fast16/research/polaris_meridian_v1/s14_first_real_token/executor.py:712-743) the same contractions run on
// quantised inputs: k_block_digits quantises per 128 elements to E4M3FN values (which the digit rows hold
// exactly), the up epilogue works on BF16 gate and up and multiplies by the route weight, the down epilogue
// and the mix round to BF16.  Every wait is bounded; a wait that runs out raises the CTA's abort
// flag, the status word is set, and the CTA waits for its copies in flight, frees its tensor memory and returns.
#include "s14_umma.cuh"

namespace s14 {

namespace {

constexpr uint32_t kNt = kBlockNt;          // most tokens of a chunk
constexpr uint32_t kNtHalf = 6;             // tokens of one MMA: N = 96 accumulator columns
constexpr uint32_t kAccCols = 16u * kNtHalf;
static_assert(kNt == 2u * kNtHalf, "a wide chunk is two halves, one per issuing thread");
constexpr uint32_t kStageA = kUnitStride;                  // a unit's codes, then its scales
// a ring stage: a unit, then the token tiles (2 KB each) of the unit's K range for as many tokens as a chunk may hold
static_assert(kStageA % 1024u == 0u && 2048u % 1024u == 0u, "operand tiles keep the 1 KB alignment of the 128-byte swizzle");
constexpr uint32_t kGThreads = 512;
constexpr uint32_t kGRingMax = 12;
constexpr uint32_t kSfbBytes = 16u * 1024u;                // an item's digit-row scale atoms: K / 256 units x 1 KB, K <= 4096
constexpr uint32_t kGProdWarp = 4, kGMmaWarp0 = 5, kGTileWarp = 7, kGLayWarp0 = 8;
constexpr uint32_t kGLayThreads = 256;
// tensor memory columns
constexpr uint32_t kGColAcc = 0;                           // [2 buffers or 2 row tiles][2 issuing threads][kAccCols]
constexpr uint32_t kGColSfa = 4u * kAccCols;              // [2 issuing threads][16]: weight scales of the unit at hand
constexpr uint32_t kGColSfb = kGColSfa + 32u;              // [2 issuing threads][16]: digit-row scales of that unit
static_assert(kGColSfb + 32u <= 512u, "tensor memory map");
// barriers
constexpr uint32_t kGBarFull = 0;
constexpr uint32_t kGBarDone = kGRingMax;
constexpr uint32_t kGBarAccDone = 2 * kGRingMax;           // [2] an item's accumulators are complete (both issuing threads)
constexpr uint32_t kGBarAccFree = kGBarAccDone + 2;        // [2] ... have been read
constexpr uint32_t kGBarSfb = kGBarAccFree + 2;            // [2] an item's digit-row scales are laid out
constexpr uint32_t kGBarFin = kGBarSfb + 2;
constexpr uint32_t kGBars = kGBarFin + 1;
constexpr uint32_t kPairsPerToken = S14_EXPERTS_PER_TOKEN + 1;   // pair = token * 7 + position in the mix (6: shared)

// What the up kernel's epilogue leaves (the down kernel: kModeOfficial rounds its rows to BF16, the others do not)
constexpr uint32_t kModeFused = 0u;      // the digit rows of the hidden values, laid out by the epilogue itself (small blocks)
constexpr uint32_t kModeOfficial = 1u;   // the official arithmetic's BF16 hidden values, times the route weight
constexpr uint32_t kModeValues = 2u;     // the F32 hidden values; a digits launch follows (large blocks)

struct GemmArgs {
    const BlockChunk *chunks;
    const uint32_t *n_items;    // device memory: written by the grouping kernel (chunks x slices or row tiles)
    const uint8_t *dig;         // digit tiles of the B vectors [vector][K / 256][2048]
    const uint8_t *exps;        // their block exponents + 100, [vector][K / 32]
    float *out;                 // down: the pairs' expert outputs [pair][hidden]
    uint8_t *hdig, *hexp;       // up: digit tiles and exponents of the pairs' hidden values
    uint32_t by_threads;        // the token tiles come by the tile threads' own copies (large blocks), else by bulk copies
    uint32_t hidden, inter, ring, stage;   // stage: bytes of a ring stage (a unit and nt_cap token tiles)
    // Expert parallel with the exchange inside the kernel: the pairs' outputs go into every rank's buffer
    // (plain stores to peer memory), and the last CTA to finish tells every rank that this rank's rows of
    // call `ep_call` are there (flags[rank] of the call's parity in every rank's buffer).
    float *out_peer[kMaxEpWorld];
    unsigned long long *flag_peer[kMaxEpWorld];
    unsigned int *ep_counter;   // this GPU's arrival counter, zero at rest
    uint32_t ep_world, ep_rank, ep_call;
    // Up kernel, kModeOfficial / kModeValues: the pairs' hidden values [pair][inter] (official: weighted and
    // BF16-valued) and, for the official arithmetic, the routes' weights [token][top_k]
    float *hval;
    const float *weights;
    uint32_t top_k;
};

// torch's .to(torch.bfloat16).float()
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// The nearest E4M3FN value (ties to even) of |v| <= 448: three mantissa bits; below 2^-6 multiples of 2^-9.
__device__ __forceinline__ float e4m3fn_round(float v) {
    const float a = fabsf(v);
    float q;
    if (a < 0.015625f) {
        q = __fmul_rn(rintf(__fmul_rn(a, 512.0f)), 0.001953125f);
    } else {
        const int e = (int)(__float_as_uint(a) >> 23) - 127;   // floor(log2 a)
        q = __fmul_rn(rintf(__fmul_rn(a, __uint_as_float((uint32_t)(130 - e) << 23))), __uint_as_float((uint32_t)(124 + e) << 23));
    }
    return copysignf(q, v);
}

// The digit tiles and block exponents of n vectors of K elements (one CTA per vector).  With `quant` the
// vector is first quantised as the official linears quantise their input
// (l42_real_reference/l42_reference.py:389-403): per 128 elements amax = max(|x|, 1e-4), scale =
// 2^ceil(log2(amax / 448)) (F32 quotient, the logarithm taken in double and rounded to F32), x / scale
// clipped to +-448, rounded to E4M3FN, times the scale.  The quantised values are F32 values with four
// significant bits, which the digit rows hold exactly.
__global__ void __launch_bounds__(512)
k_block_digits(const float *__restrict__ x, uint32_t K, uint8_t *__restrict__ dig, uint8_t *__restrict__ exps, uint32_t quant) {
    const uint32_t v = blockIdx.x, g = threadIdx.x;
    if (g >= (K >> 3)) return;  // whole warps leave: K is a multiple of 256
    const float4 p0 = __ldg(reinterpret_cast<const float4 *>(x + (size_t)v * K) + 2u * g);
    const float4 p1 = __ldg(reinterpret_cast<const float4 *>(x + (size_t)v * K) + 2u * g + 1u);
    float xs[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    if (quant) {
        // a group of 128 elements is sixteen neighbouring threads
        float am = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(xs[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        am = fmaxf(am, 1e-4f);
        int e = (int)ceilf((float)log2((double)__fdiv_rn(am, 448.0f)));
        e = e < -126 ? -126 : (e > 126 ? 126 : e);
        const float scale = __uint_as_float((uint32_t)(127 + e) << 23), inv = __uint_as_float((uint32_t)(127 - e) << 23);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            xs[i] = __fmul_rn(e4m3fn_round(fminf(fmaxf(__fmul_rn(xs[i], inv), -448.0f), 448.0f)), scale);
    }
    digits_of8(xs, g, dig + (size_t)v * (K >> 8) * 2048u, exps + (size_t)v * (K >> 5));
}

// Groups the block's (token, route) pairs by expert.  Group 0 is the shared expert (every token, mix
// position 6), group 1 + e the routed expert e; a group's members are cut into chunks of nt_cap (the
// shared expert's in token order, a routed expert's in the order its members arrive: every pair's
// result depends on that pair alone, so the order changes no bit of the output).  ids: [T, top_k]
// expert ids, negative = no route.  The page of a routed group is page_table[e], or, with per-route
// pages, the page of one of its members.  counts: [0] chunks, [1] up items, [2] down items, [3] 1 if
// an id was out of range (then no chunk is made).  One CTA of 1024 threads.
__global__ void __launch_bounds__(1024)
k_block_group(const int32_t *__restrict__ ids, const uint8_t *const *__restrict__ pages,
              const uint8_t *const *__restrict__ page_table, const uint8_t *shared_page, uint32_t T, uint32_t top_k,
              uint32_t n_experts, uint32_t S, uint32_t RT, uint32_t nt_cap, BlockChunk *__restrict__ chunks,
              uint32_t *__restrict__ counts, uint32_t ep_rank, uint32_t ep_world, uint32_t shared_by_token) {
    constexpr uint32_t kG = S14_N_ROUTED_EXPERTS + 1;
    __shared__ uint32_t cnt[kG], fill[kG], chunk0[kG + 1];
    __shared__ unsigned long long gpage[kG];
    __shared__ uint32_t bad;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, G = n_experts + 1u, n = T * top_k;
    if (tid < kG) {
        cnt[tid] = 0u;
        fill[tid] = 0u;
        gpage[tid] = tid == 0u ? (unsigned long long)shared_page
                               : ((page_table && tid < G) ? (unsigned long long)page_table[tid - 1u] : 0ull);
    }
    if (tid == 0) bad = 0u;
    __syncthreads();
    for (uint32_t i = tid; i < n; i += blockDim.x) {
        const int32_t e = __ldg(ids + i);
        if (e >= (int32_t)n_experts) bad = 1u;
        else if (e >= 0 && (uint32_t)e % ep_world == ep_rank) atomicAdd(&cnt[1 + e], 1u);  // expert parallel: the experts this rank owns
    }
    // the shared expert's members: every token; expert parallel with the shared page on every rank: the tokens
    // t with t mod world == rank (its work is a fifth of a large block's: on one rank it would bound the scaling)
    const uint32_t sh_step = shared_by_token ? ep_world : 1u, sh_first = shared_by_token ? ep_rank : 0u;
    if (tid == 0 && shared_page) cnt[0] = T > sh_first ? (T - sh_first + sh_step - 1u) / sh_step : 0u;
    __syncthreads();
    if (tid < 32u) {
        // exclusive scan of the groups' chunk counts: nine groups per lane
        constexpr uint32_t kPer = (kG + 31u) / 32u;
        uint32_t mine = 0;
        for (uint32_t k = 0; k < kPer; ++k) {
            const uint32_t g = lane * kPer + k;
            if (g < G) mine += (cnt[g] + nt_cap - 1u) / nt_cap;
        }
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
            if ((int)lane >= o) incl += v;
        }
        uint32_t c = incl - mine;
        for (uint32_t k = 0; k < kPer; ++k) {
            const uint32_t g = lane * kPer + k;
            if (g < G) {
                chunk0[g] = c;
                c += (cnt[g] + nt_cap - 1u) / nt_cap;
            }
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        if (lane == 0) {
            chunk0[G] = total;
            const uint32_t c_all = bad ? 0u : total;  // with a bad id the contraction kernels find no item, the mix writes nothing
            counts[0] = c_all;
            counts[1] = c_all * S;
            counts[2] = c_all * RT;
            counts[3] = bad;
        }
    }
    __syncthreads();
    if (bad) return;
    for (uint32_t i = tid; i < n; i += blockDim.x) {
        const int32_t e = __ldg(ids + i);
        if (e < 0 || (uint32_t)e % ep_world != ep_rank) continue;
        const uint32_t g = 1u + (uint32_t)e, t = i / top_k, m = i - t * top_k;
        const uint32_t k = atomicAdd(&fill[g], 1u);
        if (k == 0u && !page_table) gpage[g] = (unsigned long long)pages[i];
        BlockChunk *ch = chunks + chunk0[g] + k / nt_cap;
        ch->tok[k % nt_cap] = t;
        ch->pair[k % nt_cap] = t * kPairsPerToken + m;
    }
    if (shared_page) {
        for (uint32_t k = tid; sh_first + k * sh_step < T; k += blockDim.x) {
            const uint32_t t = sh_first + k * sh_step;
            BlockChunk *ch = chunks + chunk0[0] + k / nt_cap;
            ch->tok[k % nt_cap] = t;
            ch->pair[k % nt_cap] = t * kPairsPerToken + S14_EXPERTS_PER_TOKEN;
        }
    }
    __syncthreads();
    const uint32_t total = chunk0[G];
    for (uint32_t c = tid; c < total; c += blockDim.x) {
        // the chunk's group: the last g with chunk0[g] <= c
        uint32_t lo = 0, hi = G;
        while (hi - lo > 1u) {
            const uint32_t mid = (lo + hi) >> 1;
            if (chunk0[mid] <= c) lo = mid;
            else hi = mid;
        }
        const uint32_t g = lo, c0 = chunk0[g], nch = chunk0[g + 1u] - c0;
        BlockChunk *ch = chunks + c;
        ch->page = reinterpret_cast<const uint8_t *>(gpage[g]);
        ch->nt = c + 1u < c0 + nch ? nt_cap : cnt[g] - (c - c0) * nt_cap;
        ch->c0 = c0;
        ch->nch = nch;
    }
}

// An item as the CTA's roles read it, decoded once per batch into shared memory.
struct ItemRec {
    unsigned long long page;
    uint32_t nt, r;            // pairs of the chunk; slice (up) or row tile (down)
    uint32_t tok[kNt];
    uint32_t pair[kNt];
};
// kMt: row tiles (slices of the up phase) per item.
//   1 (small blocks): chunks of up to six tokens (the host uses two); the two issuing threads take the even and
//     the odd units of an item, each into an accumulator of its own, and items alternate between two
//     accumulator buffers, so that an item's epilogue runs under the next item's MMAs.
//   2 (larger blocks): the chunk's token tiles of a K range are fetched once for two units of page bytes (a
//     stage holds both units, then the tiles): half the tile bytes, and what an SM takes in is what bounds
//     these kernels.  Every issuing thread holds an accumulator per row tile and there is no second accumulator
//     buffer (the next item's MMAs wait until the epilogue has read the accumulators, while the ring keeps filling).
//     kWide (many tokens per expert): a chunk holds up to TWELVE tokens; issuing thread m takes the tokens
//     6 m .. 6 m + 5 (its own rows of the tile region, its own scale atoms, N = 96) for EVERY stage: fewer
//     passes over an expert's page.  Otherwise chunks of six and even / odd stages as with one row tile.
template <bool kDown, uint32_t kMt, bool kWide, uint32_t kMode>
__global__ void __launch_bounds__(kGThreads, 1)
k_block_gemm(const __grid_constant__ GemmArgs a, uint32_t *status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[kGBars];
    constexpr uint32_t kTok = kWide ? kNt : kNtHalf;   // most tokens of a chunk in this shape
    constexpr uint32_t kBatch = kWide ? 96u : 48u;     // items decoded at a time (the records share the static shared memory with the ring)
    __shared__ __align__(16) ItemRec s_rec[kBatch];
    __shared__ float s_up[kTok][64];                          // an item's up projections (even tokens) and gates (odd tokens), handed across
    __shared__ __align__(16) uint8_t s_hst[kTok][16 * 2 * 16]; // an up item's digit chunks per token: [row][block][16 bytes]
    __shared__ uint32_t tmem_slot, s_units;
    __shared__ int abort_flag;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t grid = gridDim.x, cta = blockIdx.x;
    const uint32_t K = kDown ? a.inter : a.hidden;
    const uint32_t nu = K >> 8;                      // units of an item
    const uint32_t KD = a.inter >> 8;
    const uint32_t ring = a.ring;
    uint8_t *const sRing = smem;
    uint8_t *const sSfb = smem + ring * a.stage;     // [2][kSfbBytes]
    const size_t page_off = kDown ? mxfp4_down_offset(a.hidden, a.inter) : 0u;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](uint32_t i) { return bar0 + i * 8u; };
    volatile int *const abortp = &abort_flag;

    if (tid < kGBars) {
        uint32_t count = 1u;
        if (tid < kGRingMax) count = a.by_threads ? 1u + kGLayThreads : 1u;   // a stage: the page copy's arrival (and the tile threads' copies)
        else if (tid >= kGBarDone && tid < kGBarDone + kGRingMax) count = kWide ? 2u : 1u;   // wide chunks: both issuing threads read every stage
        else if (tid >= kGBarAccDone && tid < kGBarAccDone + 2u) count = 2u;
        else if (tid >= kGBarAccFree && tid < kGBarAccFree + 2u) count = 128u;
        else if (tid >= kGBarSfb && tid < kGBarSfb + 2u) count = kGLayThreads;
        else if (tid == kGBarFin) count = 2u;
        mbar_init(bar(tid), count);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid == 0) {
        abort_flag = 0;
        s_units = 0;
    }
    if (warp == kGMmaWarp0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        fence_before();
    }
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t n_items = __ldcg(a.n_items);
    // The CTA's items are q = cta, cta + grid, ...  The chunks of one expert follow one another and so
    // do their items, a row tile's chunks side by side (so that CTAs that run at the same time share
    // the expert's units in the L2).
    const uint32_t R = (kDown ? (a.hidden >> 7) : (a.inter >> 6)) / kMt;   // items per chunk
    const uint32_t n_local = n_items > cta ? (n_items - cta + grid - 1u) / grid : 0u;

    const bool is_prod_a = tid == kGProdWarp * 32u, is_prod_b = tid == kGTileWarp * 32u && !a.by_threads;
    const bool is_issuer = (warp == kGMmaWarp0 || warp == kGMmaWarp0 + 1u) && lane == 0;
    // what the roles carry from item to item
    uint32_t p_slot = 0, p_round = 0, p_units = 0;             // the copying threads: next stage
    uint32_t m_slot = kWide ? 0u : warp - kGMmaWarp0, m_round = 0;   // the issuing threads: their next stage
    uint32_t gi = 0;                                           // items so far
    bool ok = true;
    const unsigned long long once = l2_policy_evict_first();

#pragma unroll 1
    for (uint32_t base = 0; base < n_local; base += kBatch) {
        const uint32_t nb = n_local - base < kBatch ? n_local - base : kBatch;
        // ---- the batch's items into shared memory: every thread decodes one (two dependent loads and
        // the chunk's record, all threads' in flight together), so that no role waits for global
        // memory at an item's start ----
        for (uint32_t i = tid; i < nb; i += kGThreads) {
            const uint32_t q = cta + (base + i) * grid;
            const BlockChunk *g = a.chunks + q / R;
            const uint32_t c0 = __ldg(&g->c0), nch = __ldg(&g->nch), j = q - c0 * R;
            const uint32_t r = j / nch;
            const BlockChunk *ch = a.chunks + c0 + (j - r * nch);
            ItemRec rec;
            rec.page = __ldg(reinterpret_cast<const unsigned long long *>(&ch->page));
            rec.nt = __ldg(&ch->nt) | (nch > 1u ? 0x100u : 0u);
            rec.r = r;
#pragma unroll
            for (uint32_t t = 0; t < kNt; ++t) {
                rec.tok[t] = __ldg(&ch->tok[t]);
                rec.pair[t] = __ldg(&ch->pair[t]);
            }
            s_rec[i] = rec;
        }
        __syncthreads();

        if (is_prod_a) {
            // ---- the copying thread of the pages: per unit of every item one ring stage (a bulk copy of
            // 17 KB of page bytes, counted in bytes on the stage's barrier) ----
#pragma unroll 1
            for (uint32_t i = 0; i < nb && ok; ++i) {
                const uint32_t multi = s_rec[i].nt >> 8;
                const uint8_t *src = reinterpret_cast<const uint8_t *>(s_rec[i].page) + page_off +
                                     (size_t)s_rec[i].r * kMt * nu * kUnitStride;
#pragma unroll 1
                for (uint32_t u = 0; u < nu; ++u) {
                    if (p_round && !mbar_wait(bar(kGBarDone + p_slot), (p_round - 1u) & 1u, abortp)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar(kGBarFull + p_slot), dst = smem_u32(sRing) + p_slot * a.stage;
                    mbar_arrive_expect(full, kMt * kStageA + (a.by_threads ? 0u : (s_rec[i].nt & 0xFFu) * 2048u));
                    // an expert with one chunk is read once; with more, its later chunks want the units in the L2
#pragma unroll
                    for (uint32_t mt = 0; mt < kMt; ++mt) {
                        if (multi) bulk_copy(dst + mt * kStageA, src + (size_t)mt * nu * kUnitStride, kStageA, full);
                        else bulk_copy_stream(dst + mt * kStageA, src + (size_t)mt * nu * kUnitStride, kStageA, full, once);
                    }
                    src += kUnitStride;
                    ++p_units;
                    if (++p_slot == ring) {
                        p_slot = 0;
                        ++p_round;
                    }
                }
            }
            s_units = p_units;
        } else if (is_prod_b) {
            // ---- small blocks: a second copying thread brings the chunk's token tiles of the unit's K range
            // behind the unit by bulk copies, counted on the same barrier (bytes that land before the barrier
            // is armed are counted all the same) ----
#pragma unroll 1
            for (uint32_t i = 0; i < nb && ok; ++i) {
                const uint32_t nt = s_rec[i].nt & 0xFFu;
                uint32_t vec[kNtHalf];   // (small blocks: chunks of up to six tokens)
#pragma unroll
                for (uint32_t t = 0; t < kNtHalf; ++t) vec[t] = kDown ? s_rec[i].pair[t] : s_rec[i].tok[t];
#pragma unroll 1
                for (uint32_t u = 0; u < nu; ++u) {
                    if (p_round && !mbar_wait(bar(kGBarDone + p_slot), (p_round - 1u) & 1u, abortp)) {
                        ok = false;
                        break;
                    }
                    const uint32_t full = bar(kGBarFull + p_slot), dst = smem_u32(sRing) + p_slot * a.stage + kMt * kStageA;
#pragma unroll
                    for (uint32_t t = 0; t < kNtHalf; ++t)
                        if (t < nt) bulk_copy(dst + t * 2048u, a.dig + ((size_t)vec[t] * nu + u) * 2048u, 2048u, full);
                    if (++p_slot == ring) {
                        p_slot = 0;
                        ++p_round;
                    }
                }
            }
        } else if (is_issuer) {
            // ---- MMA issue.  One row tile per item: thread m takes units m, m + 2, ... of every item (a ring slot
            // always belongs to the same thread: items have an even number of units and the ring an even number
            // of slots).  Two row tiles: thread m takes EVERY stage for its half of the chunk's tokens. ----
            const uint32_t m = warp - kGMmaWarp0;
            constexpr uint32_t kStep = kWide ? 1u : 2u;
            const uint64_t a_desc0 = smem_desc(smem_u32(sRing), 1, 64, 2);
            const uint64_t sf_desc0 = smem_desc(smem_u32(sRing) + kUnitBytes, 0, 8, 0);
            const uint64_t b_desc0 = smem_desc(smem_u32(sRing) + kMt * kStageA + (kWide ? m * kNtHalf * 2048u : 0u), 1, 64, 2);
            const uint32_t sfa_t = tmem + kGColSfa + m * 16u, sfb_t = tmem + kGColSfb + m * 16u;
#pragma unroll 1
            for (uint32_t i = 0; i < nb && ok; ++i, ++gi) {
                const uint32_t buf = gi & 1u, nt_all = s_rec[i].nt & 0xFFu;
                const uint32_t nt_m = !kWide ? nt_all
                                             : (m == 0u ? (nt_all < kNtHalf ? nt_all : kNtHalf) : (nt_all > kNtHalf ? nt_all - kNtHalf : 0u));
                const uint32_t idesc = umma_idesc_mxf4(16u * (nt_m ? nt_m : 1u));
                // one row tile per item: the accumulators of item gi - 2 have been read; two: those of item gi - 1
                if (kMt == 1u) {
                    if (gi >= 2u) ok = mbar_wait(bar(kGBarAccFree + buf), ((gi - 2u) >> 1) & 1u, abortp);
                } else if (gi >= 1u) {
                    ok = mbar_wait(bar(kGBarAccFree + ((gi - 1u) & 1u)), ((gi - 1u) >> 1) & 1u, abortp);
                }
                ok = ok && mbar_wait(bar(kGBarSfb + buf), (gi >> 1) & 1u, abortp);
                if (!ok) break;
                fence_after();
                const uint32_t acc = tmem + kGColAcc + ((kMt == 1u ? buf : 0u) * 2u + m) * kAccCols;   // row tile mt: + 2 * mt accumulators
                // the scale atoms of the item's digit rows: one buffer per item parity, or (wide chunks) per half
                const uint64_t sfb_desc0 = smem_desc(smem_u32(sSfb) + (kWide ? m : buf) * kSfbBytes, 0, 8, 0);
#pragma unroll 1
                for (uint32_t ku = kWide ? 0u : m; ku < nu; ku += kStep) {
                    const uint32_t s = m_slot;
                    ok = mbar_wait(bar(kGBarFull + s), m_round & 1u, abortp);
                    if (!ok) break;
                    m_slot += kStep;
                    if (m_slot >= ring) {
                        m_slot -= ring;
                        ++m_round;
                    }
                    if (nt_m) {
                        fence_async_smem();  // the token tiles came by the threads' own copies: the tensor cores read them
                        fence_after();
                        const uint64_t sfd = sf_desc0 + s * (a.stage >> 4), sbd = sfb_desc0 + ku * (1024u >> 4);
#pragma unroll
                        for (uint32_t mt = 0; mt < kMt; ++mt) {
                            tmem_copy_scales(sfa_t + mt * 8u, sfd + mt * (kStageA >> 4));
                            tmem_copy_scales(sfa_t + mt * 8u + 4u, sfd + mt * (kStageA >> 4) + (kAtomBytes >> 4));
                        }
                        tmem_copy_scales(sfb_t, sbd);
                        tmem_copy_scales(sfb_t + 4u, sbd + (kAtomBytes >> 4));
                        const uint64_t ad = a_desc0 + s * (a.stage >> 4), bd = b_desc0 + s * (a.stage >> 4);
#pragma unroll
                        for (uint32_t mt = 0; mt < kMt; ++mt) {
#pragma unroll
                            for (uint32_t kk = 0; kk < 4; ++kk) {
                                const uint32_t atom = kk >> 1, sfid = (kk & 1u) * 2u;
                                umma_mxf4(acc + mt * 2u * kAccCols, ad + mt * (kStageA >> 4) + kk * 2u, bd + kk * 2u,
                                          idesc | (sfid << 29) | (sfid << 4), (sfa_t + mt * 8u + atom * 4u) | (sfid << 30),
                                          (sfb_t + atom * 4u) | (sfid << 30), (ku >= kStep || kk) ? 1u : 0u);
                            }
                        }
                    }
                    umma_commit(bar(kGBarDone + s));
                }
                if (!ok) break;
                umma_commit(bar(kGBarAccDone + buf));
            }
        } else if (warp < 4u) {
            // ---- epilogue: per token of the chunk the two accumulators' sixteen digit columns, added in
            // double and rounded once ----
            const uint32_t row = tid;
            const uint32_t lane_base = tmem + ((warp * 32u) << 16);
#pragma unroll 1
            for (uint32_t i = 0; i < nb && ok; ++i, ++gi) {
                const uint32_t idx0 = s_rec[i].r, buf = gi & 1u, nt = s_rec[i].nt & 0xFFu;
                const uint32_t *pair = s_rec[i].pair;
                ok = epi_all(mbar_wait(bar(kGBarAccDone + buf), (gi >> 1) & 1u, abortp));
                if (!ok) break;
                fence_after();
                float v[kMt][kTok];
                // two loads of sixteen columns in flight per wait: the two issuing threads' accumulators of one token
                // (even and odd stages), or, in wide chunks, two neighbouring tokens of the half that holds them
#pragma unroll
                for (uint32_t mt = 0; mt < kMt; ++mt) {
#pragma unroll
                    for (uint32_t t = 0; t < kTok; t += (kWide ? 2u : 1u)) {
                        v[mt][t] = 0.0f;
                        if (kWide) v[mt][t + (kWide ? 1u : 0u)] = 0.0f;
                        if (t < nt) {  // uniform in the CTA
                            uint32_t r0[16], r1[16];
                            const uint32_t col0 = kWide ? (mt * 2u + t / kNtHalf) * kAccCols + 16u * (t % kNtHalf)
                                                        : ((kMt == 1u ? buf : mt) * 2u) * kAccCols + 16u * t;
                            const uint32_t col1 = kWide ? col0 + 16u : col0 + kAccCols;
                            tmem_ld16(lane_base + kGColAcc + col0, r0);
                            tmem_ld16(lane_base + kGColAcc + col1, r1);
                            tmem_ld_wait();
                            double lo0 = 0.0, hi0 = 0.0, lo1 = 0.0, hi1 = 0.0;
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                lo0 += (double)__uint_as_float(r0[8 + c]);
                                hi0 += (double)__uint_as_float(r0[c]);
                                lo1 += (double)__uint_as_float(r1[8 + c]);
                                hi1 += (double)__uint_as_float(r1[c]);
                            }
                            if (kWide) {
                                v[mt][t] = (float)(lo0 + hi0);
                                v[mt][t + (kWide ? 1u : 0u)] = (float)(lo1 + hi1);  // unused beyond nt
                            } else {
                                v[mt][t] = (float)((lo0 + hi0) + (lo1 + hi1));
                            }
                        }
                    }
                }
                fence_before();
                mbar_arrive(bar(kGBarAccFree + buf));
#pragma unroll
                for (uint32_t mt = 0; mt < kMt; ++mt) {
                    const uint32_t idx = idx0 * kMt + mt;   // the slice (up) or row tile (down)
                    if constexpr (kDown) {
                        // row idx * 128 + `row` of the pairs' expert outputs
#pragma unroll
                        for (uint32_t t = 0; t < kTok; ++t) {
                            if (t < nt) {
                                const size_t at = (size_t)pair[t] * a.hidden + idx * 128u + row;
                                const float o = kMode == kModeOfficial ? bf16_round(v[mt][t]) : v[mt][t];   // official: a linear's result is BF16
                                if (a.ep_world > 1u) {
#pragma unroll 1
                                    for (uint32_t p = 0; p < a.ep_world; ++p) a.out_peer[p][at] = o;
                                } else {
                                    a.out[at] = o;
                                }
                            }
                        }
                    } else {
                        // threads 0-63: gate of the slice's element `row`; threads 64-127: the up projection of
                        // element row - 64.  The first half works out the even tokens, the second the odd ones:
                        // each hands the other the values it lacks
                        const uint32_t el = row & 63u, par = row >> 6, blk2 = warp & 1u;
                        if (mt) epi_sync();  // the row tile before has been written out
                        if constexpr (kMode != kModeFused) {
                            // The hidden values go out as F32 values; their digit rows are the next launch's
                            // (large blocks: this epilogue then costs a third of the one that lays out the digit
                            // rows itself, and it is what the MMAs of the next item wait for).  Official
                            // arithmetic (s14_first_real_token/executor.py:712-743): gate and up rounded to BF16,
                            // the limited SwiGLU in F32, times the route's weight (not for the shared expert),
                            // rounded to BF16; the next launch also quantises them per 128 elements.
                            constexpr bool kOff = kMode == kModeOfficial;
#pragma unroll
                            for (uint32_t t = 0; t < kTok; ++t)
                                if (t < nt && (t & 1u) != par) s_up[t][el] = kOff ? bf16_round(v[mt][t]) : v[mt][t];
                            epi_sync();
#pragma unroll
                            for (uint32_t t = 0; t < kTok; ++t) {
                                if (t < nt && (t & 1u) == par) {
                                    const float other = s_up[t][el], mine = kOff ? bf16_round(v[mt][t]) : v[mt][t];
                                    const float hv = par ? swiglu_limit_f32(other, mine) : swiglu_limit_f32(mine, other);
                                    const uint32_t pr = pair[t];
                                    float wh = hv;
                                    if constexpr (kOff) {
                                        const uint32_t tok = pr / kPairsPerToken, pos = pr - tok * kPairsPerToken;
                                        if (pos < S14_EXPERTS_PER_TOKEN) wh = __fmul_rn(hv, __ldg(a.weights + tok * a.top_k + pos));
                                        wh = bf16_round(wh);
                                    }
                                    a.hval[(size_t)pr * a.inter + idx * 64u + el] = wh;
                                }
                            }
                        }
                        if constexpr (kMode == kModeFused) {
#pragma unroll
                        for (uint32_t t = 0; t < kTok; ++t)
                            if (t < nt && (t & 1u) != par) s_up[t][el] = v[mt][t];
                        epi_sync();
#pragma unroll
                        for (uint32_t t = 0; t < kTok; ++t) {
                            if (t < nt && (t & 1u) == par) {
                                // hidden value `el` of the slice -> sixteen digit nibbles; scale block = warp % 2
                                const float other = s_up[t][el];
                                const float hv = par ? swiglu_limit_f32(other, v[mt][t]) : swiglu_limit_f32(v[mt][t], other);
                                float bm = fabsf(hv);
#pragma unroll
                                for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
                                const int E = block_exponent(bm);
                                uint32_t hw, lw;
                                digit_codes16(hv, __uint_as_float((uint32_t)(150 - E) << 23), hw, lw);
                                const uint32_t ohw = __shfl_xor_sync(0xffffffffu, hw, 1), olw = __shfl_xor_sync(0xffffffffu, lw, 1);
                                // byte lane / 2 of every row's chunk holds the nibbles of lanes 2b (low) and 2b + 1; even
                                // lanes write digit rows 0-3 and 8-11, odd lanes 4-7 and 12-15
                                const uint32_t e_hw = (lane & 1u) ? ohw : hw, o_hw = (lane & 1u) ? hw : ohw;
                                const uint32_t e_lw = (lane & 1u) ? olw : lw, o_lw = (lane & 1u) ? lw : olw;
#pragma unroll
                                for (uint32_t jj = 0; jj < 4; ++jj) {
                                    const uint32_t dj = (lane & 1u) * 4u + jj;
                                    s_hst[t][(dj * 2u + blk2) * 16u + (lane >> 1)] =
                                        (uint8_t)(((e_hw >> (4u * dj)) & 0xFu) | (((o_hw >> (4u * dj)) & 0xFu) << 4));
                                    s_hst[t][((8u + dj) * 2u + blk2) * 16u + (lane >> 1)] =
                                        (uint8_t)(((e_lw >> (4u * dj)) & 0xFu) | (((o_lw >> (4u * dj)) & 0xFu) << 4));
                                }
                                if (lane == 0) a.hexp[(size_t)pair[t] * (a.inter >> 5) + idx * 2u + blk2] = (uint8_t)(E + 100);
                            }
                        }
                        epi_sync();
                        // the slice's 32 chunks (digit row, block) of every token go to their places in the pair's
                        // digit tile: 64 threads write half a chunk each; the two halves of the CTA take the
                        // tokens alternately
                        const uint32_t t64 = tid & 63u, ch16 = t64 >> 1, half = t64 & 1u, dj = ch16 >> 1, blk = ch16 & 1u;
                        const uint32_t cc = (idx & 3u) * 2u + blk;
                        const uint32_t o = (idx >> 2) * 2048u + dj * 128u + ((cc ^ (dj & 7u)) << 4) + half * 8u;
#pragma unroll
                        for (uint32_t t = 0; t < kTok; ++t) {
                            if (t < nt && (t & 1u) == (tid >> 6)) {
                                const uint2 c8 = *reinterpret_cast<const uint2 *>(&s_hst[t][(dj * 2u + blk) * 16u + half * 8u]);
                                *reinterpret_cast<uint2 *>(a.hdig + (size_t)pair[t] * KD * 2048u + o) = c8;
                            }
                        }
                        }  // (digit rows laid out here)
                    }
                }
            }
        } else if (warp >= kGLayWarp0) {
            // ---- the scale codes of the chunk's digit rows, as the atoms tensor memory takes (row n of
            // the operand = 16 * token + digit row: byte (n % 32) * 16 + (n / 32) * 4 + block % 4 of the atom
            // of four scale blocks); digit row j < 8 of a block with exponent E has the code
            // 127 + E - 23 + 3 j, row 8 + j the code 127 + E - 47 + 3 j; the exponents are stored as E + 100.
            // A thread fetches its words of the item before it waits for the buffer. ----
            const uint32_t lt = tid - kGLayWarp0 * 32u;
            const uint32_t atom = lt >> 7, r32 = (lt >> 2) & 31u, col = lt & 3u;
            const uint32_t tl = 2u * col + (r32 >> 4), j = r32 & 15u;   // the row's token inside a half, its digit row
            const int shift = j < 8u ? 4 + 3 * (int)j : 3 * (int)(j & 7u) - 20;
            const uint32_t bias = 0x01010101u * (uint32_t)shift;
#pragma unroll 1
            for (uint32_t i = 0; i < nb && ok; ++i, ++gi) {
                const uint32_t buf = gi & 1u, nt = s_rec[i].nt & 0xFFu;
                const uint32_t *vecs = kDown ? s_rec[i].pair : s_rec[i].tok;
                // ---- large blocks: the chunk's token tiles of one unit of the item, behind the unit in its ring
                // stage: sixteen bytes per copy and thread (cp.async: these bytes do not pass through the
                // bulk-copy unit that brings the pages; measured 1.83 -> 1.65 ms for 370 tokens, but 151 -> 165 us
                // for 8), the copies' completion counted on the stage's barrier ----
                const uint32_t n16 = nt * 128u;   // sixteen-byte pieces of the chunk's tiles of one unit
                auto copy_tiles = [&](uint32_t u) -> bool {
                    if (p_round && !mbar_wait(bar(kGBarDone + p_slot), (p_round - 1u) & 1u, abortp)) return false;
                    const uint32_t dst0 = smem_u32(sRing) + p_slot * a.stage + kMt * kStageA;
#pragma unroll 1
                    for (uint32_t c = lt; c < n16; c += kGLayThreads) {
                        const uint32_t tt = c >> 7, off = (c & 127u) << 4;
                        const uint8_t *src = a.dig + ((size_t)vecs[tt] * nu + u) * 2048u + off;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + tt * 2048u + off), "l"(src) : "memory");
                    }
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(kGBarFull + p_slot)) : "memory");
                    if (++p_slot == ring) {
                        p_slot = 0;
                        ++p_round;
                    }
                    return true;
                };
                // one set of atoms per item (rows of up to six tokens), in the buffer of the item's parity; wide
                // chunks: one set per half of the chunk, a buffer each, rewritten when the item before is done
                uint32_t ew[kWide ? 2 : 1][16];
#pragma unroll
                for (uint32_t h = 0; h < (kWide ? 2u : 1u); ++h) {
                    const uint32_t t = h * kNtHalf + tl;
                    const bool mine = tl < kNtHalf && t < nt;
                    const uint32_t vec = mine ? vecs[t] : 0u;
                    const uint32_t *e4 = reinterpret_cast<const uint32_t *>(a.exps + (size_t)vec * (K >> 5)) + atom;
#pragma unroll
                    for (uint32_t u = 0; u < 16; ++u) ew[h][u] = (mine && u < nu) ? __ldcg(e4 + u * 2u) + bias : 0x7F7F7F7Fu;
                }
                // wide chunks: the atoms wait for the item before, the token tiles of the item's first units do not
                // (the stages they wait for belong to the item before: an item has at least as many units as the
                // ring has stages)
                uint32_t u0 = 0;
                if (kWide && a.by_threads) {
                    const uint32_t ahead = (ring - 1u) < nu ? ring - 1u : nu;
#pragma unroll 1
                    for (; u0 < ahead && ok; ++u0) ok = copy_tiles(u0);
                    if (!ok) break;
                }
                // the buffers' last readers were the copies of item gi - 2, or (wide chunks) gi - 1
                if (!kWide) {
                    if (gi >= 2u) ok = mbar_wait(bar(kGBarAccDone + buf), ((gi - 2u) >> 1) & 1u, abortp);
                } else if (gi >= 1u) {
                    ok = mbar_wait(bar(kGBarAccDone + ((gi - 1u) & 1u)), ((gi - 1u) >> 1) & 1u, abortp);
                }
                if (!ok) break;
#pragma unroll
                for (uint32_t h = 0; h < (kWide ? 2u : 1u); ++h) {
                    uint8_t *dst = sSfb + (kWide ? h : buf) * kSfbBytes + atom * kAtomBytes + r32 * 16u + col * 4u;
#pragma unroll
                    for (uint32_t u = 0; u < 16; ++u)
                        if (u < nu) *reinterpret_cast<uint32_t *>(dst + u * 1024u) = ew[h][u];
                }
                fence_async_smem();  // tcgen05.cp reads the atoms
                mbar_arrive(bar(kGBarSfb + buf));
                if (!a.by_threads) continue;   // (small blocks: the second copying thread brings them)
#pragma unroll 1
                for (uint32_t u = u0; u < nu && ok; ++u) ok = copy_tiles(u);
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
        __syncwarp();
        __syncthreads();  // the records are rewritten; a role that gave up has raised the flag
        if (abort_flag) break;
    }
    if (is_issuer) {
        // nothing of this CTA's tensor work is in flight when the tensor memory is freed
        umma_commit(bar(kGBarFin));
        mbar_wait(bar(kGBarFin), 0, abortp);
    }
    __syncwarp();
    if (is_prod_a) {
        // copies in flight land in this CTA's shared memory: wait for them before leaving (a stage's
        // barrier completes when the unit and the token tiles are there)
        const uint32_t units = s_units, first = units > ring ? units - ring : 0u;
#pragma unroll 1
        for (uint32_t u = first; u < units; ++u) {
            const uint32_t s = u % ring, parity = (u / ring) & 1u;
            uint32_t tries = 0;
#pragma unroll 1
            while (!mbar_try(bar(kGBarFull + s), parity) && ++tries < kSpin) {
            }
        }
    }
    fence_before();
    __syncwarp();
    __syncthreads();
    if (warp == kGMmaWarp0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    }
    if (tid == 0 && abort_flag) atomicExch(status, 0x5507u);
    if constexpr (kDown) {
        if (a.ep_world > 1u) {
            // every store of this CTA to the peers' buffers is ordered before the count; the last CTA of the
            // grid publishes the call's number to every rank
            if (warp < 4u) __threadfence_system();
            __syncthreads();
            if (tid == 0) {
                __threadfence_system();
                if (atomicAdd(a.ep_counter, 1u) == grid - 1u) {
                    *a.ep_counter = 0u;
                    __threadfence_system();
                    const unsigned long long word = abort_flag ? 0ull : (unsigned long long)a.ep_call;
#pragma unroll 1
                    for (uint32_t p = 0; p < a.ep_world; ++p)
                        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.flag_peer[p] + a.ep_rank), "l"(word) : "memory");
                }
            }
        }
    }
}

// y[t, n]: the ordered mix of token t (examples/s14_vulkan_numeric.rs:936-946): acc = 0; acc += w * d
// over the routes in order; acc += d of the shared expert.  With `residual` the layer's input is added
// (y = x + acc, what a layer of a stack hands to the next); y may be x.
__global__ void __launch_bounds__(256)
k_block_mix(const float *__restrict__ d, const int32_t *__restrict__ ids, const float *__restrict__ weights,
            uint32_t top_k, int has_shared, float *y, uint32_t hidden, const uint32_t *__restrict__ counts,
            const float *x, uint32_t residual, const unsigned long long *flags, uint32_t ep_world, uint32_t ep_call,
            uint32_t wait_limit, uint32_t *status, uint32_t official) {
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (flags) {
        // expert parallel, exchange inside the kernels: every rank's rows of this call are in this rank's buffer
        // when its flag carries the call's number (bounded wait: about a microsecond per poll)
        __shared__ int s_ok;
        if (threadIdx.x == 0) {
            int ok = 1;
            for (uint32_t p = 0; p < ep_world && ok; ++p) {
                uint32_t tries = 0;
                for (;;) {
                    unsigned long long v;
                    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + p) : "memory");
                    if (v >= (unsigned long long)ep_call) break;
                    if (++tries > wait_limit) {
                        ok = 0;
                        atomicExch(status, 0x5508u);
                        break;
                    }
                    __nanosleep(1000);
                }
            }
            s_ok = ok;
        }
        __syncthreads();
        if (!s_ok) return;
    }
    if (n >= hidden || __ldcg(counts + 3)) return;
    const float *dt = d + (size_t)t * kPairsPerToken * hidden + n;
    float acc = 0.0f;
    // official arithmetic: the route's weight went into the expert's hidden values; the BF16 outputs are added
    // in F32 and the sum is rounded to BF16 (moe_branch, s14_first_real_token/executor.py:716-735)
    for (uint32_t m = 0; m < top_k; ++m)
        if (__ldg(ids + t * top_k + m) >= 0)
            acc = __fadd_rn(acc, official ? __ldcg(dt + (size_t)m * hidden)
                                          : __fmul_rn(__ldg(weights + t * top_k + m), __ldcg(dt + (size_t)m * hidden)));
    if (has_shared) acc = __fadd_rn(acc, __ldcg(dt + (size_t)S14_EXPERTS_PER_TOKEN * hidden));
    if (official) acc = bf16_round(acc);
    y[(size_t)t * hidden + n] = residual ? __fadd_rn(x[(size_t)t * hidden + n], acc) : acc;
}

constexpr int kMaxDevices = 64;
size_t g_block_limit[kMaxDevices][3] = {};

// The dynamic shared memory the contraction kernels of a shape (0: one row tile per item, 1: two, 2: two with
// wide chunks) may ask for on the current device (set once per device and shape).
size_t block_dynamic_limit(uint32_t shape) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices || shape > 2u) return 0;
    if (g_block_limit[dev][shape]) return g_block_limit[dev][shape];
    int optin = 0;
    if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    // the kernels of a shape (up in its three modes, down in two) get the same limit
    auto set_up = [&](std::initializer_list<const void *> fns) -> size_t {
        size_t fixed = 0;
        cudaFuncAttributes fa;
        for (const void *fn : fns) {
            if (cudaFuncGetAttributes(&fa, fn) != cudaSuccess) return 0;
            if (fa.sharedSizeBytes > fixed) fixed = fa.sharedSizeBytes;
        }
        if ((size_t)optin <= fixed) return 0;
        const size_t most = (size_t)optin - fixed;
        for (const void *fn : fns)
            if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most) != cudaSuccess) return 0;
        return most;
    };
#define S14_BLOCK_KERNELS(MT, WIDE)                                                                                              \
    set_up({(const void *)k_block_gemm<false, MT, WIDE, kModeFused>, (const void *)k_block_gemm<false, MT, WIDE, kModeOfficial>, \
            (const void *)k_block_gemm<false, MT, WIDE, kModeValues>, (const void *)k_block_gemm<true, MT, WIDE, kModeFused>,    \
            (const void *)k_block_gemm<true, MT, WIDE, kModeOfficial>})
    const size_t most = shape == 0u ? S14_BLOCK_KERNELS(1, false) : (shape == 1u ? S14_BLOCK_KERNELS(2, false) : S14_BLOCK_KERNELS(2, true));
#undef S14_BLOCK_KERNELS
    g_block_limit[dev][shape] = most;
    return most;
}

// Ring stages that fit beside the scale atoms; with one row tile per item an even number (a slot belongs to one issuing thread).
uint32_t block_ring(size_t limit, uint32_t stage, bool even) {
    if (limit < 2u * kSfbBytes + 2u * stage) return 0;
    uint32_t r = (uint32_t)((limit - 2u * kSfbBytes) / stage);
    if (r > kGRingMax) r = kGRingMax;
    return even ? (r & ~1u) : r;
}

}  // namespace

bool moe_block_ok(int sm_count, uint32_t hidden, uint32_t inter, uint32_t n_experts, uint32_t top_k) {
    if (sm_count <= 0 || n_experts == 0u || n_experts > S14_N_ROUTED_EXPERTS || top_k == 0u || top_k > S14_EXPERTS_PER_TOKEN)
        return false;
    if ((hidden & 511u) || (inter & 511u) || hidden < 512u || inter < 512u || hidden > 4096u || inter > 4096u) return false;
    return block_ring(block_dynamic_limit(0), kStageA + 2u * 2048u, true) >= 2u &&
           block_ring(block_dynamic_limit(1), 2u * kStageA + kNtHalf * 2048u, true) >= 2u &&
           block_ring(block_dynamic_limit(2), 2u * kStageA + kNt * 2048u, false) >= 2u;
}

size_t moe_block_max_chunks(uint32_t max_tokens) {
    // no more chunks than pairs (chunks of one token)
    return (size_t)max_tokens * kPairsPerToken;
}

int launch_moe_block(cudaStream_t st, int sm_count, const BlockWork &w, const float *x, float *y, const int32_t *ids,
                     const float *weights, const uint8_t *const *pages, const uint8_t *const *page_table,
                     const uint8_t *shared_page, uint32_t n_tokens, uint32_t top_k, uint32_t n_experts, uint32_t hidden,
                     uint32_t inter, uint32_t *status, cudaError_t *err, uint32_t nt_cap, bool residual, uint32_t ep_rank,
                     uint32_t ep_world, float *pairs_out, const BlockEp *ep, bool shared_by_token, bool official) {
    // Three shapes.  A small block (up to 12 tokens) is bound by the memory's latency: most experts have one
    // token, chunks of two and short stages make the ring deeper (more page bytes in flight), the shared expert's
    // extra chunks come from the L2, and one row tile per item keeps enough items to level out over the SMs.
    // Larger blocks take two row tiles per item (half the tile bytes); with three or more pairs per expert on
    // average they take wide chunks of twelve tokens (fewer passes over every page), else chunks of six.
    uint32_t shape;
    *err = cudaErrorInvalidConfiguration;
    if (official && (ep || pairs_out || !w.hval)) return 0;   // the official arithmetic runs on one GPU
    if (nt_cap == 0u) shape = n_tokens <= 12u ? 0u : ((uint64_t)n_tokens * top_k >= 3ull * n_experts ? 2u : 1u);
    else shape = nt_cap <= 2u ? 0u : (nt_cap <= kNtHalf ? 1u : 2u);
    nt_cap = shape == 0u ? (nt_cap ? nt_cap : 2u) : (shape == 1u ? kNtHalf : kNt);
    const uint32_t mt = shape == 0u ? 1u : 2u;
    const uint32_t stage = mt * kStageA + nt_cap * 2048u;
    const uint32_t ring = block_ring(block_dynamic_limit(shape), stage, shape != 2u);
    *err = cudaErrorInvalidConfiguration;
    if (ring < 2u || n_tokens == 0u) return 0;
    const uint32_t S = inter >> 6, RT = hidden >> 7;
    const size_t smem = (size_t)ring * stage + 2u * kSfbBytes;
    k_block_digits<<<n_tokens, 512, 0, st>>>(x, hidden, w.xdig, w.xexp, official ? 1u : 0u);
    if (ep_world == 0u) ep_world = 1u;
    k_block_group<<<1, 1024, 0, st>>>(ids, pages, page_table, shared_page, n_tokens, top_k, n_experts, S / mt, RT / mt, nt_cap,
                                     w.chunks, w.counts, ep_rank, ep_world, (shared_by_token && ep_world > 1u) ? 1u : 0u);
    if (pairs_out && !ep) {
        // expert parallel: the pairs of the experts this rank owns; the others stay zero for the sum over the ranks
        *err = cudaMemsetAsync(pairs_out, 0, (size_t)n_tokens * kPairsPerToken * hidden * sizeof(float), st);
        if (*err != cudaSuccess) return 2;
    }
    const uint32_t by_threads = nt_cap > 2u ? 1u : 0u;
    GemmArgs up = {w.chunks, w.counts + 1, w.xdig, w.xexp, nullptr, w.hdig, w.hexp, by_threads, hidden, inter, ring, stage};
    GemmArgs down = {w.chunks, w.counts + 2, w.hdig, w.hexp, pairs_out ? pairs_out : w.d, nullptr, nullptr, by_threads, hidden, inter, ring, stage};
    if (ep) {
        // exchange inside the kernel: the owned pairs' rows into every rank's buffer of the call's parity
        for (uint32_t p = 0; p < ep->world; ++p) {
            down.out_peer[p] = ep->pairs_peer[p];
            down.flag_peer[p] = ep->flags_peer[p];
        }
        down.ep_counter = ep->counter;
        down.ep_world = ep->world;
        down.ep_rank = ep->rank;
        down.ep_call = ep->call;
    }
    // Small blocks: the up epilogue lays out the digit rows of the hidden values itself.  Large blocks and the
    // official arithmetic: it leaves the values, and a second digits launch (which also quantises them per 128
    // elements for the official arithmetic) lays out the rows of all pairs' slots (a slot without a route holds
    // zeros or an earlier call's values: finite numbers nobody reads the rows of).
    const bool values = official || (shape != 0u && w.hval != nullptr);
    int launches = 4;
    if (values) {
        up.hval = w.hval;
        up.weights = weights;
        up.top_k = top_k;
        ++launches;
    }
#define S14_BLOCK_UP(MT, WIDE)                                                                                  \
    do {                                                                                                        \
        if (official) k_block_gemm<false, MT, WIDE, kModeOfficial><<<sm_count, kGThreads, smem, st>>>(up, status);   \
        else if (values) k_block_gemm<false, MT, WIDE, kModeValues><<<sm_count, kGThreads, smem, st>>>(up, status);  \
        else k_block_gemm<false, MT, WIDE, kModeFused><<<sm_count, kGThreads, smem, st>>>(up, status);              \
        if (values) k_block_digits<<<n_tokens * kPairsPerToken, 512, 0, st>>>(w.hval, inter, w.hdig, w.hexp, official ? 1u : 0u); \
        if (official) k_block_gemm<true, MT, WIDE, kModeOfficial><<<sm_count, kGThreads, smem, st>>>(down, status);  \
        else k_block_gemm<true, MT, WIDE, kModeFused><<<sm_count, kGThreads, smem, st>>>(down, status);             \
    } while (0)
    if (shape == 0u) S14_BLOCK_UP(1, false);
    else if (shape == 1u) S14_BLOCK_UP(2, false);
    else S14_BLOCK_UP(2, true);
#undef S14_BLOCK_UP
    if (pairs_out) {
        *err = cudaGetLastError();
        return launches;
    }
    k_block_mix<<<dim3((hidden + 255u) / 256u, n_tokens), 256, 0, st>>>(w.d, ids, weights, top_k, shared_page != nullptr, y, hidden,
                                                                       w.counts, x, residual ? 1u : 0u, nullptr, 1u, 0u, 0u, status,
                                                                       official ? 1u : 0u);
    *err = cudaGetLastError();
    return launches + 1;
}

cudaError_t launch_block_mix(cudaStream_t st, const float *pairs, const int32_t *ids, const float *weights, uint32_t n_tokens,
                             uint32_t top_k, bool has_shared, const float *x, float *y, uint32_t hidden, const uint32_t *counts,
                             const BlockEp *ep, uint32_t *status) {
    k_block_mix<<<dim3((hidden + 255u) / 256u, n_tokens), 256, 0, st>>>(pairs, ids, weights, top_k, has_shared, y, hidden, counts, x,
                                                                       x ? 1u : 0u, ep ? ep->flags : nullptr, ep ? ep->world : 1u,
                                                                       ep ? ep->call : 0u, ep ? ep->wait_limit : 0u, status, 0u);
    return cudaGetLastError();
}

}  // namespace s14
