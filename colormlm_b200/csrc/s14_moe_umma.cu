// The pairwise-order MoE layer of one token on the fifth-generation tensor cores:
// tcgen05.mma kind::mxf4.block_scale consumes the page bytes as they are (packed E2M1, one
// UE8M0 scale per 32 elements along K), so no thread decodes or scales a weight.
//
// The matvec as a block-scaled MMA.  A = 128 weight rows x 64 K-elements per instruction; its
// scales go to tensor memory with tcgen05.cp.  B = the activation vector as sixteen balanced
// base-8 digit rows: within a scale block of 32 elements with largest magnitude < 2^E
// (-80 <= E <= 127), every element is q * 2^(E-47) with q a 48-bit integer (exact for every F32
// value down to 2^-24 of the block's largest), q = hi * 8^8 + lo, and hi, lo are written with eight
// digits d_j in [-4, 4] each -- all of them E2M1 values.  Row j < 8 holds the digits of hi with the
// UE8M0 scale 2^(E-23+3j), row 8 + j the digits of lo with 2^(E-47+3j).  Accumulator column j holds
// the digit-j share of the dot product: a sum of small integers times powers of two, which the F32
// accumulator in tensor memory holds exactly at the magnitudes of this path, so the sixteen columns
// added in double and rounded once give the double-accumulated dot product rounded to F32.
//
// Work.  An expert page is stored as units of 128 rows x 256 K-elements (s14_page_layout.h); a unit
// and its scale atoms are two plain bulk copies (cp.async.bulk, no multicast) into one ring slot.
//   up item   (job, slice of 64 intermediate elements): hidden / 256 units accumulate into one
//             accumulator (lanes 0-63 the gate, 64-127 the up projection); the epilogue applies the
//             limited SwiGLU, writes the 64 hidden values as digit rows into the job's digit tile in
//             global memory (L2) and counts the slice on the job's counter.
//   down item (job, tile of 128 output rows): waits (bounded) until the job's counter says that
//             every slice is there, takes the job's digit tile into shared memory, and accumulates
//             intermediate / 256 units into one accumulator: the finished rows of the expert's
//             output.  The last item of a row tile to finish (a counter, no waiting) applies the
//             ordered mix to that tile.
// No output passes through partial sums of several CTAs, so the result does not depend on how
// items are dealt.  Items are dealt to the CTAs (one per SM, all resident) in a fixed pattern that
// levels the number of units per CTA; a CTA runs its up items first, then its down items.
//
// Roles inside a CTA: one copying thread, two MMA-issuing threads (even and odd units of an item,
// an accumulator each), four epilogue warps (tcgen05.ld, sums, SwiGLU, digits, mix), eight warps
// that fetch digit tiles for the down items.  Every wait (mbarrier, counter, peer word) is bounded;
// a wait that runs out raises the CTA's abort flag, the status word is set, and the CTA waits for
// its copies in flight, frees its tensor memory and returns.
#include "s14_umma.cuh"

namespace s14 {

namespace {

constexpr uint32_t kSlot = kUnitStride;             // ring slot: a unit's codes, then its scales (17 KB, keeps 1 KB alignment)
constexpr uint32_t kMaxRing = 12;                  // ring slots are an even number: a slot belongs to one issuing thread
constexpr uint32_t kThreads = 512;                 // sixteen warps; every thread owns eight elements of the token
constexpr uint32_t kTokenThreads = 512;
constexpr uint32_t kEpiThreads = 128;              // warps 0-3: one per lane quadrant of tensor memory
constexpr uint32_t kMmaWarp0 = 5;                  // warps 5, 6: lane 0 issues
constexpr uint32_t kLoadWarp0 = 8;                 // warps 8-15 fetch digit tiles (and pick the routes)
constexpr uint32_t kLoadThreads = 256;
constexpr uint32_t kProdWarp = 4;                  // lane 0 copies (the warp has no other role after the top of a layer)
constexpr uint32_t kMaxItems = 32;                 // items a CTA can hold
constexpr uint32_t kJobsMax = S14_EXPERTS_PER_TOKEN + 1;
constexpr uint32_t kTileMax = 32768;               // digit tile of a 4096-long vector: 16 units of 2 KB
constexpr uint32_t kExpMax = 128;                  // its block exponents
// tensor memory columns
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColAcc = 0;      // [2 buffers][2 issuing threads][16]
constexpr uint32_t kColSfa = 64;     // [2 issuing threads][16]: weight scales of the unit each thread is at
// Scales of digit rows: an atom (four scale blocks) is four columns (N-rows 0-31, 32-63, ...; a
// 16-row operand uses the first).  Scale addresses given to the MMA stay atom-aligned.
constexpr uint32_t kColSfbX = 96;    // hidden / 32 columns: the token's digit rows
constexpr uint32_t kColSfbH = 224;   // [2 tiles][128]: the hidden values' digit rows
static_assert(kColSfbH + 2 * 128 <= kTmemCols, "tensor memory map");
constexpr uint32_t kMaxHidden = 4096;
constexpr uint32_t kSpinGlobal = 1u << 20;  // polls (100 ns apart) of a counter before giving up
// the context's counter array ([0] is the router kernel's); [1, kCntEnd) are zero between launches
constexpr uint32_t kCntExit = 2;
constexpr uint32_t kCntEnd = 4;
constexpr uint32_t kRouterSlots = 2;                 // experts a CTA scores at most
constexpr uint32_t kItemDown = 0x80000000u;
constexpr uint32_t kTraceWords = 96;   // time marks per CTA of a profiling run
// The kernel's scratch in global memory, all of it stamped words but the launch count: a head (the
// launch count, then the expert scores, [2 layer parities][256]), then per job a digit tile (a word
// per four bytes of the tile) and the tile's block exponents (a word each).
constexpr uint32_t kScratchScores = 256;
constexpr uint32_t kScratchHead = 8192;
constexpr uint32_t kTileWordBytes = 2u * kTileMax;   // a job's tile as words
constexpr uint32_t kExpWordBytes = 8u * kExpMax;     // its block exponents as words
// after them: the experts' outputs [job slot][kMaxHidden] and the token between the layers of a
// stack [2 layer parities][kMaxHidden], a word per value
constexpr uint32_t kMaxLayers = 62;    // a stamp is launch count * 64 + layer + 1

// Barriers.
constexpr uint32_t kBarFull = 0;                      // ring slot filled (one arrival + the copies' bytes)
constexpr uint32_t kBarDone = kMaxRing;               // the slot's MMAs have completed (the copies may reuse it)
constexpr uint32_t kBarAccDone = 2 * kMaxRing;        // [2] an item's accumulators are complete (both issuing threads)
constexpr uint32_t kBarAccFree = kBarAccDone + 2;     // [2] ... have been read
constexpr uint32_t kBarXReady = kBarAccFree + 2;      // the token's digit scales are in tensor memory
constexpr uint32_t kBarHReady = kBarXReady + 1;       // [2] a digit tile of hidden values is in place
constexpr uint32_t kBarHFree = kBarHReady + 2;        // [2] ... is not read any more
constexpr uint32_t kBarFin = kBarHFree + 2;           // both issuing threads have finished
constexpr uint32_t kBarRoutes = kBarFin + 1;          // the jobs and the CTA's items are in shared memory
constexpr uint32_t kBarWr = kBarRoutes + 1;           // the layer's router rows of this CTA are in shared memory
constexpr uint32_t kBarPages = kBarWr + 1;            // the picked experts' pages are in the job records (early lists)
constexpr uint32_t kBars = kBarPages + 1;
constexpr uint32_t kRouteWarp = 15;                   // the warp that publishes the CTA's expert scores

// Instruction descriptor: A and B E2M1 (format 1), both K-major, N = 16, UE8M0 scales, M = 128.
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24);

}  // namespace

// The items of CTA c of G: its up items (job j, slice) first, then its down items (job j, row tile),
// each as down-bit | j << 8 | index.  KU, KD: units of an up and of a down item.  Writes at most
// `cap` items, returns the CTA's number of items.
//
// n_early: the first n_early jobs' pages are known before the token's routes are (the shared expert
// of a routed layer).  Their up items run while the routes are being picked, when the memory is idle,
// and do not count in the levelling.  All up items q = j * S + slice go round the CTAs (q mod G); the
// CTAs are then numbered from the one after the last early item (c_rot), so that the CTAs that hold an
// early item are among those with fewer of the other up items.  The down items p = j * RT + tile are
// dealt as described below.
__host__ __device__ uint32_t layer_work_list(uint32_t c, uint32_t G, uint32_t n_jobs, uint32_t S, uint32_t RT,
                                             uint32_t KU, uint32_t KD, uint32_t *items, uint32_t cap, uint32_t n_early) {
    const uint32_t U = n_jobs * S, D = n_jobs * RT;
    uint32_t n = 0;
    if (U == 0u || G == 0u) return 0u;
    if (n_early > n_jobs) n_early = n_jobs;
    const uint32_t F = n_early * S, UR = U - F;
    for (uint32_t q = c; q < U; q += G, ++n)
        if (n < cap) items[n] = ((q / S) << 8) | (q % S);
    const uint32_t c_rot = (c + G - F % G) % G;
    // CTAs c_rot = 0 .. r-1 hold a_max of the levelled up items, the others one fewer
    const uint32_t a_max = UR ? (UR + G - 1u) / G : 1u, r = UR - (a_max - 1u) * G;
    // The CTAs with one up item fewer are free a whole up item earlier, but a job's down items can start
    // only some microseconds after its last slice (SwiGLU, digits, publication, the tile's way into shared
    // memory), which is about what a down item itself takes: each of them takes ONE down item of the jobs
    // that are finished by then (the early jobs, and the jobs whose slices all lie one round of up
    // items earlier); the rest goes round all CTAs.
    const uint32_t n_light = G - r;
    const uint32_t ready = RT * (n_early + ((a_max - 1u) * G) / S);
    uint32_t D1 = n_light;
    if (D1 > ready) D1 = ready;
    if (D1 > D) D1 = D;
    (void)KU;
    (void)KD;
    if (c_rot >= r && c_rot - r < D1) {
        const uint32_t p = c_rot - r;
        if (n < cap) items[n] = 0x80000000u | ((p / RT) << 8) | (p % RT);
        ++n;
    }
    // Without early jobs the first round starts at CTA 0 (the CTAs with more up items get the jobs that
    // finish first) and further rounds with the CTAs that have fewer up items.  With early jobs the
    // up items are level already, and every round starts with the CTAs that have fewer of them.
    for (uint32_t k = 0;; ++k) {
        const uint32_t pos = (k == 0u && n_early == 0u) ? c : (c_rot + G - r) % G;
        const uint32_t p = D1 + k * G + pos;
        if (D1 + k * G >= D) break;
        if (p < D) {
            if (n < cap) items[n] = 0x80000000u | ((p / RT) << 8) | (p % RT);
            ++n;
        }
    }
    return n;
}

namespace {

// the one device copy of the deal (its divisions make it long; a CTA calls it once)
__device__ __noinline__ uint32_t work_list_once(uint32_t c, uint32_t G, uint32_t n_jobs, uint32_t S, uint32_t RT, uint32_t KU,
                                                uint32_t KD, uint32_t *items, uint32_t n_early) {
    const uint32_t n = layer_work_list(c, G, n_jobs, S, RT, KU, KD, items, kMaxItems, n_early);
    return n < kMaxItems ? n : kMaxItems;
}
// Nothing on the kernel's paths may live in local memory: nearly all of the SM's L1 is carved out as
// shared memory, so the 544 threads' stack frames would miss it and every local access would cost
// an L2 round trip (measured: a 100-instruction block went from 0.25 to 3 microseconds).  Helpers are
// inlined, arrays are indexed by unrolled loops, and only code that runs once per launch or layer
// with little live state (the deal, the route records) is kept out of line.

// 512 threads = 16 warps, four per sub-partition of the SM: up to 128 registers per thread.
template <bool kTrace>
__global__ void __launch_bounds__(kThreads, 1)
k_moe_layer_umma(const JobTable *__restrict__ dev_table, const __grid_constant__ JobTable param_table,
                 const float *__restrict__ x, float *d_out, float *__restrict__ y, uint8_t *tiles,
                 unsigned int *counters, uint32_t *__restrict__ status, uint32_t hidden, uint32_t inter,
                 uint32_t ring, unsigned long long *trace, const __grid_constant__ FusedRouter rt,
                 const __grid_constant__ EpExchange ep, const StackLayer *__restrict__ stack, uint32_t n_layers,
                 float *hbuf, uint32_t residual) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[kBars];
    __shared__ __align__(16) uint8_t sE[kExpMax];        // block exponents of the token's digits
    __shared__ __align__(16) uint8_t sEh[2][kExpMax];    // ... of the digit tiles of hidden values
    __shared__ __align__(16) uint8_t s_hst[16 * 2 * 16]; // an up item's digit chunks: [row][block][16 bytes]
    __shared__ float s_up[64];                           // an item's up projection, handed to the gate threads
    // per layer parity: the mix, in route order: weight (shared expert: 1) and row of the expert
    // outputs, bit 31 set for the shared expert; the layer's jobs, from the routes or the caller's table
    __shared__ float s_mix_w[2][kJobsMax];
    __shared__ uint32_t s_mix_slot[2][kJobsMax];
    __shared__ Job s_jobs[2][kJobsMax];
    __shared__ uint32_t s_n_mix, s_n_jobs;
    __shared__ uint32_t s_items[kMaxItems];
    __shared__ uint32_t s_n_items;
    __shared__ unsigned long long s_page[S14_N_ROUTED_EXPERTS];  // the layer's page table, parked a layer ahead
    __shared__ float s_bias[S14_N_ROUTED_EXPERTS];       // the layer's bias, likewise
    __shared__ StackLayer s_layer[2];                    // the layer's own pointers, by layer parity
    __shared__ uint32_t s_prod[8];                       // the copying thread's position between its steps
    __shared__ uint32_t s_ep_step, s_stamp0;
    __shared__ uint32_t s_pick_id[8];                    // the picked experts by rank, their scores and pages
    __shared__ float s_pick_score[8];
    __shared__ unsigned long long s_pick_page[8];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ int s_behind;   // expert parallel: a peer's word carries a later step's number
    __shared__ int s_last;     // this CTA finished the last job of a row tile / is the last CTA to leave
    __shared__ uint32_t s_abort_code;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t grid = gridDim.x, cta = blockIdx.x;
    const uint32_t KU = hidden >> 8;   // units of an up item
    const uint32_t KD = inter >> 8;    // units of a down item
    const uint32_t RT = hidden >> 7;   // row tiles of w2
    const uint32_t S = inter >> 6;     // slices of an expert
    const uint32_t L = n_layers ? n_layers : 1u;
    uint8_t *const sRing = smem;
    uint8_t *const sBx = smem + ring * kSlot;   // the token's digit tile, 2 KB per 256 K-elements
    uint8_t *const sBh = sBx + KU * 2048u;      // two digit tiles of hidden values
    const uint32_t tile_bytes = KD * 2048u;
    uint8_t *const sWr = sBh + 2u * tile_bytes; // the router rows of this CTA's experts (BF16), a layer ahead
    // Values that cross CTAs inside a layer travel as 8-byte words {stamp, value}: the reader polls the
    // word itself until it carries the stamp of this launch and layer, so no fence, counter or vote
    // stands between the writer's store and the reader's load.
    unsigned long long *const score_words = reinterpret_cast<unsigned long long *>(tiles + kScratchScores);
    uint8_t *const tile0 = tiles + kScratchHead;                           // [job][kTileWordBytes]
    unsigned long long *const tile_exps =
        reinterpret_cast<unsigned long long *>(tile0 + (size_t)kJobsMax * kTileWordBytes);  // [job][kExpMax] after the tiles
    unsigned long long *const d_words = tile_exps + (size_t)kJobsMax * kExpMax;            // [slot][kMaxHidden]
    unsigned long long *const x_words = d_words + (size_t)kJobsMax * kMaxHidden;            // [2][kMaxHidden]
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](uint32_t i) { return bar0 + i * 8u; };
    volatile int *const abortp = &abort_flag;
    // Optional per-CTA time marks (SM clock) for profiling runs: kTraceWords words per CTA, word 0 the
    // global timer at entry; taken in the second layer of a stack (its code has run before), else in
    // the only one.  One designated thread writes each mark.
    // The kernel is compiled twice: the marks exist in the profiling build only.
    auto trace_base = [&]() -> unsigned long long * { return (kTrace && trace) ? trace + (size_t)cta * kTraceWords : nullptr; };
    const uint32_t trace_layer = L > 1u ? 1u : 0u;
    unsigned long long *tr = trace_layer == 0u ? trace_base() : nullptr;
    auto mark = [&](uint32_t i) {
        if constexpr (kTrace) {
            if (tr && i < kTraceWords) tr[i] = (unsigned long long)clock64();
        }
    };
    // a mark that is taken only when `dep` has been computed
    auto mark_after = [&](uint32_t i, uint32_t dep) {
        if constexpr (kTrace) {
            if (tr && i < kTraceWords) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%clock64;" : "=l"(t) : "r"(dep) : "memory");
                tr[i] = t;
            }
        }
    };
    if (kTrace && trace && tid == 0) {
        unsigned long long gt;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
        trace_base()[0] = gt;
        trace_base()[1] = (unsigned long long)clock64();
    }

    // Thread t < 512 owns elements 8t .. 8t+7 of the token (hidden <= 4096), for the digits and for
    // the router's dot products.
    const bool routes_here = rt.weight != nullptr || stack != nullptr;
    const bool ep_on = ep.world > 1u;
    const bool table_param = !routes_here && dev_table == nullptr;
    // the CTA's items are known at once unless the number of jobs depends on the routes (expert
    // parallel: a rank keeps the experts it owns) or the table comes from an earlier kernel
    const bool early = table_param || (routes_here && rt.ep_world <= 1u);
    // the shared expert of a layer that picks its own routes: its up items run while the routes are picked
    const uint32_t n_early_jobs = (early && routes_here && rt.has_shared) ? 1u : 0u;
    const bool has_x = tid < (hidden >> 3);
    const bool is_producer = tid == kProdWarp * 32u;
    // The kernel is launched as a programmatic dependent of whatever precedes it in the stream: its
    // CTAs may be placed as soon as SMs are free and set themselves up (barriers, tensor memory, the
    // first copies of pages whose addresses are launch arguments); everything an earlier kernel may
    // have written (the token, the counters, a device job table, the step count) is read only after
    // cudaGridDependencySynchronize() below.  In the same way the next launch may be set up from now
    // on.  Weights and page tables are constant during a step.
    cudaTriggerProgrammaticLaunchCompletion();

    // ---- set-up: the barriers by the first threads, the jobs and items that are known at launch
    // by warp 1 ----
    if (tid < kBars) {
        uint32_t count = 1u;  // ring slots, routes
        if (tid >= kBarAccDone && tid < kBarAccDone + 2u) count = 2u;
        else if (tid >= kBarAccFree && tid < kBarAccFree + 2u) count = kEpiThreads;
        else if (tid == kBarXReady) count = 256u;
        else if (tid >= kBarHReady && tid < kBarHReady + 2u) count = kLoadThreads;
        else if (tid >= kBarHFree && tid < kBarHFree + 2u) count = 2u;
        else if (tid == kBarFin) count = 2u;
        mbar_init(bar(tid), count);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2u && lane < sizeof(StackLayer) / 8u) {
        // the first layer's pointers (launch arguments, or the stack's table, which no kernel writes)
        unsigned long long v = 0ull;
        if (stack) v = __ldg(reinterpret_cast<const unsigned long long *>(stack) + lane);
        else if (lane == 0u) v = (unsigned long long)rt.weight;
        else if (lane == 1u) v = (unsigned long long)rt.bias;
        else if (lane == 2u) v = (unsigned long long)rt.page_table;
        else if (lane == 3u) v = (unsigned long long)rt.shared_page;
        else if (lane == 4u) v = (unsigned long long)rt.ids_out;
        else if (lane == 5u) v = (unsigned long long)rt.weights_out;
        reinterpret_cast<unsigned long long *>(&s_layer[0])[lane] = v;
    }
    if (warp == 1u) {
        uint32_t nj = 0;
        if (lane == 0) {
            abort_flag = 0;
            s_behind = 0;
            s_last = 0;
            s_abort_code = 0x5501u;
            s_n_items = 0;
            s_n_jobs = 0;
            s_n_mix = 0;
        }
        if (lane < 8u) s_prod[lane] = lane == 6u ? 1u : 0u;  // nothing issued yet, no wait has run out
        __syncwarp();
        if (table_param) {
            nj = min(param_table.n_jobs, kJobsMax);
            const uint32_t m0 = param_table.token_job_begin[0];
            const uint32_t nm = min(param_table.token_job_begin[1] - m0, kJobsMax);
            if (lane < nj) s_jobs[0][lane] = param_table.jobs[lane];
            if (lane < nm) {
                const Job &jb = param_table.jobs[param_table.token_jobs[m0 + lane]];
                s_mix_w[0][lane] = jb.weight;
                s_mix_slot[0][lane] = jb.out_index | (jb.is_shared ? 0x80000000u : 0u);
            }
            if (lane == 0) {
                s_n_mix = nm;
                s_n_jobs = nj;
            }
        } else if (early) {
            nj = rt.top_k + (rt.has_shared ? 1u : 0u);
            if (lane == 0) s_n_jobs = nj;
        }
        if (early && lane == 1u) s_n_items = work_list_once(cta, grid, nj, S, RT, KU, KD, s_items, n_early_jobs);
    }
    __syncwarp();
    __syncthreads();
    if (tid == 0) mark(2);
    // a caller's table is complete now; otherwise the routes barrier opens when the routes are picked
    if (tid == 32u && table_param) mbar_arrive(bar(kBarRoutes));

    uint32_t tmem = 0;
    // (s_ep_step: the exchange's step count; s_stamp0: the launch count, shifted: a layer's stamp is
    // s_stamp0 + layer + 1.  Both are read once, by one thread, after the dependency wait of the first
    // layer; the other threads see them after the layer's first barrier.)

    // ---- the copying thread: the units of the CTA's items in order, layer after layer, each one
    // bulk copy (codes and scales, 17 KB of consecutive page bytes) into the next ring slot.  It shares
    // the top of every layer with the other threads (its eight elements of the token), so it works in
    // two steps per layer: after the top of layer l, the rest of layer l's list (waiting, bounded, for the
    // routes where an item needs them), then the head of layer l + 1's list: at most `ring` units of the
    // leading items whose page is known without the routes (the shared expert; every job of a caller's
    // table), which wait only for slots that layer l's own MMAs free.  The head of the first layer is
    // asked for before the token is there.  (p_layer, p_i, p_u): the next unit to ask for. ----
    // Its position lives in shared memory between the steps (one thread reads and writes it), so that
    // it does not hold registers of every thread for the whole kernel.
    auto produce = [&](uint32_t ll, bool head) {
        uint32_t p_slot = s_prod[0], p_round = s_prod[1], p_layer = s_prod[2], p_i = s_prod[3], p_u = s_prod[4];
        uint32_t p_units = s_prod[5];
        bool p_ok = s_prod[6] != 0u;
        auto leave = [&]() {
            s_prod[0] = p_slot, s_prod[1] = p_round, s_prod[2] = p_layer, s_prod[3] = p_i, s_prod[4] = p_u;
            s_prod[5] = p_units, s_prod[6] = p_ok ? 1u : 0u;
        };
        if (p_layer > ll || !p_ok) return;
        const unsigned long long stream_policy = l2_policy_evict_first();
        const uint32_t par_l = ll & 1u;
        const uint32_t n_static = table_param ? s_n_jobs : n_early_jobs;
        bool routes_known = table_param;
        uint32_t n_it = early ? s_n_items : 0u;  // late lists are read after the routes barrier
        uint32_t budget = ring;
#pragma unroll 1
        for (;;) {
            if (!routes_known) {
                const bool is_static = p_i < n_it && ((s_items[p_i] >> 8) & 0xFFu) < n_static;
                if (!is_static) {
                    if (head) return leave();
                    if (ll == 0u) mark(3);
                    // with a list known from the start the copies need only the picked experts' pages, which
                    // are in the job records half a microsecond before the routes' weights are
                    if (!mbar_wait(bar((early && routes_here) ? kBarPages : kBarRoutes), par_l, abortp)) {
                        p_ok = false;
                        return leave();
                    }
                    routes_known = true;
                    n_it = s_n_items;
                    if (routes_here && ll + 1u < L) {
                        // this layer's scores are done: its router rows make room for the next layer's
                        const uint16_t *wrn = s_layer[par_l ^ 1u].router_weight;
                        const uint32_t rows = (cta < rt.n_experts ? 1u : 0u) + (cta + grid < rt.n_experts ? 1u : 0u);
                        mbar_arrive_expect(bar(kBarWr), rows * hidden * 2u);
#pragma unroll 1
                        for (uint32_t k = 0; k < rows; ++k)
                            bulk_copy(smem_u32(sWr) + k * hidden * 2u, wrn + (size_t)(cta + k * grid) * hidden, hidden * 2u, bar(kBarWr));
                    }
                }
            }
            if (p_i >= n_it) break;
            const uint32_t item = s_items[p_i], j = (item >> 8) & 0xFFu, idx = item & 0xFFu;
            const bool down = (item & kItemDown) != 0u;
            const uint32_t nu = down ? KD : KU;
            const uint8_t *page = (!routes_known && !table_param) ? s_layer[par_l].shared_page : s_jobs[par_l][j].page;
            const uint8_t *a = page + (down ? mxfp4_down_offset(hidden, inter) : 0u) + ((size_t)idx * nu + p_u) * kUnitStride;
#pragma unroll 1
            for (; p_u < nu; ++p_u) {
                if (head) {
                    if (budget == 0u) return leave();
                    --budget;
                }
                if (p_round && !mbar_wait(bar(kBarDone + p_slot), (p_round - 1u) & 1u, abortp)) {
                    p_ok = false;
                    return leave();
                }
                const uint32_t full = bar(kBarFull + p_slot);
                mbar_arrive_expect(full, kSlot);
                bulk_copy_stream(smem_u32(sRing) + p_slot * kSlot, a, kSlot, full, stream_policy);
                a += kUnitStride;
                ++p_units;
                if (++p_slot == ring) {
                    p_slot = 0;
                    ++p_round;
                }
            }
            p_u = 0;
            ++p_i;
        }
        p_layer = ll + 1u;  // the list is done
        p_i = 0;
        leave();
    };
    // This CTA's share of a shared expert's page into the L2: units cta, cta + grid, ...
    auto prefetch_shared = [&](const uint8_t *page) {
        if (!page) return;
        const uint32_t units = (uint32_t)(mxfp4_page_bytes(hidden, inter) / kUnitStride);
#pragma unroll 1
        for (uint32_t u = cta; u < units; u += grid) l2_prefetch(page + (size_t)u * kUnitStride, kUnitStride);
    };
    if (is_producer) {
        if (n_early_jobs) prefetch_shared(s_layer[0].shared_page);  // the first layer's, before the token is there
        if (routes_here) {
            // the first layer's router rows; those of layer l + 1 follow when layer l's routes are known
            const uint16_t *wr0 = s_layer[0].router_weight;
            const uint32_t rows = (cta < rt.n_experts ? 1u : 0u) + (cta + grid < rt.n_experts ? 1u : 0u);
            mbar_arrive_expect(bar(kBarWr), rows * hidden * 2u);
#pragma unroll 1
            for (uint32_t k = 0; k < rows; ++k)
                bulk_copy(smem_u32(sWr) + k * hidden * 2u, wr0 + (size_t)(cta + k * grid) * hidden, hidden * 2u, bar(kBarWr));
        }
        produce(0u, true);
    }
    __syncwarp();
    {
        uint32_t gi0 = 0;                       // items of earlier layers
        uint32_t m_slot = warp - kMmaWarp0, m_round = 0;  // issuing threads: position in the CTA's sequence of units
        uint32_t n_loaded = 0;                  // digit tiles of hidden values so far (issuing and tile threads)
        bool alive = true;
#pragma unroll 1
        for (uint32_t l = 0; l < L; ++l) {
            const uint32_t par = l & 1u;
            if constexpr (kTrace) tr = (l == trace_layer) ? trace_base() : nullptr;
            // what a layer of a stack brings of its own; a single layer takes it from the launch arguments
            // (s_layer[par]: what the layer brings of its own, in shared memory since the layer before)
            // the token: the caller's for the first layer, then stamped words written by the mix of the layer before
            // (x_words + par * kMaxHidden: this layer's; the other half: the next layer's)
            // The layer's router rows of this CTA's experts (cta, cta + grid) come into shared memory by
            // bulk copies a layer ahead; the bias of those experts and the page table are parked in shared
            // memory by the threads that need them, right after the routing of the layer before (the first
            // layer's before the token is waited for): with the weight stream saturating the memory, such
            // a load takes microseconds, which nobody may wait for once the token is there.
            float xs[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            if (routes_here && l == 0u) {
                if (warp >= kLoadWarp0 && tid - kLoadWarp0 * 32u < rt.n_experts) {
                    const float *l_bias = stack ? stack[0].bias : rt.bias;
                    const uint8_t *const *l_table = stack ? stack[0].page_table : rt.page_table;
                    s_page[tid - kLoadWarp0 * 32u] = __ldg(reinterpret_cast<const unsigned long long *>(l_table) + (tid - kLoadWarp0 * 32u));
                    s_bias[tid - kLoadWarp0 * 32u] = l_bias ? __ldg(l_bias + (tid - kLoadWarp0 * 32u)) : 0.0f;
                }
            }
            if (l == 0u) {
                cudaGridDependencySynchronize();
                if (tid == 0) {
                    s_ep_step = ep_on ? __ldcg(ep.step) : 0u;
                    s_stamp0 = __ldcg(reinterpret_cast<const uint32_t *>(tiles)) << 6;
                }
            }
            if (l == 0u) {
                if (has_x) {
                    const float4 p0 = __ldcg(reinterpret_cast<const float4 *>(x) + 2u * tid);
                    const float4 p1 = __ldcg(reinterpret_cast<const float4 *>(x) + 2u * tid + 1u);
                    xs[0] = p0.x, xs[1] = p0.y, xs[2] = p0.z, xs[3] = p0.w;
                    xs[4] = p1.x, xs[5] = p1.y, xs[6] = p1.z, xs[7] = p1.w;
                }
            } else {
                // The token of this layer is the output of the one before, as stamped words.  One lane of
                // a warp polls (bounded) one word -- warps that have nothing else to do wait here for most
                // of the layer before, and 75 000 polling threads would flood the L2 --; then every thread
                // takes the words of its eight elements, four loads in flight together, and repeats
                // (bounded) while one of them is not there yet.
                bool ok = alive;
                if (has_x && ok) {
                    const uint32_t want = s_stamp0 + l + 1u;
                    const unsigned long long *mine = x_words + (size_t)par * kMaxHidden + 8u * tid;
                    uint32_t tries = 0;
                    if (lane == 0) {
#pragma unroll 1
                        while ((uint32_t)(ld_relaxed_gpu(mine) >> 32) != want) {
                            if (++tries > kSpinGlobal || abort_flag) {
                                ok = false;
                                break;
                            }
                            __nanosleep(100);
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // (has_x is uniform in a warp)
                    if constexpr (kTrace) {
                        if (l == trace_layer + 1u && lane == 0 && (warp == 0u || warp == 15u)) {
                            unsigned long long *t2 = trace_base();
                            if (t2) t2[85u + (warp ? 2u : 0u)] = (unsigned long long)clock64();
                        }
                    }
#pragma unroll 1
                    while (ok) {
                        ulonglong2 w[4];
                        bool all = true;
#pragma unroll
                        for (uint32_t q = 0; q < 4; ++q) {
                            w[q] = ld_relaxed_gpu2(mine + 2u * q);
                            all = all && (uint32_t)(w[q].x >> 32) == want && (uint32_t)(w[q].y >> 32) == want;
                            xs[2 * q] = __uint_as_float((uint32_t)w[q].x);
                            xs[2 * q + 1] = __uint_as_float((uint32_t)w[q].y);
                        }
                        if (all) break;
                        if (++tries > kSpinGlobal || abort_flag) ok = false;
                        __nanosleep(100);
                    }
                    if (!ok) abort_flag = 1;
                    if constexpr (kTrace) {
                        if (l == trace_layer + 1u && lane == 0 && (warp == 0u || warp == 15u)) {
                            unsigned long long *t2 = trace_base();
                            if (t2) t2[86u + (warp ? 2u : 0u)] = (unsigned long long)clock64();
                        }
                    }
                }
                alive = token_all(ok && !abort_flag);
                if (!alive) break;
                if constexpr (kTrace) {
                    if (l == trace_layer + 1u && tid == 0) {
                        unsigned long long *t2 = trace_base();
                        if (t2) t2[89] = (unsigned long long)clock64();
                    }
                }
            }
            if (tid == 0) mark(4);
            // tensor memory, while the first token is on its way
            if (l == 0u && warp == kMmaWarp0) {
                asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                             "r"(kTmemCols)
                             : "memory");
                asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
                fence_before();
            }

            if (routes_here) {
                // ---- expert scores: logit = x . w in double (warp sums, then the sixteen warps in order),
                // rounded to F32; score and score + bias go to global memory, then the CTA counts itself ----
                double *s_red = reinterpret_cast<double *>(sBh);  // [slot][warp]; no digit tile is in use now
                const bool wr_ok = mbar_wait(bar(kBarWr), par, abortp);
#pragma unroll
                for (uint32_t k = 0; k < kRouterSlots; ++k) {
                    if (cta + k * grid < rt.n_experts) {  // uniform in the CTA
                        uint4 q = make_uint4(0u, 0u, 0u, 0u);
                        if (has_x && wr_ok) q = reinterpret_cast<const uint4 *>(sWr + k * hidden * 2u)[tid];
                        const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
                        double acc0 = 0.0, acc1 = 0.0;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            acc0 += (double)xs[i * 2] * (double)__uint_as_float(wd[i] << 16);
                            acc1 += (double)xs[i * 2 + 1] * (double)__uint_as_float(wd[i] & 0xffff0000u);
                        }
                        const double ws = warp_sum(acc0 + acc1);
                        if (lane == 0) s_red[k * (kTokenThreads / 32u) + warp] = ws;
                    }
                }
                if (tid == 0) mark(64);
                token_sync();
                if (tid == kRouteWarp * 32u) {
                    mark(65);
                }
                // one warp finishes the scores, publishes them and counts the CTA while the other warps
                // turn to the digits
                if (warp == kRouteWarp) {
                    // every CTA writes the word of expert `cta`, whether that expert exists or not: its
                    // stamp also tells the other CTAs that this one has reached the layer
                    if (lane < kRouterSlots && (lane == 0u || cta + lane * grid < rt.n_experts)) {
                        const uint32_t e = cta + lane * grid;
                        float sc = 0.0f;
                        if (e < rt.n_experts) {
                            double sum = 0.0;
#pragma unroll
                            for (uint32_t w = 0; w < kTokenThreads / 32u; ++w) sum += s_red[lane * (kTokenThreads / 32u) + w];
                            sc = router_score_f32(sum, rt.score_fn);
                        }
                        if (e < S14_N_ROUTED_EXPERTS)
                            st_relaxed_gpu(score_words + par * S14_N_ROUTED_EXPERTS + e, ((unsigned long long)(s_stamp0 + l + 1u) << 32) | __float_as_uint(sc));
                    }
                    if (lane == 0) mark(5);
                }
            }

            // the token's digits (they do not depend on the routes)
            if (has_x) digits_of8(xs, tid, sBx, sE);
            fence_async_smem();  // the digit tile is read by the tensor cores
            if (tid == 0) mark(9);
            if (warp == 4u && l + 1u < L && lane < sizeof(StackLayer) / 8u)
                reinterpret_cast<unsigned long long *>(&s_layer[par ^ 1u])[lane] =
                    __ldg(reinterpret_cast<const unsigned long long *>(stack + l + 1u) + lane);  // read from the next layer's top on
            token_sync();        // every block exponent is written, the tensor memory address too; s_red is not read any more
            fence_after();
            tmem = tmem_slot;
            if (tid == 0) mark(10);
            if (warp < 8u) {
                store_digit_scales(tmem + kColSfbX, sE, hidden, warp & 3u, warp >> 2, 2u, lane);
                fence_before();
                mbar_arrive(bar(kBarXReady));
            }
            if (tid == 0) mark(6);
            if (routes_here && warp >= kLoadWarp0) {
                // ---- the routes, by the 256 tile threads: thread e takes expert e.  Every CTA's scores are
                // needed: all CTAs are resident (one per SM), the wait is bounded.  An expert's rank is the
                // number of experts that come before it (larger score + bias, or the same and a lower id);
                // the experts of rank < top_k are the routes, in rank order. ----
                const uint32_t lt = tid - kLoadWarp0 * 32u;
                // thread e polls (bounded) the word of expert e; the words of experts that do not exist
                // but whose number is a CTA's are waited for as well, so that no CTA is a layer behind
                bool ok = true;
                unsigned long long word = 0ull;
                if (lt < rt.n_experts || lt < grid) {
                    const uint32_t want = s_stamp0 + l + 1u;
                    uint32_t tries = 0;
#pragma unroll 1
                    while ((uint32_t)((word = ld_relaxed_gpu(score_words + par * S14_N_ROUTED_EXPERTS + lt)) >> 32) != want) {
                        if (++tries > kSpinGlobal || abort_flag) {
                            ok = false;
                            break;
                        }
                        __nanosleep(20);
                    }
                }
                if (lt == 0) mark(7);
                ok = load_all(ok);
                if (ok) {
                    // Selection by counting, no serial rounds.  A key is (score + bias as an ordered integer,
                    // ~id): all keys differ, a larger key comes first.  Thread e counts the keys of its warp's
                    // 32 experts that beat its own; the experts of rank < top_k within a warp are the warp's
                    // candidates (slot = warp * 8 + rank).  Then one thread per candidate slot counts the
                    // candidates that beat it: rank < top_k among the candidates = the route of that rank.
                    unsigned long long *s_cand = reinterpret_cast<unsigned long long *>(sBh);              // [64] keys, 0 = none
                    float *s_cand_score = reinterpret_cast<float *>(sBh + 512);                            // [64]
                    unsigned long long *s_cand_page = reinterpret_cast<unsigned long long *>(sBh + 1024);  // [64]
                    unsigned long long *s_keys = reinterpret_cast<unsigned long long *>(sBh + 2048);       // [256]
                    const uint32_t wl = warp - kLoadWarp0;
                    unsigned long long key = 0ull;
                    float sc = 0.0f;
                    if (lt < rt.n_experts) {
                        sc = __uint_as_float((uint32_t)word);
                        const uint32_t bits = __float_as_uint(__fadd_rn(sc, s_bias[lt]));
                        const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
                        key = ((unsigned long long)ordered << 32) | (unsigned long long)(0xffffffffu - lt);
                    }
                    if (lt == 0) mark(68);
                    s_keys[lt] = key;
                    if (lane < 8u) s_cand[wl * 8u + lane] = 0ull;
                    __syncwarp();
                    {
                        uint32_t rank = 0;
                        const ulonglong2 *row = reinterpret_cast<const ulonglong2 *>(s_keys + wl * 32u);
#pragma unroll
                        for (uint32_t i = 0; i < 16; ++i) {
                            const ulonglong2 v = row[i];
                            rank += (v.x > key ? 1u : 0u) + (v.y > key ? 1u : 0u);
                        }
                        if (key != 0ull && rank < rt.top_k) {
                            s_cand[wl * 8u + rank] = key;
                            s_cand_score[wl * 8u + rank] = sc;
                            s_cand_page[wl * 8u + rank] = s_page[lt];
                        }
                    }
                    if (lt == 0) mark(69);
                    load_sync();
                    if (lt < 64u) {
                        const unsigned long long mine = s_cand[lt];
                        uint32_t rank = 0;
                        const ulonglong2 *row = reinterpret_cast<const ulonglong2 *>(s_cand);
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i) {
                            const ulonglong2 v = row[i];
                            rank += (v.x > mine ? 1u : 0u) + (v.y > mine ? 1u : 0u);
                        }
                        if (mine != 0ull && rank < rt.top_k) {
                            s_pick_id[rank] = 0xffffffffu - (uint32_t)mine;
                            s_pick_score[rank] = s_cand_score[lt];
                            s_pick_page[rank] = s_cand_page[lt];
                            // (no expert parallelism: the job of route `rank` follows the shared expert's)
                            if (early) s_jobs[par][n_early_jobs + rank].page = reinterpret_cast<const uint8_t *>(s_cand_page[lt]);
                        }
                    }
                    load_sync();  // the picks are written; every candidate's page has been read
                    if (early && lt == 0) mbar_arrive(bar(kBarPages));
                    if (wl == 0u) {
                        __syncwarp();
                        if (lane == 0) mark(71);
                        // The routes from the picked experts (rank order = largest score + bias first, lowest
                        // id on ties): lane j takes route j.  The same sums and weights as k_router's last
                        // block: weight = score / sum of the picked scores x route_scale.  The jobs are the
                        // shared expert first (its page can be asked for before the routes exist), then the
                        // routed experts in route order; the mix is in route order, the shared expert last.
                        // Expert parallel: the rank keeps the jobs of the experts it owns and, as the shared
                        // expert's owner, the shared job; every job writes the row of its route slot.
                        {
                            const uint32_t top_k = rt.top_k;
                            const uint32_t shared_here = (rt.has_shared && rt.shared_owner == rt.ep_rank) ? 1u : 0u;
                            float sum = 0.0f;
#pragma unroll 1
                            for (uint32_t j = 0; j < top_k; ++j) sum = __fadd_rn(sum, s_pick_score[j]);  // every lane, the same order
                            const bool is_route = lane < top_k;
                            const uint32_t id = is_route ? s_pick_id[lane] : 0u;
                            const bool owned = is_route && (rt.ep_world <= 1u || (id % rt.ep_world) == rt.ep_rank);
                            const uint32_t owned_mask = __ballot_sync(0xffffffffu, owned);
                            const uint32_t pos = shared_here + __popc(owned_mask & ((1u << lane) - 1u));
                            if (is_route) {
                                const float w = __fmul_rn(__fdiv_rn(s_pick_score[lane], sum), rt.route_scale);
                                if (cta == 0u && s_layer[par].ids_out) s_layer[par].ids_out[lane] = (int32_t)id;
                                if (cta == 0u && s_layer[par].weights_out) s_layer[par].weights_out[lane] = w;
                                s_mix_w[par][lane] = w;  // every route's weight, also of experts other ranks own
                                s_mix_slot[par][lane] = lane;
                                if (owned) {
                                    s_jobs[par][pos].page = reinterpret_cast<const uint8_t *>(s_pick_page[lane]);
                                    s_jobs[par][pos].kind = S14_PAGE_MXFP4;
                                    s_jobs[par][pos].token = 0;
                                    s_jobs[par][pos].weight = w;
                                    s_jobs[par][pos].is_shared = 0;
                                    s_jobs[par][pos].out_index = lane;
                                }
                            } else if (lane == top_k) {
                                if (shared_here) {
                                    s_jobs[par][0].page = s_layer[par].shared_page;
                                    s_jobs[par][0].kind = rt.shared_kind;
                                    s_jobs[par][0].token = 0;
                                    s_jobs[par][0].weight = 1.0f;
                                    s_jobs[par][0].is_shared = 1;
                                    s_jobs[par][0].out_index = top_k;
                                }
                                if (rt.has_shared) {
                                    s_mix_w[par][top_k] = 1.0f;
                                    s_mix_slot[par][top_k] = top_k | 0x80000000u;
                                }
                                s_n_mix = top_k + (rt.has_shared ? 1u : 0u);
                                s_n_jobs = shared_here + __popc(owned_mask);
                            }
                        }
                        __syncwarp();
                        if (lane == 0 && !early)
                            s_n_items = work_list_once(cta, grid, s_n_jobs, S, RT, KU, KD, s_items, 0u);
                        __syncwarp();
                    }
                } else if (lt == 0) {
                    abort_flag = 1;
                    s_n_items = 0;
                }
                if (lt == 0) {
                    mark(72);
                    mbar_arrive(bar(kBarRoutes));
                }
                if (l + 1u < L && lt < rt.n_experts) {
                    // the next layer's page table and bias (thread e alone reads and writes entry e)
                    const float *nb = stack[l + 1u].bias;
                    s_page[lt] = __ldg(reinterpret_cast<const unsigned long long *>(stack[l + 1u].page_table) + lt);
                    s_bias[lt] = nb ? __ldg(nb + lt) : 0.0f;
                }
            } else if (!routes_here && !table_param && warp == kRouteWarp) {
                const JobTable &tab = *dev_table;
                const uint32_t nj = min(tab.n_jobs, kJobsMax);
                const uint32_t m0 = tab.token_job_begin[0], nm = min(tab.token_job_begin[1] - m0, kJobsMax);
                if (lane < nj) s_jobs[0][lane] = tab.jobs[lane];
                if (lane < nm) {
                    const uint32_t jb = tab.token_jobs[m0 + lane];
                    s_mix_w[0][lane] = tab.jobs[jb].weight;
                    s_mix_slot[0][lane] = tab.jobs[jb].out_index | (tab.jobs[jb].is_shared ? 0x80000000u : 0u);
                }
                if (lane == 0) {
                    s_n_jobs = nj;
                    s_n_mix = nm;
                    s_n_items = work_list_once(cta, grid, nj, S, RT, KU, KD, s_items, 0u);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarRoutes));
            }

            // ---- roles.  Each waits (bounded) until the jobs and the CTA's items are there ----
            const bool is_issuer = (warp == kMmaWarp0 || warp == kMmaWarp0 + 1u) && lane == 0;
            const bool role_thread = is_issuer || warp < kEpiThreads / 32u || warp >= kLoadWarp0;
            // Where the list is known from the start (`early`), only what needs the routes waits for
            // them: the tile threads (which pick them) here, the epilogue before its first item of a
            // routed expert or down item; the issuing threads follow the ring and the tiles.
            bool routes_ok = true, routes_known = early;
            if (role_thread && (!early || warp >= kLoadWarp0)) {
                routes_ok = mbar_wait(bar(kBarRoutes), par, abortp);
                routes_known = true;
            }
            const uint32_t n_jobs = routes_ok ? s_n_jobs : 0u, n_items = routes_ok ? s_n_items : 0u;
            if (kTrace && tid == 0 && tr) tr[15] = n_items | (ring << 8) | (n_jobs << 16);

            if (is_issuer) {
                // ---- MMA issue.  Issuing a tcgen05 operation costs the thread 70-90 cycles (measured), more
                // than a 16 KB unit may take, so two threads issue: thread m takes units m, m + 2, ... of every
                // item (every item has an even number of units and the ring an even number of slots, so a slot
                // always belongs to the same thread, which sees each phase of its barrier) and accumulates
                // into an accumulator of its own.  Items alternate between two accumulator buffers. ----
                const uint32_t m = warp - kMmaWarp0;
                const uint64_t a_desc0 = smem_desc(smem_u32(sRing), 1, 64, 2);
                const uint64_t sf_desc0 = smem_desc(smem_u32(sRing) + kUnitBytes, 0, 8, 0);
                const uint64_t bx_desc0 = smem_desc(smem_u32(sBx), 1, 64, 2);
                const uint32_t sfa_t = tmem + kColSfa + m * 16u;  // a thread's copies and MMAs execute in issue order
                bool ok = n_items == 0u || mbar_wait(bar(kBarXReady), par, abortp);
                uint32_t cur_job = 0xFFFFFFFFu, hb = 0;
#pragma unroll 1
                for (uint32_t i = 0; i < n_items && ok; ++i) {
                    const uint32_t gi = gi0 + i;
                    const uint32_t item = s_items[i], j = (item >> 8) & 0xFFu, buf = gi & 1u;
                    const bool down = (item & kItemDown) != 0u;
                    const uint32_t nu = down ? KD : KU;
                    if (gi >= 2u) ok = mbar_wait(bar(kBarAccFree + buf), ((gi - 2u) >> 1) & 1u, abortp);
                    uint64_t b_desc0 = bx_desc0;
                    uint32_t sfb0 = tmem + kColSfbX;
                    bool last_user = false;
                    if (down) {
                        if (j != cur_job) {
                            hb = n_loaded & 1u;
                            ok = ok && mbar_wait(bar(kBarHReady + hb), (n_loaded >> 1) & 1u, abortp);
                            cur_job = j;
                            ++n_loaded;
                        }
                        b_desc0 = smem_desc(smem_u32(sBh + hb * tile_bytes), 1, 64, 2);
                        sfb0 = tmem + kColSfbH + hb * 128u;
                        last_user = i + 1u >= n_items || ((s_items[i + 1u] >> 8) & 0xFFu) != j;
                    }
                    if (!ok) break;
                    fence_after();
                    const uint32_t acc = tmem + kColAcc + (buf * 2u + m) * 16u;
#pragma unroll 1
                    for (uint32_t ku = m; ku < nu; ku += 2u) {
                        const uint32_t s = m_slot;
                        ok = mbar_wait(bar(kBarFull + s), m_round & 1u, abortp);
                        if (!ok) break;
                        m_slot += 2u;
                        if (m_slot >= ring) {
                            m_slot -= ring;
                            ++m_round;
                        }
                        if (ku == 0u) mark(16u + i * 4u);
                        fence_after();
                        const uint64_t sfd = sf_desc0 + s * (kSlot >> 4);
                        tmem_copy_scales(sfa_t, sfd);
                        tmem_copy_scales(sfa_t + 4u, sfd + (kAtomBytes >> 4));
                        const uint64_t ad = a_desc0 + s * (kSlot >> 4), bd = b_desc0 + ku * (2048u >> 4);
                        const uint32_t sfb_t = sfb0 + ku * 8u;
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk) {
                            const uint32_t atom = kk >> 1, sfid = (kk & 1u) * 2u;
                            umma_mxf4(acc, ad + kk * 2u, bd + kk * 2u, kIdesc | (sfid << 29) | (sfid << 4),
                                      (sfa_t + atom * 4u) | (sfid << 30), (sfb_t + atom * 4u) | (sfid << 30),
                                      (ku >= 2u || kk) ? 1u : 0u);
                        }
                        umma_commit(bar(kBarDone + s));
                    }
                    if (!ok) break;
                    umma_commit(bar(kBarAccDone + buf));
                    if (down && last_user) umma_commit(bar(kBarHFree + hb));
                }
            } else if (warp < kEpiThreads / 32u) {
                // ---- epilogue: the item's two accumulators (sixteen digit columns each) are added in double
                // and rounded once ----
                const uint32_t row = tid;
                const uint32_t lane_base = tmem + ((warp * 32u) << 16);
                bool ok = true;
                if (ep_on && n_items) {
                    // A slot buffer may be written for step s only when every peer has finished reading step
                    // s - 2 from it: each rank tells every other rank the number of steps it has finished
                    // (one 8-byte word per rank in the exchange buffer).
                    // A wait that runs out is reported (status 0x5505) and the step goes on all the same:
                    // the peer whose buffer is then overwritten is hopelessly late, finds later steps' numbers
                    // there (0x5504) and catches up at full speed.  A rank that wrote nothing after such a
                    // wait would leave the late rank waiting for words that never come, and the two would
                    // stay apart for good.
                    if (tid == 0) {
                        const unsigned long long *mine = ep.slots[ep.rank] + 2u * (size_t)(S14_EXPERTS_PER_TOKEN + 1) * hidden + 8u;
                        bool waiting = true;
#pragma unroll 1
                        for (uint32_t p = 0; p < ep.world && waiting; ++p) {
                            if (p == ep.rank) continue;
                            uint32_t tries = 0;
#pragma unroll 1
                            while ((int32_t)((uint32_t)ld_relaxed_sys(mine + p) - s_ep_step + 1u) < 0) {
                                if (abort_flag) {
                                    ok = false;
                                    waiting = false;
                                    break;
                                }
                                if (++tries > ep.wait_limit) {
                                    atomicExch(status, 0x5505u);
                                    waiting = false;
                                    break;
                                }
                                __nanosleep(100);
                            }
                        }
                    }
                    ok = epi_all(ok);
                }
#pragma unroll 1
                for (uint32_t i = 0; i < n_items && ok; ++i) {
                    const uint32_t gi = gi0 + i;
                    const uint32_t item = s_items[i], j = (item >> 8) & 0xFFu, idx = item & 0xFFu, buf = gi & 1u;
                    const bool down = (item & kItemDown) != 0u;
                    bool seen = true;
                    if (!routes_known && (down || j >= n_early_jobs)) {
                        seen = mbar_wait(bar(kBarRoutes), par, abortp);
                        routes_known = true;
                        if (tid == 0) mark(8);
                    }
                    ok = epi_all(seen && mbar_wait(bar(kBarAccDone + buf), (gi >> 1) & 1u, abortp));
                    if (!ok) break;
                    if (tid == 0) mark(17u + i * 4u);
                    fence_after();
                    // the accumulators of the even and of the odd units, one after the other (sixteen registers at a time)
                    double sum = 0.0;
#pragma unroll
                    for (uint32_t half = 0; half < 2; ++half) {
                        uint32_t a[16];
                        tmem_ld16(lane_base + kColAcc + (buf * 2u + half) * 16u, a);
                        tmem_ld_wait();
                        double lo = 0.0, hi = 0.0;  // the digits of lo (columns 8-15) and of hi (0-7): two chains
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            lo += (double)__uint_as_float(a[8 + c]);
                            hi += (double)__uint_as_float(a[c]);
                        }
                        sum += lo + hi;
                    }
                    fence_before();
                    mbar_arrive(bar(kBarAccFree + buf));
                    if (tid == 0) mark(52u + i);
                    const float v = (float)sum;
                    if (!down) {
                        // lanes 0-63: gate of the slice's element `row`; lanes 64-127: its up projection
                        if (row >= 64u) s_up[row - 64u] = v;
                        epi_sync();
                        if (tid == 0 && i == 0u) mark(73);
                        int E = -80;
                        if (row < 64u) {
                            // hidden value `row` of the slice -> sixteen digit nibbles; scale block = warp
                            if (tid == 0 && i == 0u) mark_after(77, __float_as_uint(v) ^ __float_as_uint(s_up[row]));
                            const float hv = swiglu_limit_f32(v, s_up[row]);
                            if (tid == 0 && i == 0u) mark_after(78, __float_as_uint(hv));
                            float bm = fabsf(hv);
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
                            E = block_exponent(bm);
                            if (tid == 0 && i == 0u) mark_after(79, (uint32_t)E);
                            uint32_t hw, lw;
                            digit_codes16(hv, __uint_as_float((uint32_t)(150 - E) << 23), hw, lw);
                            if (tid == 0 && i == 0u) mark_after(74, hw ^ lw);
                            const uint32_t ohw = __shfl_xor_sync(0xffffffffu, hw, 1), olw = __shfl_xor_sync(0xffffffffu, lw, 1);
                            // byte lane / 2 of every row's chunk holds the nibbles of lanes 2b (low) and 2b + 1; even
                            // lanes write digit rows 0-3 and 8-11, odd lanes 4-7 and 12-15
                            const uint32_t e_hw = (lane & 1u) ? ohw : hw, o_hw = (lane & 1u) ? hw : ohw;
                            const uint32_t e_lw = (lane & 1u) ? olw : lw, o_lw = (lane & 1u) ? lw : olw;
#pragma unroll
                            for (uint32_t jj = 0; jj < 4; ++jj) {
                                const uint32_t dj = (lane & 1u) * 4u + jj;
                                s_hst[(dj * 2u + warp) * 16u + (lane >> 1)] =
                                    (uint8_t)(((e_hw >> (4u * dj)) & 0xFu) | (((o_hw >> (4u * dj)) & 0xFu) << 4));
                                s_hst[((8u + dj) * 2u + warp) * 16u + (lane >> 1)] =
                                    (uint8_t)(((e_lw >> (4u * dj)) & 0xFu) | (((o_lw >> (4u * dj)) & 0xFu) << 4));
                            }
                        }
                        epi_sync();
                        if (tid == 0) mark(58u + i);
                        // The slice's 32 chunks (digit row, block) go to their places in the job's digit tile as
                        // stamped words, four bytes of the tile each: thread t < 64 writes half a chunk with one
                        // 16-byte store.  The readers poll the words themselves, so nothing else is published.
                        const unsigned long long stamp_hi = (unsigned long long)(s_stamp0 + l + 1u) << 32;
                        if (tid < 64u) {
                            const uint32_t ch = tid >> 1, half = tid & 1u, dj = ch >> 1, blk = ch & 1u, cc = (idx & 3u) * 2u + blk;
                            const uint2 c8 = *reinterpret_cast<const uint2 *>(s_hst + (dj * 2u + blk) * 16u + half * 8u);
                            const uint32_t o = (idx >> 2) * 2048u + dj * 128u + ((cc ^ (dj & 7u)) << 4) + half * 8u;
                            st_relaxed_gpu2(tile0 + (size_t)j * kTileWordBytes + 2u * o, stamp_hi | c8.x, stamp_hi | c8.y);
                        }
                        if (row < 64u && lane == 0)
                            st_relaxed_gpu(tile_exps + (size_t)j * kExpMax + idx * 2u + warp, stamp_hi | (uint32_t)(E + 100));
                    } else {
                        // row idx * 128 + `row` of the expert's output
                        const uint32_t n = idx * 128u + row, slot = s_jobs[par][j].out_index;
                        if (ep_on) {
                            // into the route slot's row of every rank's slot buffer, the value with the step's
                            // number in one 8-byte store
                            const size_t at = ((size_t)(s_ep_step & 1u) * ep.n_slots + slot) * hidden + n;
                            const unsigned long long word = ((unsigned long long)(s_ep_step + 1u) << 32) | __float_as_uint(v);
#pragma unroll 1
                            for (uint32_t p = 0; p < ep.world; ++p) st_relaxed_sys(ep.slots[p] + at, word);
                        } else {
                            __stcg(d_out + (size_t)slot * hidden + n, v);
                            if (y) {
                                // ---- the ordered mix (examples/s14_vulkan_numeric.rs:936-946): acc = 0; acc += w * d
                                // in route order; acc += d_shared.  Every expert's output row travels as stamped
                                // words; the CTA that holds the row tile of the last job mixes the tile: its
                                // threads poll (bounded) the words of all the jobs, all loads in flight together.
                                // In a stack the result, plus the layer's input if the stack keeps a residual, is
                                // the next layer's token, again as stamped words. ----
                                const uint32_t want = s_stamp0 + l + 1u;
                                st_relaxed_gpu(d_words + (size_t)slot * kMaxHidden + n, ((unsigned long long)want << 32) | __float_as_uint(v));
                                if (j + 1u == n_jobs) {
                                    const uint32_t nm = s_n_mix;
                                    const unsigned long long *dw = d_words + n;
                                    // the layer's input for the residual: asked for now, not after the wait below
                                    // (from the L2: the L1 may hold this word's value of two layers ago)
                                    float x_in = 0.0f;
                                    if (residual)
                                        x_in = l == 0u ? __ldcg(x + n)
                                                       : __uint_as_float((uint32_t)ld_relaxed_gpu(x_words + (size_t)par * kMaxHidden + n));
                                    uint32_t vals[kJobsMax];
                                    uint32_t tries = 0;
                                    bool got = true;
#pragma unroll 1
                                    for (;;) {
                                        uint32_t missing = 0u;
#pragma unroll
                                        for (uint32_t jj = 0; jj < kJobsMax; ++jj) {
                                            // (rows past the mix are not used: any row will do)
                                            const uint32_t r = jj < nm ? (s_mix_slot[par][jj] & 0x7FFFFFFFu) : slot;
                                            // (no branch between the loads: they must all be in flight together)
                                            const unsigned long long t = ld_relaxed_gpu(dw + (size_t)r * kMaxHidden);
                                            const bool own = r == slot;  // this item's own row: the value is at hand
                                            missing |= own ? 0u : ((uint32_t)(t >> 32) ^ want);
                                            vals[jj] = own ? __float_as_uint(v) : (uint32_t)t;
                                        }
                                        if (missing == 0u) break;
                                        if (++tries > kSpinGlobal || abort_flag) {
                                            abort_flag = 1;
                                            got = false;
                                            break;
                                        }
                                        __nanosleep(40);
                                    }
                                    if (got) {
                                        float acc = 0.0f;
#pragma unroll
                                        for (uint32_t jj = 0; jj < kJobsMax; ++jj) {
                                            if (jj < nm) {
                                                const float dv = __uint_as_float(vals[jj]);
                                                acc = (s_mix_slot[par][jj] >> 31) ? __fadd_rn(acc, dv) : __fadd_rn(acc, __fmul_rn(s_mix_w[par][jj], dv));
                                            }
                                        }
                                        const float out = residual ? __fadd_rn(x_in, acc) : acc;
                                        if (l + 1u == L) y[n] = out;
                                        else st_relaxed_gpu(x_words + (size_t)(par ^ 1u) * kMaxHidden + n, ((unsigned long long)(want + 1u) << 32) | __float_as_uint(out));
                                        if (s_layer[par].y_out) s_layer[par].y_out[n] = acc;
                                    }
                                }
                            }
                        }
                    }
                    if (tid == 0) mark(18u + i * 4u);
                }
            } else if (warp >= kLoadWarp0) {
                // ---- digit tiles of the down items: wait (bounded) until every slice of the job has been
                // counted, then take the job's tile from global memory (L2) into one of two tile buffers
                // and its scale codes into tensor memory ----
                const uint32_t lt = tid - kLoadWarp0 * 32u;
                uint32_t cur_job = 0xFFFFFFFFu;
                bool ok = true;
#pragma unroll 1
                for (uint32_t i = 0; i < n_items && ok; ++i) {
                    const uint32_t item = s_items[i], j = (item >> 8) & 0xFFu;
                    if (!(item & kItemDown) || j == cur_job) continue;
                    const uint32_t hb = n_loaded & 1u;
                    bool mine = true;
                    if (lt == 0 && n_loaded >= 2u) mine = mbar_wait(bar(kBarHFree + hb), ((n_loaded >> 1) - 1u) & 1u, abortp);
                    ok = load_all(mine);  // the tile buffer is free
                    if (!ok) break;
                    // The job's tile and block exponents arrive as stamped words from the CTAs that run its
                    // up items.  Every thread asks for all its words at once (a round trip to the L2 costs
                    // a microsecond while the weights stream, so the loads must not follow one another):
                    // eight 16-byte loads of the tile and one exponent; then it asks again (bounded, a
                    // pause between tries) for those that did not carry this layer's stamp yet.
                    const uint32_t want = s_stamp0 + l + 1u;
                    const uint8_t *src = tile0 + (size_t)j * kTileWordBytes;
                    uint8_t *dst = sBh + hb * tile_bytes;
                    if (lt == 0) mark(40u + i);
#pragma unroll 1
                    for (uint32_t k0 = 0; k0 < KD && mine; k0 += 8u) {
                        ulonglong2 v[8];
                        unsigned long long ew = (unsigned long long)want << 32;
                        const bool has_exp = k0 == 0u && lt < (inter >> 5);
                        uint32_t tries = 0;
#pragma unroll
                        for (uint32_t q = 0; q < 8; ++q)
                            if (k0 + q < KD) v[q] = ld_relaxed_gpu2(src + ((size_t)(k0 + q) * kLoadThreads + lt) * 16u);
                        if (has_exp) ew = ld_relaxed_gpu(tile_exps + (size_t)j * kExpMax + lt);
#pragma unroll 1
                        for (;;) {
                            bool all = (uint32_t)(ew >> 32) == want;
#pragma unroll
                            for (uint32_t q = 0; q < 8; ++q)
                                if (k0 + q < KD) all = all && (uint32_t)(v[q].x >> 32) == want && (uint32_t)(v[q].y >> 32) == want;
                            if (all) break;
                            if (++tries > kSpinGlobal || abort_flag) {
                                mine = false;
                                break;
                            }
                            __nanosleep(64);
                            // what is missing, again: all of it in flight together
#pragma unroll
                            for (uint32_t q = 0; q < 8; ++q)
                                if (k0 + q < KD && ((uint32_t)(v[q].x >> 32) != want || (uint32_t)(v[q].y >> 32) != want))
                                    v[q] = ld_relaxed_gpu2(src + ((size_t)(k0 + q) * kLoadThreads + lt) * 16u);
                            if ((uint32_t)(ew >> 32) != want) ew = ld_relaxed_gpu(tile_exps + (size_t)j * kExpMax + lt);
                        }
                        if (mine) {
#pragma unroll
                            for (uint32_t q = 0; q < 8; ++q)
                                if (k0 + q < KD)
                                    *reinterpret_cast<uint2 *>(dst + ((k0 + q) * kLoadThreads + lt) * 8u) = make_uint2((uint32_t)v[q].x, (uint32_t)v[q].y);
                            if (has_exp) sEh[hb][lt] = (uint8_t)ew;
                        }
                    }
                    if (!mine) abort_flag = 1;
                    fence_async_smem();
                    ok = load_all(mine);
                    if (!ok) break;
                    if (lt == 0) mark(46u + i);
                    if (warp < kLoadWarp0 + 4u) {
                        store_digit_scales(tmem + kColSfbH + hb * 128u, sEh[hb], inter, warp & 3u, 0u, 1u, lane);
                        fence_before();
                    }
                    mbar_arrive(bar(kBarHReady + hb));
                    if (lt == 0) mark(19u + i * 4u);
                    cur_job = j;
                    ++n_loaded;
                }
            }
            if (is_producer) {
                // While the routes are being picked the memory is idle: this CTA's share of the NEXT layer's
                // shared expert (its address is known) is asked into the L2, where that layer's copies find
                // it a layer-time later instead of taking HBM time from the routed experts' stream.
                if (n_early_jobs && l + 1u < L) prefetch_shared(s_layer[par ^ 1u].shared_page);
                produce(l, false);
                if (l + 1u < L) produce(l + 1u, true);
                if (l + 1u == L) mark(12);
            }
            // the other lanes of its warp wait here (a warp barrier, no polling) until it has finished:
            // a lane that polls for the next layer's token would take the warp's issue slots from it
            if (warp == kProdWarp) __syncwarp();
            gi0 += n_items;
        }
        if ((warp == kMmaWarp0 || warp == kMmaWarp0 + 1u) && lane == 0) {
            // nothing of this CTA's tensor work is in flight when the tensor memory is freed
            umma_commit(bar(kBarFin));
            mbar_wait(bar(kBarFin), 0, abortp);
        }
    }
    if constexpr (kTrace) tr = trace_base();

    // ---- the CTA's items are done (or given up) ----
    if (is_producer) {
        // copies in flight land in this CTA's shared memory: wait for them before leaving
        const uint32_t p_units = s_prod[5];  // units the copying thread has issued
        const uint32_t first = p_units > ring ? p_units - ring : 0u;
#pragma unroll 1
        for (uint32_t u = first; u < p_units; ++u) {
            const uint32_t s = u % ring, parity = (u / ring) & 1u;
            uint32_t tries = 0;
#pragma unroll 1
            while (!mbar_try(bar(kBarFull + s), parity) && ++tries < kSpin) {
            }
        }
    }
    fence_before();
    __syncwarp();  // the copying and the issuing threads rejoin their warps
    __syncthreads();
    if (tid == 0) mark(13);
    if (warp == kMmaWarp0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
    }
    if (ep_on && ep.wait_and_mix && cta < RT && tid < kEpiThreads && !abort_flag) {
        // ---- exchange: row tile `cta` of every slot arrives in this rank's own buffer from the slot's
        // owner; a thread polls (bounded) one word per slot until it carries this step's number, then
        // the row is mixed in route order, the shared expert last ----
        const uint32_t n = cta * 128u + tid;
        float acc = 0.0f;
        bool ok = true;
#pragma unroll 1
        for (uint32_t jj = 0; jj < ep.n_slots && ok; ++jj) {
            const unsigned long long *w = ep.slots[ep.rank] + ((size_t)(s_ep_step & 1u) * ep.n_slots + jj) * hidden + n;
            unsigned long long got = ld_relaxed_sys(w);
            uint32_t tries = 0;
            // A word with an earlier step's number is waited for.  One with a LATER number means that a
            // peer gave up on this rank and ran ahead: the words this rank still misses belong to
            // steps its peers have left behind and would never come, so it reports that, waits for
            // nothing more in this step and runs at full speed until it is level again.
#pragma unroll 1
            while ((int32_t)((uint32_t)(got >> 32) - (s_ep_step + 1u)) < 0) {
                if (s_behind) break;
                if (++tries > ep.wait_limit || abort_flag) {
                    s_abort_code = 0x5503u;
                    abort_flag = 1;
                    ok = false;
                    break;
                }
                __nanosleep(100);
                got = ld_relaxed_sys(w);
            }
            if ((int32_t)((uint32_t)(got >> 32) - (s_ep_step + 1u)) > 0) {
                s_behind = 1;
                atomicExch(status, 0x5504u);
            }
            const float dv = __uint_as_float((uint32_t)got);
            acc = jj < rt.top_k ? __fadd_rn(acc, __fmul_rn(s_mix_w[0][jj], dv)) : __fadd_rn(acc, dv);
        }
        if (ok && y) y[n] = acc;
    }
    __syncwarp();
    __syncthreads();
    // the last CTA to leave puts the counters back to zero for the next launch
    if (tid == 0) {
        if (abort_flag) atomicExch(status, s_abort_code);
        __threadfence();
        s_last = atomicAdd(counters + kCntExit, 1u) == grid - 1u;
        mark(14);
    }
    __syncwarp();
    __syncthreads();
    if (s_last) {
#pragma unroll 1
        for (uint32_t i = 1u + tid; i < kCntEnd; i += kThreads) counters[i] = 0u;
        if (tid == 0) *reinterpret_cast<uint32_t *>(tiles) = (s_stamp0 >> 6) + 1u;  // the next launch's stamps differ
        if (ep_on && tid == 0) {
            // every CTA has read the step count and finished reading this step's words
            *ep.step = s_ep_step + 1u;
            const size_t credit = 2u * (size_t)(S14_EXPERTS_PER_TOKEN + 1) * hidden + 8u;
#pragma unroll 1
            for (uint32_t p = 0; p < ep.world; ++p)
                if (p != ep.rank) st_relaxed_sys(ep.slots[p] + credit + ep.rank, (unsigned long long)(s_ep_step + 1u));
        }
    }
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
constexpr int kMaxDevices = 64;

// Largest dynamic size the kernel may ask for on a device (the limit minus its static part); 0:
// not configured yet or failed.  The attribute belongs to a device, so it is set once per device,
// with that device current.
size_t g_dynamic_limit[kMaxDevices] = {};

size_t dynamic_limit() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    if (g_dynamic_limit[dev]) return g_dynamic_limit[dev];
    cudaFuncAttributes fa, fb;
    if (cudaFuncGetAttributes(&fa, k_moe_layer_umma<false>) != cudaSuccess) return 0;
    if (cudaFuncGetAttributes(&fb, k_moe_layer_umma<true>) != cudaSuccess) return 0;
    const size_t most = kMaxSmem - (fa.sharedSizeBytes > fb.sharedSizeBytes ? fa.sharedSizeBytes : fb.sharedSizeBytes);
    if (cudaFuncSetAttribute(k_moe_layer_umma<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most) != cudaSuccess) return 0;
    if (cudaFuncSetAttribute(k_moe_layer_umma<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most) != cudaSuccess) return 0;
    g_dynamic_limit[dev] = most;
    return most;
}

// shared memory beside the ring: the token's digit tile, two tiles of hidden values, two router rows
size_t umma_fixed_smem(uint32_t hidden, uint32_t inter) {
    return (size_t)(hidden >> 8) * 2048u + 2u * (size_t)(inter >> 8) * 2048u + (size_t)kRouterSlots * hidden * 2u;
}

// Ring slots that fit beside them: an even number.
uint32_t ring_slots(uint32_t hidden, uint32_t inter, size_t limit) {
    const size_t fixed = umma_fixed_smem(hidden, inter);
    if (limit < fixed + 2u * kSlot) return 0;
    uint32_t r = (uint32_t)((limit - fixed) / kSlot);
    if (r > kMaxRing) r = kMaxRing;
    return r & ~1u;
}

}  // namespace

size_t umma_trace_bytes(int sm_count) { return (size_t)sm_count * kTraceWords * sizeof(unsigned long long); }
uint32_t umma_trace_words() { return kTraceWords; }

size_t umma_scratch_bytes() {
    // the head, then a digit tile and its block exponents per job; zero when the context is created
    return (size_t)kScratchHead + (size_t)kJobsMax * (kTileWordBytes + kExpWordBytes) +
           (size_t)(kJobsMax + 2u) * kMaxHidden * sizeof(unsigned long long);
}

bool umma_layer_ok(int sm_count, uint32_t n_tokens, uint32_t n_jobs_max, uint32_t hidden, uint32_t inter) {
    if (n_tokens != 1u || n_jobs_max == 0u || n_jobs_max > kJobsMax || sm_count <= 0) return false;
    if ((hidden & 511u) || (inter & 511u) || hidden < 512u || inter < 512u || hidden > kMaxHidden || inter > 4096u) return false;
    // no CTA's share may exceed the item list
    uint32_t items[1];
    for (uint32_t c = 0; c < (uint32_t)sm_count; ++c)
        for (uint32_t n_early = 0; n_early < 2u; ++n_early)
            if (layer_work_list(c, (uint32_t)sm_count, n_jobs_max, inter >> 6, hidden >> 7, hidden >> 8, inter >> 8, items, 0,
                                n_early) > kMaxItems)
                return false;
    return ring_slots(hidden, inter, dynamic_limit()) >= 2u;
}

bool umma_router_ok(int sm_count, uint32_t n_experts) {
    return n_experts > 0u && n_experts <= kRouterSlots * (uint32_t)sm_count && n_experts <= S14_N_ROUTED_EXPERTS &&
           sm_count <= (int)kLoadThreads;  // one selecting thread per expert and per CTA's word
}

cudaError_t launch_moe_layer_umma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                                  const float *x, float *d, float *y, uint8_t *tiles, unsigned int *counters,
                                  uint32_t *status, uint32_t hidden, uint32_t inter, const FusedRouter *router,
                                  const EpExchange *ep, unsigned long long *trace, const StackLayer *stack,
                                  uint32_t n_layers, float *hbuf, bool residual) {
    const uint32_t ring = ring_slots(hidden, inter, dynamic_limit());
    if (ring < 2u) return cudaErrorInvalidConfiguration;
    FusedRouter rt = {};
    if (router) rt = *router;
    if (!stack) rt.has_shared = rt.shared_page != nullptr;
    EpExchange ex = {};
    if (ep) ex = *ep;
    if (ex.world > 1u && !router) return cudaErrorInvalidValue;  // the mix needs every route's weight
    if (stack && (!router || n_layers == 0u || n_layers > kMaxLayers || (n_layers > 1u && !hbuf) || ex.world > 1u || rt.ep_world > 1u))
        return cudaErrorInvalidValue;  // a stack routes its own layers on one GPU
    const size_t smem = (size_t)ring * kSlot + umma_fixed_smem(hidden, inter);
    // A programmatic dependent of the previous launch on the single-GPU path.  The expert-parallel
    // paths (exchange inside the kernel, or expert outputs handed to a collective) are ordinary
    // launches; the kernel's own dependency calls are then no-ops.
    const bool pdl = ex.world <= 1u && y != nullptr;
    if (trace)
        return launch_pdl(k_moe_layer_umma<true>, dim3(sm_count), dim3(kThreads), smem, st, pdl, dev, param, x, d, y, tiles,
                          counters, status, hidden, inter, ring, trace, rt, ex, stack, stack ? n_layers : 1u, hbuf,
                          residual ? 1u : 0u);
    return launch_pdl(k_moe_layer_umma<false>, dim3(sm_count), dim3(kThreads), smem, st, pdl, dev, param, x, d, y, tiles,
                      counters, status, hidden, inter, ring, trace, rt, ex, stack, stack ? n_layers : 1u, hbuf,
                      residual ? 1u : 0u);
}

}  // namespace s14
