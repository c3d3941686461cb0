// Internal declarations shared by the kernel file and the C-ABI file.
#ifndef S14_INTERNAL_H
#define S14_INTERNAL_H

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/polaris_s14_cuda.h"

namespace s14 {

// One (expert page, token) pair of a fused layer call.
struct Job {
    const uint8_t *page;
    uint32_t kind;      // S14_PAGE_MXFP4 | S14_PAGE_FP8
    uint32_t token;     // row of x / y
    float weight;       // route weight (unused for the shared expert)
    uint32_t is_shared; // added last with weight 1
    uint32_t out_index; // row of the per-job down outputs this job writes (its job id unless
                        // the caller wants route slots, as the expert-parallel exchange does)
};

constexpr uint32_t kMaxTokens = S14_MAX_BLOCK_TOKENS;
constexpr uint32_t kMaxJobs = kMaxTokens * (S14_EXPERTS_PER_TOKEN + 1);

// Jobs are stored grouped by expert page (so that a page's second reader finds it
// in L2); token_jobs lists each token's jobs in mix order (route order, shared last).
struct JobTable {
    uint32_t n_jobs;
    uint32_t n_tokens;
    uint32_t token_job_begin[kMaxTokens + 1];
    uint8_t token_jobs[kMaxJobs];
    Job jobs[kMaxJobs];
};

// Optional per-kernel timing marks of one routed layer call: events are recorded before the
// router (0), before the up phase (1), between up and down (2), before the mix (3), after it (4).
struct KernelMarks {
    cudaEvent_t ev[5];
};

struct UmmaScratch;

// Expert-parallel exchange of the tcgen05 layer kernel over peer memory.  Every rank holds an
// exchange buffer: two slot buffers [n_slots, hidden] of 8-byte words {F32 bits, step + 1} (steps
// alternate between them), then the rank's own step count (64 bytes), then one 8-byte word per
// rank: the number of steps that rank has finished.  A rank stores the down vectors of the
// experts it owns into the slot rows of EVERY rank's buffer, each value with the step's number in
// one 8-byte store (plain stores to peer memory; an aligned 8-byte store arrives whole, so the
// number validates the value beside it and no fence or flag is needed); each rank polls (bounded)
// the words it needs in its own buffer and mixes from them.  Before a rank writes the slot buffer
// of step s it waits (bounded) until every peer has finished step s - 2, the last reader of that
// buffer; a rank that owns nothing in a step is waited for in this way too.  world <= 1: no exchange.
constexpr uint32_t kMaxEpWorld = 8;
struct EpExchange {
    unsigned long long *slots[kMaxEpWorld];  // rank p's exchange buffer, as mapped on this rank
    uint32_t *step;                // this rank's step count (device memory, kept by the kernel)
    uint32_t world, rank;
    uint32_t n_slots;              // top_k (+ 1 with a shared expert)
    uint32_t wait_and_mix;         // 0: publish only (single-GPU emulation of the other ranks)
    uint32_t wait_limit;           // polls (about a microsecond each) of one word before the rank gives up
};
inline size_t ep_exchange_slot_bytes(uint32_t hidden) {
    return sizeof(unsigned long long) * 2u * (S14_EXPERTS_PER_TOKEN + 1) * hidden;
}
inline size_t ep_exchange_bytes(uint32_t hidden) {
    return ep_exchange_slot_bytes(hidden) + 64u + sizeof(unsigned long long) * kMaxEpWorld;
}

// What the router reads and writes, for a layer call that computes its own routes: the tcgen05
// layer kernel scores the experts in its first microseconds (every CTA a few of them), and every
// CTA then picks the routes from the scores; other layer kernels run k_router first.
struct FusedRouter {
    const uint16_t *weight;            // [n_experts, hidden] BF16
    const float *bias;                 // [n_experts] or NULL
    float *scores, *select;            // [n_experts] scratch: score, score + bias
    uint32_t n_experts, score_fn, top_k;
    float route_scale;
    int32_t *ids_out;                  // [top_k] or NULL
    float *weights_out;                // [top_k] or NULL
    JobTable *table_out;               // the device job table k_router fills
    const uint8_t *const *page_table;  // [n_experts] expert pages (MXFP4)
    const uint8_t *shared_page;        // or NULL
    uint32_t shared_kind;
    uint32_t ep_rank, ep_world, shared_owner;
    uint32_t has_shared;               // every layer has a shared expert (a stack's layers say where)
};

// What one layer of a decode stack brings of its own (device memory, constant during a step): the
// tcgen05 layer kernel walks an array of these in one launch, the output of a layer (plus its input,
// if the stack keeps a residual) being the next layer's token.  Router shape, score function, top_k
// and page kind are the stack's and come with FusedRouter.
struct StackLayer {
    const uint16_t *router_weight;     // [n_experts, hidden] BF16
    const float *bias;                 // [n_experts] or NULL
    const uint8_t *const *page_table;  // [n_experts] expert pages (MXFP4)
    const uint8_t *shared_page;        // MXFP4 page; NULL only if no layer of the stack has one
    int32_t *ids_out;                  // [top_k] or NULL: the layer's route
    float *weights_out;                // [top_k] or NULL
    float *y_out;                      // [hidden] or NULL: the layer's MoE output before the residual
};

cudaError_t launch_mxfp4_matvec(cudaStream_t st, uint32_t mode, int sm_count, const float *x,
                                const uint8_t *w, const uint8_t *s, float *y, uint32_t n, uint32_t k);
cudaError_t launch_fp8_matvec(cudaStream_t st, uint32_t mode, int sm_count, uint32_t scale_format,
                              uint32_t n_tokens, const float *x, const uint8_t *w, const void *s,
                              float *y, uint32_t n, uint32_t k);
cudaError_t launch_swiglu_limit(cudaStream_t st, const float *gate, const float *up, float *y,
                                uint32_t n);
cudaError_t launch_route_mix(cudaStream_t st, const float *expert, float *routed, uint32_t n,
                             float weight);
cudaError_t launch_moe_accumulate(cudaStream_t st, const float *expert, float *acc, uint32_t n,
                                  float weight);
// Which implementation the calling thread's last launch_moe_layer chose (S14_LAYER_PATH_* of the header).
uint32_t last_layer_path();
// Returns the number of kernels launched.  h: [kMaxJobs, inter], d: [kMaxJobs, hidden].
int launch_moe_layer(cudaStream_t st, uint32_t mode, int sm_count, const JobTable *dev_table,
                     const JobTable &param_table, uint32_t n_tokens, uint32_t n_jobs_max,
                     uint32_t hidden, uint32_t inter, const float *x, float *h, float *d, float *y,
                     cudaError_t *err, const KernelMarks *km = nullptr, bool all_mxfp4 = false,
                     unsigned int *counters = nullptr, const struct UmmaScratch *umma = nullptr,
                     const FusedRouter *router = nullptr, const EpExchange *ep = nullptr);
// Scratch of the tcgen05 layer kernel (s14_moe_umma.cu): per job the digit tile of its hidden
// values and the tile's block exponents (umma_scratch_bytes), and the device status word a
// timed-out wait sets.
struct UmmaScratch {
    uint8_t *tiles;
    uint32_t *status;
    unsigned long long *trace;  // per-CTA time marks of the last launch (profiling runs), or nullptr
};
size_t umma_scratch_bytes();
size_t umma_trace_bytes(int sm_count);
uint32_t umma_trace_words();
// One token, every job an MXFP4 page, hidden and inter multiples of 512 that fit shared and tensor memory.
// Sets the kernel's shared-memory attribute for the current device on first use.
bool umma_layer_ok(int sm_count, uint32_t n_tokens, uint32_t n_jobs_max, uint32_t hidden, uint32_t inter);
// Whether the tcgen05 layer kernel can score n_experts itself (a CTA scores at most two; at most 256 CTAs).
bool umma_router_ok(int sm_count, uint32_t n_experts);
// The items CTA c of G runs, in order (see s14_moe_umma.cu); returns their number, writes at most cap.
__host__ __device__ uint32_t layer_work_list(uint32_t c, uint32_t G, uint32_t n_jobs, uint32_t S, uint32_t RT,
                                             uint32_t KU, uint32_t KD, uint32_t *items, uint32_t cap, uint32_t n_early);
// Both phases and the mix in one launch (y == nullptr: the expert outputs go to d, the caller mixes).
// With a router the kernel computes the routes itself and the job tables are not read.
cudaError_t launch_moe_layer_umma(cudaStream_t st, int sm_count, const JobTable *dev, const JobTable &param,
                                  const float *x, float *d, float *y, uint8_t *tiles, unsigned int *counters,
                                  uint32_t *status, uint32_t hidden, uint32_t inter,
                                  const FusedRouter *router = nullptr, const EpExchange *ep = nullptr,
                                  unsigned long long *trace = nullptr, const StackLayer *stack = nullptr,
                                  uint32_t n_layers = 1, float *hbuf = nullptr, bool residual = false);
int launch_router(cudaStream_t st, const s14_router_desc &r, float *scores, float *select,
                  JobTable *table_out, const uint8_t *const *page_table, const uint8_t *shared_page,
                  uint32_t shared_kind, unsigned int *counter, cudaError_t *err,
                  const KernelMarks *km = nullptr, uint32_t ep_rank = 0, uint32_t ep_world = 1,
                  uint32_t shared_owner = 0);
// out[i] = residual ? x[i] + y[i] : y[i]; y_copy (or NULL) also receives y (a stack's layers launched one by one).
cudaError_t launch_stack_step(cudaStream_t st, const float *x, const float *y, float *out, float *y_copy,
                              uint32_t n, bool residual);
cudaError_t launch_mix_slots(cudaStream_t st, const float *slots, const float *weights, uint32_t n_routed,
                             int has_shared, float *y, uint32_t hidden);
cudaError_t launch_head_logits(cudaStream_t st, int sm_count, const float *x, uint32_t n_tokens,
                               const uint16_t *w, uint32_t n_rows, uint32_t hidden, float *out,
                               uint32_t out_stride);
cudaError_t launch_greedy_argmax(cudaStream_t st, const float *logits, uint32_t vocab,
                                 int64_t *result);

// ---- a block of tokens through one layer, grouped by expert (s14_moe_block.cu) ----
constexpr uint32_t kBlockNt = 12;  // most tokens of one chunk (two MMAs of N = 96: sixteen digit rows per token)
// Up to kBlockNt (token, route) pairs that share an expert page.  The chunks of one expert follow
// one another: c0 is the first of them, nch their number.
struct BlockChunk {
    const uint8_t *page;
    uint32_t nt;               // pairs in the chunk
    uint32_t c0, nch;
    uint32_t tok[kBlockNt];    // the pairs' tokens (rows of x)
    uint32_t pair[kBlockNt];   // token * 7 + position in the mix (6: the shared expert)
    uint32_t pad;
};
// Device workspace of a block object, sized for max_tokens at creation.
struct BlockWork {
    BlockChunk *chunks;
    uint32_t *counts;          // [0] chunks, [1] up items, [2] down items, [3] an expert id was out of range
    uint8_t *xdig, *xexp;      // the tokens' digit tiles and block exponents
    uint8_t *hdig, *hexp;      // the pairs' hidden values likewise
    float *d;                  // the pairs' expert outputs [pair, hidden]
    float *hval;               // official arithmetic: the pairs' weighted hidden values [pair, inter] (NULL until asked for)
};
// Expert-parallel exchange of the block kernels over peer memory: every rank holds two pair buffers
// [pairs, hidden] F32 (calls alternate between them) and, per buffer, one 8-byte word per rank: the number
// of the last call whose rows that rank has written there.  The down kernel stores the rows of the experts it
// owns into every rank's buffer (plain stores to peer memory) and its last CTA publishes the call's number;
// the mix waits (bounded) until every rank's word says this call.  A rank writes call s + 1 only after its own
// mix of call s, which waited for every rank's rows of call s; so a rank that writes into a buffer for call
// s + 2 knows that every rank has finished reading call s from it: two buffers are enough.
struct BlockEp {
    float *pairs_peer[kMaxEpWorld];               // the call's pair buffer of rank p, as mapped on this rank
    unsigned long long *flags_peer[kMaxEpWorld];  // ... its flag words [world]
    const unsigned long long *flags;              // this rank's own flag words of the call's buffer
    unsigned int *counter;                        // arrival counter of the down kernel's CTAs (zero at rest)
    uint32_t world, rank, call, wait_limit;
};
// Whether the grouped tensor-core kernels can run these sizes on the current device.
bool moe_block_ok(int sm_count, uint32_t hidden, uint32_t inter, uint32_t n_experts, uint32_t top_k);
size_t moe_block_max_chunks(uint32_t max_tokens);
// ids / weights: device [n_tokens, top_k] (a negative id: no route); pages: device [n_tokens, top_k] page of every
// route, or NULL with page_table [n_experts].  Returns the number of kernels launched.
int launch_moe_block(cudaStream_t st, int sm_count, const BlockWork &w, const float *x, float *y, const int32_t *ids,
                     const float *weights, const uint8_t *const *pages, const uint8_t *const *page_table,
                     const uint8_t *shared_page, uint32_t n_tokens, uint32_t top_k, uint32_t n_experts, uint32_t hidden,
                     uint32_t inter, uint32_t *status, cudaError_t *err, uint32_t nt_cap = 0, bool residual = false,
                     uint32_t ep_rank = 0, uint32_t ep_world = 1, float *pairs_out = nullptr, const BlockEp *ep = nullptr,
                     bool shared_by_token = false, bool official = false);
// With pairs_out (expert parallel: rank ep_rank of ep_world computes the experts e with e mod world == rank) the
// pairs' expert outputs [n_tokens * 7, hidden] go there, zero where another rank owns the expert, and no mix runs;
// launch_block_mix mixes such a buffer once the ranks' buffers have been added up (x: the layer's input for a residual, or NULL).
cudaError_t launch_block_mix(cudaStream_t st, const float *pairs, const int32_t *ids, const float *weights, uint32_t n_tokens,
                             uint32_t top_k, bool has_shared, const float *x, float *y, uint32_t hidden, const uint32_t *counts,
                             const BlockEp *ep = nullptr, uint32_t *status = nullptr);
// Scores and routes of many tokens (s14_kernels.cu): the tokens of a tile share the router rows in
// shared memory; one warp per token selects.  Same arithmetic as launch_router.  Returns the number
// of kernels launched.
int launch_router_batch(cudaStream_t st, const s14_router_desc &r, float *scores, float *select, cudaError_t *err);

// ---- the steps on either side of the MoE inside one layer (s14_glue.cu) ----
// dots: [n_tokens, 24] scratch, mean_sq: [n_tokens] scratch.  Returns the number of kernels launched.
int launch_hc_pre(cudaStream_t st, bool bf16, bool head, uint32_t n_tokens, uint32_t hidden, const void *x, const float *fn,
                  const float *scale, const float *base, float norm_eps, uint32_t iters, float hc_eps, float *dots, float *mean_sq,
                  void *reduced, float *post, float *comb, float *pre, cudaError_t *err);
cudaError_t launch_hc_post(cudaStream_t st, bool bf16, uint32_t n_tokens, uint32_t hidden, const void *branch, const void *residual,
                           const float *post, const float *comb, void *merged);
cudaError_t launch_rms_norm(cudaStream_t st, bool bf16, uint32_t n_tokens, uint32_t hidden, const void *x, const float *w, float eps,
                            void *out);
cudaError_t launch_router_hash(cudaStream_t st, const s14_router_desc &r, const int64_t *tid2eid);
cudaError_t launch_bf16_to_f32(cudaStream_t st, const uint16_t *in, float *out, uint32_t n);
cudaError_t launch_f32_to_bf16(cudaStream_t st, const float *in, uint16_t *out, uint32_t n);

}  // namespace s14


#endif
