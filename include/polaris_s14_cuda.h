/*
 * polaris_s14_cuda.h - C ABI of the B200 (sm_100a) implementation of the S14 MoE
 * expert hot path: MXFP4 w1/w3 matvec -> limit-10 SwiGLU -> w2 matvec ->
 * route-weighted mix over the routed experts plus the shared expert, the FP8
 * E4M3 block-scaled projection matvec, and the router's (score+bias) top-k.
 *
 * This is the boundary a Rust `-sys` crate (or any FFI) binds.  Every entry
 * point names the reference interface it stands in for, by file:line inside
 * the reference project.  Conventions:
 *   - plain pointers and sizes only; device buffers are {pointer, size} pairs;
 *   - every call returns an int32 status (0 = ok); the message of the last
 *     failure on the calling thread is returned by s14_last_error();
 *   - `stream` is a cudaStream_t passed as void* (NULL = the context's compute
 *     stream); "cmd_" calls only enqueue work, exactly as the reference's
 *     cmd_* calls only record into a command buffer: uploads, ordering against
 *     other streams and read-back stay with the caller;
 *   - a context is bound to one device and is not thread-safe.
 * There is no CPU fallback anywhere behind this header.
 */
#ifndef POLARIS_S14_CUDA_H
#define POLARIS_S14_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define S14_API __attribute__((visibility("default")))

/* ---- status codes -------------------------------------------------------- */
#define S14_OK 0
#define S14_ERR_CONTRACT 1 /* shape / capacity / weight / route contract violated */
#define S14_ERR_CUDA 2     /* a CUDA runtime call failed */
#define S14_ERR_POOL 3     /* page pool state: full, stale generation, not loading ... */
#define S14_ERR_CODE 4     /* a NaN code (UE8M0 0xFF, E4M3 0x7F/0xFF) in a payload */
#define S14_ERR_DEVICE 5   /* the device status word reported a problem */

/* reference: scheduler/s14_runner/src/memory.rs:3, ssd_inference/src/s14_vulkan.rs:14-18 */
#define S14_EXPERT_PAGE_BYTES 13369344ull
#define S14_SHARED_EXPERT_PAGE_BYTES 25167360ull
#define S14_ROUTED_EXPERT_KIND 0x53
#define S14_SHARED_EXPERT_KIND 0x54
/* reference: scheduler/s14_runner/src/contract.rs:6-13 */
#define S14_HIDDEN_SIZE 4096u
#define S14_N_ROUTED_EXPERTS 256u
#define S14_EXPERTS_PER_TOKEN 6u
#define S14_MAX_BLOCK_TOKENS 8u /* largest exact-cascade verify block, cascade.rs:19 */

/* Page encodings understood by the fused layer kernels. */
#define S14_PAGE_MXFP4 0u /* [w1][w3][w2] E2M1 codes, then [s1][s3][s2] UE8M0 per 32 */
#define S14_PAGE_FP8 1u   /* [w1][w3][w2] E4M3 codes, then [s1][s3][s2] UE8M0 per 128x128 */

/* Summation order of every matvec of a context.
 *   S14_ACCUM_PAIRWISE  : the fast path.  Every product x * w is exact and the products of a row
 *                         are added in a wider format than F32, then rounded to F32 once per
 *                         row: the result is the reference's dot product with the accumulator
 *                         widened to double (what the reference's Python code computes with
 *                         accumulation_dtype=float64, local_s14_primitives/mxfp4.py:172-275).
 *                         One-token layers of MXFP4 pages run on the tensor cores (activations
 *                         as sixteen base-8 digit rows, tcgen05 block-scaled MMA, columns added
 *                         in double); everything else on F32 / F64 register kernels (a warp per
 *                         row, F32 inside a scale block, F64 across blocks and lanes).
 *   S14_ACCUM_REFERENCE : one thread per output row, k ascending, two separate
 *                         multiply-then-add steps per packed byte, (x*w)*s - the
 *                         exact evaluation order of the reference's F32 CPU code
 *                         (examples/s14_vulkan_numeric.rs:1669-1714); bit-identical
 *                         to it, and slower. */
#define S14_ACCUM_PAIRWISE 0u
#define S14_ACCUM_REFERENCE 1u

/* Router score function (executor.py:641-642 uses sqrt(softplus)). */
#define S14_SCORE_SIGMOID 0u
#define S14_SCORE_SQRT_SOFTPLUS 1u

/* FP8 block-scale storage (s14_fp8_matvec.comp:51-53 uses UE8M0 bytes;
 * local_s14_primitives/fp8.py:37-46 also accepts floats). */
#define S14_SCALE_UE8M0 0u
#define S14_SCALE_F32 1u

typedef struct s14_ctx s14_ctx;
typedef struct s14_pool s14_pool;
typedef struct s14_moe_pages s14_moe_pages;

S14_API const char *s14_last_error(void);

/* ---- context: replaces VulkanContext::init + S14NumericPipelines::new/destroy
 *      (ssd_inference/src/device.rs:26-76, s14_vulkan.rs:195-205, 417-424) ------ */
S14_API int32_t s14_ctx_create(int32_t device, s14_ctx **out);
S14_API int32_t s14_ctx_destroy(s14_ctx *ctx);
S14_API void *s14_ctx_compute_stream(s14_ctx *ctx);
S14_API void *s14_ctx_copy_stream(s14_ctx *ctx);
S14_API int32_t s14_ctx_synchronize(s14_ctx *ctx);
S14_API int32_t s14_ctx_set_accumulation(s14_ctx *ctx, uint32_t mode);
S14_API uint32_t s14_ctx_accumulation(const s14_ctx *ctx);
S14_API int32_t s14_ctx_sm_count(const s14_ctx *ctx);
/* Reads and clears the device status word (0 = no kernel reported a problem). */
S14_API int32_t s14_ctx_device_status(s14_ctx *ctx, uint32_t *status);
/* Number of kernels this context has launched since creation. */
S14_API uint64_t s14_ctx_launch_count(const s14_ctx *ctx);
/* Which implementation the context's last MoE layer or stack call ran (the library chooses by
 * accumulation mode, page kinds, token count and sizes; no counterpart in the reference):
 * exactly one of the first five values, ORed with ROUTER_KERNEL if the routes came from a kernel
 * launch of their own instead of being picked inside the layer kernel.  0: no such call yet. */
#define S14_LAYER_PATH_TENSOR 1u           /* tcgen05 layer kernel, one launch per layer-token */
#define S14_LAYER_PATH_TENSOR_PER_TOKEN 2u /* a block of tokens: one launch of it per token */
#define S14_LAYER_PATH_TENSOR_STACK 3u     /* a whole stack of layers in one launch of it */
#define S14_LAYER_PATH_F32 4u              /* F32 register kernels, pairwise order */
#define S14_LAYER_PATH_REFERENCE 5u        /* reference-order kernels */
#define S14_LAYER_PATH_TENSOR_BLOCK 6u     /* grouped tcgen05 kernels: every expert page streamed once per block */
#define S14_LAYER_PATH_ROUTER_KERNEL 0x100u
S14_API uint32_t s14_ctx_last_layer_path(const s14_ctx *ctx);

/* Per-kernel timing of s14_cmd_routed_moe_layer for profiling runs: while enabled,
 * every such call records CUDA events around its kernels, waits for the stream and
 * accumulates the durations (router, up phase, down phase, mix), the counterpart of
 * the reference's timestamp queries (examples/s14_vulkan_numeric.rs:1088-1101,
 * 1220-1260).  Not for timed throughput runs: the call becomes blocking. */
S14_API int32_t s14_ctx_set_kernel_timing(s14_ctx *ctx, int32_t enable);
S14_API int32_t s14_ctx_kernel_times(s14_ctx *ctx, double ms_out[4], uint64_t *calls);

/* Time marks inside the tensor-core layer kernel, for profiling runs (no counterpart in the
 * reference): while enabled, the kernel's launches run a second build of the kernel in which every
 * CTA writes words_per_cta (96) words: word 0 the GPU's global timer (ns) at entry, the others SM
 * clock values taken in the second layer of a stack (in the only layer of a single-layer launch):
 * 2 set-up done, 4 token read, 64 router dot products, 5 scores written, 9 token digits written,
 * 6 their scales in tensor memory, 7 all scores seen, 68 keys made, 69 first selection level,
 * 71 second level, 72 routes written, 8 routes known to the epilogue; per item i of the CTA's list
 * (i < 5): 16+4i first unit in shared memory, 17+4i accumulators complete, 52+i accumulators read,
 * 58+i hidden digits made (up items), 18+4i epilogue done, 40+i digit tile asked for, 46+i tile in
 * shared memory, 19+4i tile ready (down items); 12 all copies issued, 13 items done, 14 exit;
 * 85/86 (warp 0) and 87/88 (warp 15): the NEXT layer's token: first word seen, all words taken; 89
 * every warp has its words;
 * word 15 = items | ring slots << 8 | jobs << 16.  A word that was not written is 0.  read copies
 * the marks of the last launch ([n_ctas][words_per_cta]). */
S14_API int32_t s14_ctx_set_layer_trace(s14_ctx *ctx, int32_t enable);
S14_API int32_t s14_ctx_read_layer_trace(s14_ctx *ctx, uint64_t *out, uint32_t cap_words, uint32_t *n_ctas,
                                         uint32_t *words_per_cta);

/* ---- byte contracts: S14MatvecShape (s14_vulkan.rs:40-114) ------------------- */
typedef struct {
    uint32_t n;
    uint32_t k;
} s14_matvec_shape;

S14_API int32_t s14_shape_new(uint32_t n, uint32_t k, s14_matvec_shape *out);
S14_API int32_t s14_shape_validate_mxfp4(s14_matvec_shape shape);
S14_API int32_t s14_shape_validate_fp8(s14_matvec_shape shape);
S14_API int32_t s14_shape_fp32_input_bytes(s14_matvec_shape shape, uint64_t *out);
S14_API int32_t s14_shape_fp32_output_bytes(s14_matvec_shape shape, uint64_t *out);
S14_API int32_t s14_shape_mxfp4_weight_bytes(s14_matvec_shape shape, uint64_t *out);
S14_API int32_t s14_shape_mxfp4_scale_bytes(s14_matvec_shape shape, uint64_t *out);
S14_API int32_t s14_shape_fp8_weight_bytes(s14_matvec_shape shape, uint64_t *out);
S14_API int32_t s14_shape_fp8_scale_bytes(s14_matvec_shape shape, uint64_t *out);

/* MXFP4 expert page = up | down in one pool slot (S14_EXPERT_PAGE_BYTES at hidden 4096,
 * intermediate 2048): the bytes of the six checkpoint tensors, stored so that everything the
 * tcgen05 layer kernel fetches in one step is one contiguous run, already in the order the tensor
 * cores read shared memory.  A unit is 128 matrix rows x 256 K-elements: 16 KB of E2M1 codes, 128
 * rows of 128 bytes, the 16-byte chunk (one scale block, low nibble = even k) number c of row m at
 * position c ^ (m % 8), then the rows' UE8M0 codes for the unit's eight scale blocks as two atoms of
 * 512 bytes (four blocks each) in the order the block-scaled MMA takes scales into tensor memory:
 * byte (m % 32) * 16 + (m / 32) * 4 + block % 4.  17 408 bytes per unit.
 *   up      [inter/64 slices][hidden/256 units]: rows 0-63 of a unit are w1 rows of the slice,
 *           rows 64-127 the same rows of w3;
 *   down    [hidden/128 row tiles][inter/256 units] of w2.
 * hidden and intermediate must be multiples of 256.  A "tensor page" is the six tensors one after
 * the other in the checkpoint's ABI (w1 | w3 | w2 | s1 | s3 | s2); these host functions convert
 * between the two, once, at load time.  The reference fixes no layout inside a slot
 * (examples/s14_vulkan_numeric.rs:331-366 uploads six buffers), so they have no counterpart
 * there.  FP8 pages keep their tensors unchanged. */
S14_API int32_t s14_mxfp4_expert_page_from_tensors(uint32_t hidden, uint32_t inter, const uint8_t *tensor_page,
                                                   uint8_t *page);
S14_API int32_t s14_mxfp4_expert_page_to_tensors(uint32_t hidden, uint32_t inter, const uint8_t *page,
                                                 uint8_t *tensor_page);

/* validate_ue8m0_codes / validate_e4m3fn_codes (s14_vulkan.rs:143-156): host
 * bytes, checked before upload.  On failure *bad_index (may be NULL) receives the
 * first offending byte. */
S14_API int32_t s14_validate_ue8m0_codes(const uint8_t *codes, uint64_t len, uint64_t *bad_index);
S14_API int32_t s14_validate_e4m3fn_codes(const uint8_t *codes, uint64_t len, uint64_t *bad_index);

/* ---- the five primitive operators: S14NumericPipelines::bind_* / cmd_*
 *      (s14_vulkan.rs:207-415).  bind validates shapes and capacities and fills a
 *      dispatch record; cmd enqueues it. ---------------------------------------- */
typedef struct {
    void *ptr;     /* device pointer */
    uint64_t size; /* bytes available at ptr */
} s14_buffer;

typedef struct {
    s14_matvec_shape shape;
    const float *x;
    const uint8_t *packed_weight;
    const uint8_t *weight_scale;
    float *y;
} s14_mxfp4_dispatch;

typedef struct {
    s14_matvec_shape shape;
    uint32_t scale_format; /* S14_SCALE_UE8M0 | S14_SCALE_F32 */
    uint32_t n_tokens;     /* 1..8 rows of x / y, row stride k / n floats */
    const float *x;
    const uint8_t *weight;
    const void *weight_scale;
    float *y;
} s14_fp8_dispatch;

typedef struct {
    uint32_t n;
    const float *gate;
    const float *up;
    float *y;
} s14_swiglu_limit_dispatch;

typedef struct {
    uint32_t n;
    float route_weight;
    const float *expert;
    float *routed;
} s14_route_mix_dispatch;

typedef struct {
    uint32_t n;
    float weight;
    const float *expert;
    float *accumulator;
} s14_moe_accumulate_dispatch;

/* bind_mxfp4 (s14_vulkan.rs:207-237) / cmd_mxfp4_matvec (:338-351) */
S14_API int32_t s14_bind_mxfp4(s14_ctx *ctx, s14_matvec_shape shape, const s14_buffer *x,
                               const s14_buffer *packed_weight, const s14_buffer *weight_scale,
                               const s14_buffer *y, s14_mxfp4_dispatch *out);
S14_API int32_t s14_cmd_mxfp4_matvec(s14_ctx *ctx, void *stream, const s14_mxfp4_dispatch *dispatch);

/* bind_fp8 (s14_vulkan.rs:239-269) / cmd_fp8_matvec (:355-368).  The _ex form adds
 * the two options the reference's callers need around it: F32 block scales and
 * 1..8 tokens per weight pass. */
S14_API int32_t s14_bind_fp8(s14_ctx *ctx, s14_matvec_shape shape, const s14_buffer *x,
                             const s14_buffer *weight, const s14_buffer *weight_scale,
                             const s14_buffer *y, s14_fp8_dispatch *out);
S14_API int32_t s14_bind_fp8_ex(s14_ctx *ctx, s14_matvec_shape shape, uint32_t scale_format,
                                uint32_t n_tokens, const s14_buffer *x, const s14_buffer *weight,
                                const s14_buffer *weight_scale, const s14_buffer *y,
                                s14_fp8_dispatch *out);
S14_API int32_t s14_cmd_fp8_matvec(s14_ctx *ctx, void *stream, const s14_fp8_dispatch *dispatch);

/* bind_swiglu_limit (s14_vulkan.rs:271-291) / cmd_swiglu_limit (:370-384) */
S14_API int32_t s14_bind_swiglu_limit(s14_ctx *ctx, uint32_t n, const s14_buffer *gate,
                                      const s14_buffer *up, const s14_buffer *y,
                                      s14_swiglu_limit_dispatch *out);
S14_API int32_t s14_cmd_swiglu_limit(s14_ctx *ctx, void *stream,
                                     const s14_swiglu_limit_dispatch *dispatch);

/* bind_route_mix (s14_vulkan.rs:293-314) / cmd_route_mix (:386-400): routed = w * expert */
S14_API int32_t s14_bind_route_mix(s14_ctx *ctx, uint32_t n, float route_weight,
                                   const s14_buffer *expert, const s14_buffer *routed,
                                   s14_route_mix_dispatch *out);
S14_API int32_t s14_cmd_route_mix(s14_ctx *ctx, void *stream, const s14_route_mix_dispatch *dispatch);

/* bind_moe_accumulate (s14_vulkan.rs:316-334) / cmd_moe_accumulate (:402-415):
 * accumulator += w * expert */
S14_API int32_t s14_bind_moe_accumulate(s14_ctx *ctx, uint32_t n, float weight,
                                        const s14_buffer *expert, const s14_buffer *accumulator,
                                        s14_moe_accumulate_dispatch *out);
S14_API int32_t s14_cmd_moe_accumulate(s14_ctx *ctx, void *stream,
                                       const s14_moe_accumulate_dispatch *dispatch);

/* ---- fused layer: the 35-dispatch recording of
 *      examples/s14_vulkan_numeric.rs:1143-1218 as two or three kernels ---------- */

/* One token's route as the reference hands it over (RouteDecision,
 * s14_runner/src/runner.rs:121-126) with the pages already resolved to device
 * addresses of pinned pool slots (SlotBinding -> slot_offset,
 * vram_pool.rs:30-35, 397-399). */
typedef struct {
    uint32_t n_routed;                             /* 1..S14_EXPERTS_PER_TOKEN */
    uint16_t expert_ids[S14_EXPERTS_PER_TOKEN];    /* identity, used to group tokens */
    float weights[S14_EXPERTS_PER_TOKEN];          /* finite, >= 0 */
    const uint8_t *pages[S14_EXPERTS_PER_TOKEN];   /* MXFP4 pages, device addresses */
} s14_token_route;

typedef struct {
    uint32_t hidden;       /* K of w1/w3, N of w2: 1024, 2048 or 4096 */
    uint32_t inter;        /* N of w1/w3, K of w2: 1024, 2048 or 4096 */
    uint32_t n_tokens;     /* 1..S14_MAX_BLOCK_TOKENS */
    uint32_t shared_kind;  /* S14_PAGE_MXFP4 | S14_PAGE_FP8 */
    const uint8_t *shared_page; /* device address, NULL = no shared expert */
    const s14_token_route *routes; /* host array [n_tokens] */
    const float *x;        /* device [n_tokens, hidden] */
    float *y;              /* device [n_tokens, hidden] */
} s14_moe_layer_desc;

/* Enqueue one MoE layer for 1..8 tokens: every distinct expert's weights are read
 * once for all tokens routed to it; per token the routed outputs are mixed in
 * route order, then the shared output is added with weight 1
 * (examples/s14_vulkan_numeric.rs:929-947).  Uses the context's scratch. */
S14_API int32_t s14_cmd_moe_layer(s14_ctx *ctx, void *stream, const s14_moe_layer_desc *desc);

/* Which work the CTA `cta` of `n_ctas` (one per SM) does in a one-token layer of `n_jobs` experts on
 * the tensor-core path, in the order it does it: items_out[i] = down << 31 | job << 8 | index, where
 * an up item is (job, slice of 64 intermediate elements: w1 / w3 rows, SwiGLU) and a down item
 * (job, tile of 128 rows of w2).  n_early_jobs: the leading jobs whose pages are known before the
 * token's routes are (1 for a layer that picks its routes itself and has a shared expert, which is job
 * 0; else 0): their up items lead the lists and run while the routes are being picked.  Writes at
 * most `cap` items; *count receives the CTA's number of items.  Host arithmetic only, for tests and
 * for reading profiles; no counterpart in the reference. */
S14_API int32_t s14_layer_work_list(uint32_t cta, uint32_t n_ctas, uint32_t n_jobs, uint32_t n_early_jobs,
                                    uint32_t hidden, uint32_t inter, uint32_t *items_out, uint32_t cap,
                                    uint32_t *count);

/* Router (s14_first_real_token/executor.py:638-668): logits = x . Wr^T with Wr
 * BF16 [n_experts, hidden]; score = sigmoid | sqrt(softplus); select top_k of
 * score + bias (ties -> lowest index, descending order); weights = score[idx] /
 * sum * route_scale.  ids_out int32 [n_tokens, top_k], weights_out F32 likewise,
 * both device memory.  bias may be NULL. */
typedef struct {
    uint32_t n_experts; /* <= 256 */
    uint32_t hidden;    /* multiple of 256 */
    uint32_t n_tokens;  /* 1..8 */
    uint32_t top_k;     /* 1..8 */
    uint32_t score_fn;
    float route_scale;
    const float *x;
    const uint16_t *router_weight_bf16;
    const float *bias;
    int32_t *ids_out;
    float *weights_out;
} s14_router_desc;

S14_API int32_t s14_cmd_router(s14_ctx *ctx, void *stream, const s14_router_desc *desc);

/* Router + layer without a host round trip for one decode token: the router's
 * ids index `page_table` (device array [n_experts] of device page addresses, all
 * resident).  ids_out / weights_out (device, may be NULL) receive the route. */
typedef struct {
    s14_router_desc router; /* n_tokens must be 1; ids_out/weights_out optional */
    uint32_t inter;
    uint32_t shared_kind;
    const uint8_t *const *page_table;
    const uint8_t *shared_page;
    float *y;
} s14_routed_layer_desc;

S14_API int32_t s14_cmd_routed_moe_layer(s14_ctx *ctx, void *stream,
                                         const s14_routed_layer_desc *desc);

/* A decode stack: the MoE layers of a token step one after the other, the output of a layer being
 * the next layer's token - h <- h + moe_l(h) with `residual`, h <- moe_l(h) without - which is what
 * the runner's token step asks of its executor layer by layer
 * (scheduler/s14_runner/src/runner.rs:312-358: routed_and_shared_moe_then_hc_post per layer, with
 * the attention and hyper-connection steps taken as the identity) and what the reference's own
 * prefill / decode loop does with its layers (ssd_inference/src/forward.rs:544-549).  In pairwise
 * order with MXFP4 pages the whole stack is ONE launch of the tensor-core layer kernel, which walks
 * the layers itself (one CTA per SM stays resident, the next layer's shared expert is asked for
 * while the last rows of the layer before are mixed); otherwise the layers are launched one by one.
 * Every layer's result is the one s14_cmd_routed_moe_layer gives for the same token.
 *   create:  copies the layers' descriptors to the device once (the bind step).  All pointers are
 *            device addresses that stay valid while the stack is used; ids_out / weights_out
 *            ([top_k], the layer's route) and y_out ([hidden], the layer's MoE output before the
 *            residual) may be NULL.  Either every layer has a shared expert or none has.
 *   decode:  x [hidden] -> h_out [hidden], both device memory; x and h_out may be the same buffer. */
typedef struct {
    const uint16_t *router_weight_bf16;
    const float *bias;
    const uint8_t *const *page_table;
    const uint8_t *shared_page;
    int32_t *ids_out;
    float *weights_out;
    float *y_out;
} s14_stack_layer;

typedef struct {
    uint32_t n_layers;   /* 1..62 */
    uint32_t n_experts;  /* <= 256 */
    uint32_t hidden;     /* 1024, 2048 or 4096 */
    uint32_t inter;      /* 1024, 2048 or 4096 */
    uint32_t top_k;      /* 1..6 */
    uint32_t score_fn;
    float route_scale;
    uint32_t shared_kind; /* S14_PAGE_MXFP4 | S14_PAGE_FP8 */
    uint32_t residual;    /* 1: h <- h + moe(h) */
} s14_stack_config;

typedef struct s14_stack s14_stack;
S14_API int32_t s14_stack_create(s14_ctx *ctx, const s14_stack_config *config, const s14_stack_layer *layers,
                                 s14_stack **out);
S14_API int32_t s14_stack_destroy(s14_stack *stack);
S14_API int32_t s14_cmd_stack_decode(s14_ctx *ctx, void *stream, s14_stack *stack, const float *x, float *h_out);
/* The same for a caller that holds the token in host memory: copies host_x [hidden] to the device,
 * runs the stack, copies h [hidden] back and waits. */
S14_API int32_t s14_stack_decode_host(s14_ctx *ctx, s14_stack *stack, const float *host_x, float *host_h);

/* Expert-parallel decode (no counterpart in the reference, which has no multi-GPU code).  Every
 * rank of `ep_world` runs the replicated router on the same token and computes the experts it
 * owns - routed expert e belongs to rank e mod ep_world (its page_table entry must be resident
 * there; other entries are not read), the shared expert to `shared_owner`.  slots_out
 * [top_k (+1), hidden] receives the unmixed down vector of every owned expert in the row of its
 * route slot (shared expert last) and zeros elsewhere, so an all-reduce (sum) over the ranks
 * yields every slot exactly; router.ids_out / weights_out receive the route on every rank.
 * s14_cmd_moe_mix_slots then performs the reference's ordered mix on the gathered slots, which
 * makes the result bit-identical to the single-GPU layer for any number of ranks. */
S14_API int32_t s14_cmd_routed_moe_experts_ep(s14_ctx *ctx, void *stream,
                                              const s14_routed_layer_desc *desc, uint32_t ep_rank,
                                              uint32_t ep_world, uint32_t shared_owner,
                                              float *slots_out);
S14_API int32_t s14_cmd_moe_mix_slots(s14_ctx *ctx, void *stream, const float *slots,
                                      const float *weights_dev, uint32_t n_routed, int32_t has_shared,
                                      float *y, uint32_t hidden);

/* Expert-parallel decode with the exchange inside the layer kernel (no counterpart in the
 * reference).  Same partition as above.  Every rank owns an exchange buffer (two slot buffers
 * [top_k + 1, hidden] of 8-byte words, a step count) that the other ranks map: the layer kernel
 * stores the down vectors of the experts it owns into the route slot's row of EVERY rank's slot
 * buffer, each value together with the step's number in one 8-byte store (plain stores to peer
 * memory over NVLink), polls - bounded, a few seconds; a wait that runs out sets the device
 * status word 0x5503; a word that carries a later step's number, i.e. a peer that gave up on this
 * rank and ran ahead, sets 0x5504 and ends the waiting of that step, so that the rank catches up
 * and the ranks fall into step again -
 * the words it needs in its own buffer until they carry this step's number,
 * and performs the ordered mix from them.  No fence, flag or collective call on the way.  One
 * launch per rank and step, no collective call; y is bit-identical to the single-GPU layer on
 * every rank.  Every rank must issue the same sequence of steps.
 *   create:   allocates the buffer; handle_out (S14_EP_HANDLE_BYTES, may be NULL) receives the
 *             CUDA IPC handle to hand to the other ranks' processes.
 *   connect:  handles = world x S14_EP_HANDLE_BYTES in rank order (own entry ignored).
 *   connect_local: the ranks are contexts of this process on the same GPU (tests: ranks other
 *             than the last one run with wait_and_mix = 0 - they publish and return - so that no
 *             launch waits for a later launch of the same GPU).
 *   A rank may write a slot buffer for step s only when every peer has finished reading step
 *   s - 2 from it: behind the slot buffers every exchange buffer holds one 8-byte word per rank, the
 *   number of steps that rank has finished, which the rank's last CTA of a step stores into every
 *   peer's buffer; a step starts by waiting (bounded) until every peer's word in its own buffer
 *   says at least s - 1.  A wait that runs out sets status 0x5505 and the step goes on all the same:
 *   the peer that is then overwritten is far behind, finds later steps' numbers in its buffer
 *   (0x5504) and catches up without waiting, so that the ranks fall into step again.
 *   Teardown is a contract between the ranks, because every rank's kernel stores into every other
 *   rank's buffer: (1) every rank calls s14_ep_exchange_disconnect, which waits for all work of its
 *   device and closes its mappings of the other ranks' buffers; (2) the ranks pass a host barrier;
 *   (3) every rank calls s14_ep_exchange_destroy or s14_ctx_destroy, which frees its own buffer.
 *   Both destroy calls return S14_ERR_CONTRACT, and free nothing, while the exchange is connected.
 * Pairwise accumulation and MXFP4 pages only. */
#define S14_EP_HANDLE_BYTES 64
S14_API int32_t s14_ep_exchange_create(s14_ctx *ctx, uint32_t rank, uint32_t world, uint32_t hidden,
                                       uint8_t *handle_out);
S14_API int32_t s14_ep_exchange_connect(s14_ctx *ctx, const uint8_t *handles);
S14_API int32_t s14_ep_exchange_connect_local(s14_ctx *ctx, s14_ctx *const *ranks);
/* How long a rank waits for a word of another rank: `polls` of about a microsecond each (default
 * 2^22, a few seconds).  When it runs out the kernel sets the device status word 0x5503, writes no
 * y and returns; the context stays usable. */
S14_API int32_t s14_ep_exchange_set_wait_limit(s14_ctx *ctx, uint32_t polls);
S14_API int32_t s14_ep_exchange_disconnect(s14_ctx *ctx);
S14_API int32_t s14_ep_exchange_destroy(s14_ctx *ctx);
S14_API int32_t s14_cmd_routed_moe_layer_ep(s14_ctx *ctx, void *stream, const s14_routed_layer_desc *desc,
                                            uint32_t shared_owner, int32_t wait_and_mix);

/* The routed layer for a caller that holds the token in host memory: copies host_x
 * [hidden] to the device, runs router + layer on the resident pages (desc->router.x,
 * ids_out, weights_out and desc->y are ignored), copies y [hidden] and, when the
 * pointers are not NULL, the route (top_k ids and weights) back, and waits. */
S14_API int32_t s14_routed_moe_layer_host(s14_ctx *ctx, const s14_routed_layer_desc *desc,
                                          const float *host_x, float *host_y, int32_t *host_ids,
                                          float *host_weights);

/* A block of tokens through one MoE layer with the tokens GROUPED BY EXPERT: a verify block (K = 2..8,
 * s14_runner/src/cascade.rs:19) or a prefill of hundreds of tokens (the reference's prefill walks
 * its tokens one by one through the same layer loop, ssd_inference/src/forward.rs:544-549; the
 * semantics are that loop, examples/s14_vulkan_numeric.rs:929-947, applied to every token).  Every
 * distinct expert's page is streamed once from memory for all the tokens routed to it (in chunks of
 * two tokens for blocks of up to 12 tokens, of twelve for blocks with at least three (token, route)
 * pairs per expert, else of six; an expert's later chunks find the page in the
 * L2): per layer five launches - digit rows of the tokens, grouping of the (token, route) pairs by
 * expert, the w1 | w3 contraction with SwiGLU, the w2 contraction, the ordered mix (blocks of more than 12
 * tokens: six, the digit rows of the hidden values being a launch of their own) - the two
 * contractions on tcgen05 kind::mxf4.block_scale with N = 16 digit rows per token of a chunk; the
 * routed call runs two router launches first (scores of all tokens, one warp per token selects).  Every token's y is bit-identical to what
 * s14_cmd_moe_layer / s14_cmd_routed_moe_layer give for that token alone in pairwise order.
 * MXFP4 pages only (routed and shared); hidden and intermediate multiples of 512 up to 4096.
 *   create:  allocates the workspace for up to max_tokens (<= 1024) tokens:
 *            about max_tokens * (28 * hidden + 85 * intermediate + 8 * hidden) bytes.
 *   s14_cmd_moe_block:        routes from the host (desc->n_tokens up to max_tokens; expert_ids < 256
 *            identify the groups, a group's page is the page of one of its members).  The routes are
 *            staged through one pinned buffer of the block object: not for stream capture.
 *   s14_cmd_routed_moe_block: router on the device (desc->router.n_tokens up to max_tokens, top_k <= 6);
 *            ids_out / weights_out [n_tokens, top_k] may be NULL.
 *   One call at a time per block object (calls on one stream are ordered).  A wait that runs out
 *   inside a kernel sets the context's device status word to 0x5507.  A block object is used only
 *   while its context lives; destroying it afterwards is allowed. */
typedef struct s14_block s14_block;
S14_API int32_t s14_block_create(s14_ctx *ctx, uint32_t hidden, uint32_t inter, uint32_t max_tokens, s14_block **out);
S14_API int32_t s14_block_destroy(s14_block *blk);
/* residual != 0: the calls that follow write y = x + moe(x), the step of a stack of layers
 * (h <- h + moe_l(h), as s14_stack_create's `residual`); y may then be the same buffer as x. */
S14_API int32_t s14_block_set_residual(s14_block *blk, int32_t residual);
/* The arithmetic of the block's experts.  S14_BLOCK_SEMANTICS_F32 (the default): F32 values, every matvec's
 * exact sum rounded once, the route weight applied in the mix (examples/s14_vulkan_numeric.rs:929-947).
 * S14_BLOCK_SEMANTICS_OFFICIAL: the official expert arithmetic of
 * fast16/research/polaris_meridian_v1/s14_first_real_token/executor.py:712-743 (finish_layer) with
 * l42_real_reference/l42_reference.py:389-419 (_activation_quant, _linear_fp4): every linear quantises its
 * input per 128 elements to E4M3FN with a power-of-two scale and rounds its result to BF16; gate and up in
 * BF16, the limited SwiGLU in F32; a routed expert's hidden values are multiplied by the route weight and
 * rounded to BF16 BEFORE w2 (the shared expert's are rounded only); the experts' BF16 outputs are added in
 * F32 in route order, the shared expert last, and y is that sum rounded to BF16 (moe_branch; with the
 * residual switch y = x + moe_branch).  The dot products are exact sums rounded once to F32, where the
 * reference's are a float32 BLAS call in the library's order.  x holds F32 values (the reference's are
 * BF16-valued).  MXFP4 pages, the shared expert's included; s14_cmd_moe_block and s14_cmd_routed_moe_block
 * only: the expert-parallel calls refuse an official block, and an official block takes no exchange.
 * The quantisation and the digit rows of the hidden values are a launch of their own between the two
 * contractions (as for large blocks in the F32 arithmetic): six launches per layer. */
#define S14_BLOCK_SEMANTICS_F32 0u
#define S14_BLOCK_SEMANTICS_OFFICIAL 1u
S14_API int32_t s14_block_set_semantics(s14_block *blk, uint32_t semantics);
S14_API int32_t s14_cmd_moe_block(s14_ctx *ctx, void *stream, s14_block *blk, const s14_moe_layer_desc *desc);
S14_API int32_t s14_cmd_routed_moe_block(s14_ctx *ctx, void *stream, s14_block *blk, const s14_routed_layer_desc *desc);
/* Expert parallel (no counterpart in the reference; partition as s14_cmd_routed_moe_experts_ep: expert e
 * on rank e mod world, the shared expert on shared_owner; the tokens are on every rank).  Every rank
 * routes all tokens itself, groups the (token, route) pairs of the experts IT owns and writes their
 * expert outputs into pairs_out [n_tokens * 7, hidden] (pair = token * 7 + position in the route,
 * 6: the shared expert), zeros where another rank owns the expert; ids_out / weights_out are
 * required.  The caller adds the ranks' buffers up (one all-reduce: every row has one non-zero
 * contributor, so the sum is exact) and calls s14_cmd_moe_block_mix on every rank: y is then
 * bit-identical to the single-GPU block for any number of ranks.  x_residual: the layer's input to
 * add (y = x + moe(x)), or NULL. */
/* shared_owner of the two expert-parallel block calls: a rank, or S14_EP_SHARED_BY_TOKEN - the shared
 * page is resident on EVERY rank and rank r runs the shared expert for the tokens t with
 * t mod world == r (in a large block the shared expert is a fifth of the work; on one rank it bounds
 * the scaling). */
#define S14_EP_SHARED_BY_TOKEN 0xFFFFFFFFu
S14_API int32_t s14_cmd_routed_moe_block_experts_ep(s14_ctx *ctx, void *stream, s14_block *blk,
                                                    const s14_routed_layer_desc *desc, uint32_t ep_rank,
                                                    uint32_t ep_world, uint32_t shared_owner, float *pairs_out);
S14_API int32_t s14_cmd_moe_block_mix(s14_ctx *ctx, void *stream, s14_block *blk, const float *pairs, const int32_t *ids,
                                      const float *weights, uint32_t n_tokens, uint32_t top_k, int32_t has_shared,
                                      const float *x_residual, float *y);
/* The same partition with the exchange INSIDE the block kernels (no collective call): every rank owns
 * two pair buffers [max_tokens * 7, hidden] F32 (calls alternate between them) that the other ranks
 * map (CUDA IPC); the w2 kernel stores the rows of the experts it owns into EVERY rank's buffer (plain
 * stores to peer memory over NVLink) and its last CTA publishes the call's number to every rank (one
 * 8-byte word per rank and buffer); the mix waits - bounded, about a microsecond per poll, default 2^22
 * polls; a wait that runs out sets the device status word 0x5508 and writes no y - until every rank's
 * word carries this call's number.  A rank writes call s + 1 only after its own mix of call s, which
 * waited for every rank, so two buffers are enough.  Every rank issues the same sequence of calls; y
 * is bit-identical to the single-GPU block on every rank.
 *   create / connect / connect_local / disconnect: as s14_ep_exchange_* (connect_local: the ranks are
 *   block objects of this process on one GPU; tests run every rank but the last with wait_and_mix = 0).
 *   Teardown: every rank s14_block_ep_disconnect, a host barrier, then s14_block_destroy (which refuses
 *   while connected). */
S14_API int32_t s14_block_ep_create(s14_block *blk, uint32_t rank, uint32_t world, uint8_t *handle_out);
S14_API int32_t s14_block_ep_connect(s14_block *blk, const uint8_t *handles);
S14_API int32_t s14_block_ep_connect_local(s14_block *blk, s14_block *const *ranks);
S14_API int32_t s14_block_ep_set_wait_limit(s14_block *blk, uint32_t polls);
S14_API int32_t s14_block_ep_disconnect(s14_block *blk);
S14_API int32_t s14_cmd_routed_moe_block_ep(s14_ctx *ctx, void *stream, s14_block *blk, const s14_routed_layer_desc *desc,
                                            uint32_t shared_owner, int32_t wait_and_mix);
/* After the stream is synchronised: the last call's number of chunks, up items, down items, and 1 if
 * an expert id was outside the table (the call then wrote no result). */
S14_API int32_t s14_block_last_counts(s14_block *blk, uint32_t counts_out[4]);

/* ---- the steps on either side of the MoE inside one layer ------------------------------------
 * Hyper-connection reduce and expand, RMSNorm, the head's reduce and the hash route of the first
 * layers (local_s14_primitives/hc.py:19-148, final_head.py:43-110,
 * s14_first_real_token/executor.py:638-668, 712-743: hc_pre -> RMSNorm -> route -> experts -> hc_post).
 * A token's state is hc = 4 streams of `hidden` values, F32 or BF16 (the reference's state is BF16
 * [1, 1, 4, 4096]); results are rounded to the streams' type where the Python code casts back.  The
 * long sums (mean of squares, the 24 dot products with hc_fn) are accumulated in double and rounded
 * to F32 once, exp is evaluated in double; everything else is the Python expressions' F32
 * arithmetic in their order.  1..1024 tokens, hidden a multiple of 256 up to 8192.
 *   hc_pre:   x [T, 4, hidden] -> reduced [T, hidden] (stream type), post [T, 4], comb [T, 4, 4] (F32)
 *   hc_post:  merged[t][o] = post[t][o] * branch[t] + sum_h comb[t][h][o] * residual[t][h]  ([T, 4, hidden])
 *   rms_norm: out = weight * (x * rsqrt(mean(x^2) + eps)), x [T, hidden]
 *   hc_head_reduce: hc_fn [4, 4 * hidden], hc_scale [1], hc_base [4] -> reduced [T, hidden], pre [T, 4]
 *   router_hash: ids_out[t] = tid2eid_rows[t] (device int64 [T, top_k], the current token's row of the
 *            layer's tid2eid), weights_out = the router's scores of those experts / their sum * route_scale;
 *            desc->bias is not used. */
#define S14_STREAM_F32 0u
#define S14_STREAM_BF16 1u
typedef struct {
    uint32_t n_tokens;
    uint32_t hc;             /* 4 */
    uint32_t hidden;
    uint32_t dtype;          /* S14_STREAM_* of x and reduced */
    uint32_t sinkhorn_iters; /* the reference: 20 */
    float norm_eps, hc_eps;  /* the reference: 1e-6 both */
    const float *hc_fn;      /* [(2 + hc) * hc, hc * hidden] F32 */
    const float *hc_scale;   /* [3] */
    const float *hc_base;    /* [(2 + hc) * hc] */
} s14_hc_params;
S14_API int32_t s14_cmd_hc_pre(s14_ctx *ctx, void *stream, const s14_hc_params *params, const void *x, void *reduced,
                               float *post, float *comb);
S14_API int32_t s14_cmd_hc_post(s14_ctx *ctx, void *stream, uint32_t n_tokens, uint32_t hc, uint32_t hidden, uint32_t dtype,
                                const void *branch, const void *residual, const float *post, const float *comb, void *merged);
S14_API int32_t s14_cmd_rms_norm(s14_ctx *ctx, void *stream, uint32_t n_tokens, uint32_t hidden, uint32_t dtype, const void *x,
                                 const float *weight, float eps, void *out);
S14_API int32_t s14_cmd_hc_head_reduce(s14_ctx *ctx, void *stream, const s14_hc_params *params, const void *x, void *reduced,
                                       float *pre);
S14_API int32_t s14_cmd_router_hash(s14_ctx *ctx, void *stream, const s14_router_desc *desc, const int64_t *tid2eid_rows);

/* The executor's two device steps (NativeS14Executor, s14_runner/src/runner.rs:86-118) as single
 * calls on a token's BF16 state, composed of the calls above (no new arithmetic):
 *   routed_and_shared_moe_then_hc_post: ffn_input (BF16 [hidden], the FFN site's hc_pre + RMSNorm
 *     output) -> F32 -> the MoE layer of s14_cmd_moe_layer with the route's pages -> the branch rounded
 *     to BF16 -> hc_post with the site's post / comb over the post-attention state -> state_out.
 *     (The experts run this library's F32 semantics - exact sums, one rounding -, not the official
 *     BF16 / FP8-requantised intermediate roundings of executor.py:712-743.)
 *   hc_head_norm_full_logits (final_head.py:152-191): head reduce -> RMSNorm -> the BF16 head's
 *     logits for n_rows vocabulary rows (the full logits, or a shard's); the caller takes the argmax
 *     (s14_cmd_greedy_argmax), as the runner does. */
typedef struct {
    uint32_t hidden, inter;
    uint32_t shared_kind;
    const s14_token_route *route;      /* host: the token's route with its pages */
    const uint8_t *shared_page;
    const uint16_t *ffn_input_bf16;    /* device [hidden] */
    const uint16_t *residual_bf16;     /* device [4, hidden]: the post-attention state */
    const float *post, *comb;          /* device [4], [4, 4]: the FFN site's */
    uint16_t *state_out_bf16;          /* device [4, hidden] */
    uint16_t *moe_branch_out_bf16;     /* device [hidden], or NULL */
} s14_exec_moe_desc;
S14_API int32_t s14_exec_routed_and_shared_moe_then_hc_post(s14_ctx *ctx, void *stream, const s14_exec_moe_desc *desc);
S14_API int32_t s14_exec_hc_head_norm_full_logits(s14_ctx *ctx, void *stream, const s14_hc_params *head,
                                                  const float *norm_weight, const uint16_t *head_weight_bf16,
                                                  uint32_t n_rows, const uint16_t *state_bf16, float *logits_out);

/* LM head (local_s14_primitives/final_head.py:113-149): logits[v] = x . W[v,:]
 * for the rows [row_begin, row_begin + n_rows) of a BF16 [vocab, hidden] matrix
 * whose first stored row is row_begin (a vocabulary shard); logits_out points at
 * the shard's first logit.  n_tokens 1..8. */
S14_API int32_t s14_cmd_head_logits(s14_ctx *ctx, void *stream, const float *x, uint32_t n_tokens,
                                    const uint16_t *weight_bf16, uint32_t n_rows, uint32_t hidden,
                                    float *logits_out, uint32_t logits_stride);

/* greedy_full_vocab_argmax (s14_runner/src/runner.rs:485-508): lowest id wins
 * ties; a NaN anywhere yields -1.  result is a device int64. */
S14_API int32_t s14_cmd_greedy_argmax(s14_ctx *ctx, void *stream, const float *logits,
                                      uint32_t vocab, int64_t *result);

/* The layer for callers that must not allocate: code that runs where cudaMalloc is off
 * limits (inside a CUDA graph capture that some other component owns, in a latency-critical
 * serving loop whose memory plan is frozen after start-up, or under a harness that forbids
 * device allocation after initialisation) and therefore cannot create an s14_ctx, whose
 * constructor allocates its scratch.  This entry point has no counterpart in the reference.
 * It takes no context: the scratch between the up and down phases lives in file-scope device
 * arrays inside the library (about 230 KB per GPU, held until the process exits), so the limits
 * are one token per call (desc->n_tokens == 1, at most 6 routed experts plus the shared one)
 * and hidden, intermediate each one of 1024, 2048 or 4096 (the sizes the layer kernels are built
 * for); anything else is refused with S14_ERR_CONTRACT.  It calls
 * no cudaMalloc, cudaFree or allocating library routine.  `device` is the ordinal the pointers
 * in desc belong to; `stream` a stream of that device (NULL = the legacy default stream).  The
 * device is made current for the call and the caller's current device is put back before it
 * returns, on success and on failure.
 * The first call on a device resolves the addresses of the arrays and the kernel attributes (once
 * per device and process, also when several host threads make it together);
 * make that first call before any stream capture.  All calls on a device share the one scratch
 * and its arrival counters (cleared at the start of every call): calls that overlap on the
 * GPU - different streams without ordering, or several host threads - race on it. */
S14_API int32_t s14_moe_layer_noalloc(int32_t device, void *stream, uint32_t accumulation,
                                      const s14_moe_layer_desc *desc);

/* The same layer for a caller that holds x and y in host memory (pinned or
 * pageable): copies host_x [n_tokens, hidden] to context-owned device staging,
 * runs the layer on the resident pages named by desc (desc->x / desc->y are
 * ignored), copies the result to host_y and waits for it. */
S14_API int32_t s14_moe_layer_host(s14_ctx *ctx, const s14_moe_layer_desc *desc, const float *host_x,
                                   float *host_y);

/* ---- page pool: VramPool (ssd_inference/src/vram_pool.rs:16-422) ------------- */
typedef struct {
    uint32_t layer;
    uint8_t kind;
    uint32_t slot;
} s14_expert_key;

typedef struct {
    s14_expert_key key;
    uint32_t slot;
    uint64_t generation;
} s14_slot_binding; /* a SlotLease carries exactly one of these */

typedef struct {
    s14_expert_key key;
    uint32_t slot;
    uint64_t generation;
    int32_t has_evicted;
    s14_expert_key evicted;
} s14_loading_reservation;

/* VramPool::new (vram_pool.rs:76-114): one cudaMalloc of n_slots * slot_bytes.
 * ctx == NULL builds the bookkeeping-only pool the reference's unit tests use
 * (new_for_tests, vram_pool.rs:408-421): no device memory, slot addresses NULL. */
S14_API int32_t s14_pool_create(s14_ctx *ctx, uint32_t n_slots, uint64_t slot_bytes, s14_pool **out);
/* The same bookkeeping over slots in host memory (no device, no kernels): for tests of the loader
 * below on a machine without a GPU. */
S14_API int32_t s14_pool_create_host(uint32_t n_slots, uint64_t slot_bytes, s14_pool **out);
S14_API int32_t s14_pool_destroy(s14_pool *pool);
S14_API uint32_t s14_pool_capacity(const s14_pool *pool);
S14_API uint64_t s14_pool_slot_bytes(const s14_pool *pool);
S14_API uint32_t s14_pool_n_loaded(const s14_pool *pool);
S14_API uint64_t s14_pool_total_bytes(const s14_pool *pool);
S14_API uint64_t s14_pool_slot_offset(const s14_pool *pool, uint32_t slot);
S14_API void *s14_pool_slot_ptr(const s14_pool *pool, uint32_t slot);
/* lookup (vram_pool.rs:130-138): *found = 0/1 */
S14_API int32_t s14_pool_lookup(s14_pool *pool, s14_expert_key key, int32_t *found, uint32_t *slot);
/* lookup_and_pin (:141-166) */
S14_API int32_t s14_pool_lookup_and_pin(s14_pool *pool, s14_expert_key key, int32_t *found,
                                        s14_slot_binding *lease);
/* reserve_loading_generation (:178-243) */
S14_API int32_t s14_pool_reserve_loading_generation(s14_pool *pool, s14_expert_key key,
                                                    s14_loading_reservation *out);
/* mark_ready (:246-268) */
S14_API int32_t s14_pool_mark_ready(s14_pool *pool, uint32_t slot, s14_expert_key key);
/* validate_publish_batch (:271-316) */
S14_API int32_t s14_pool_validate_publish_batch(const s14_pool *pool,
                                                const s14_loading_reservation *reservations,
                                                uint32_t count);
/* publish_batch_and_pin (:320-326) */
S14_API int32_t s14_pool_publish_batch_and_pin(s14_pool *pool,
                                               const s14_loading_reservation *reservations,
                                               uint32_t count, s14_slot_binding *leases_out);
/* validate_binding (:353-370) */
S14_API int32_t s14_pool_validate_binding(const s14_pool *pool, s14_slot_binding binding);
/* release_after_compute_fence (:372-376) */
S14_API int32_t s14_pool_release_after_compute_fence(s14_pool *pool, s14_slot_binding lease);
/* cancel_loading (:379-385) / cancel_reservation (:387-408) */
S14_API int32_t s14_pool_cancel_loading(s14_pool *pool, uint32_t slot, s14_expert_key key);
S14_API int32_t s14_pool_cancel_reservation(s14_pool *pool, s14_loading_reservation reservation);

/* ExpertLoader::enqueue_from_buf / wait_all (ssd_inference/src/expert_loader.rs:
 * 362-442, 286-297): copy `bytes` of a page from pinned host memory into the
 * reserved slot with cudaMemcpyAsync on the context's copy stream.  The "transfer
 * fence" is a CUDA event: s14_pool_transfer_fence records it after the uploads
 * enqueued so far, s14_pool_wait_transfer_fence blocks the host on it, and
 * s14_pool_compute_wait_transfer makes the compute stream wait for it. */
S14_API int32_t s14_pool_upload_page_async(s14_pool *pool, const s14_loading_reservation *reservation,
                                           const void *host_bytes, uint64_t bytes);
S14_API int32_t s14_pool_transfer_fence(s14_pool *pool);
S14_API int32_t s14_pool_wait_transfer_fence(s14_pool *pool);
S14_API int32_t s14_pool_compute_wait_transfer(s14_pool *pool, void *compute_stream);
/* ExpertLoader (ssd_inference/src/expert_loader.rs:163-442): pages go to pool slots through a ring
 * of pipeline_depth pinned staging buffers with a fence each (one cudaMemcpyAsync per page on the
 * context's copy stream).  A ring entry is reused only after its transfer has completed and its
 * page has been published; a page is not visible through s14_pool_lookup before that.
 *   enqueue_from_buf (:362-442): a page that is Ready or in flight is not loaded again; otherwise
 *     the next ring entry is reclaimed (this is the only wait), a slot is reserved (may evict), the
 *     bytes are copied to the entry's staging buffer and the transfer is started; *slot_out is the
 *     pool slot.  A failure cancels the reservation.
 *   batch_enqueue_from_bufs (batch_enqueue, :299-358): earlier work is settled first, duplicates are
 *     loaded once, more distinct pages than the pool has slots are refused before anything is
 *     issued; waves of pipeline_depth pages, every wave but the last drained before the next one
 *     starts, so that no page overwrites staging memory an earlier transfer still reads.
 *   wait_all (:291-297): every transfer complete, every page Ready.
 * The reference's reader-based enqueue (file range reads into the staging buffer) is not mirrored:
 * the page source is the caller's. */
typedef struct s14_loader s14_loader;
S14_API int32_t s14_loader_create(s14_pool *pool, uint32_t pipeline_depth, s14_loader **out);
S14_API int32_t s14_loader_destroy(s14_loader *loader);
S14_API int32_t s14_loader_enqueue_from_buf(s14_loader *loader, s14_expert_key key, const void *data, uint64_t bytes,
                                            uint32_t *slot_out);
S14_API int32_t s14_loader_batch_enqueue_from_bufs(s14_loader *loader, const s14_expert_key *keys,
                                                   const void *const *datas, const uint64_t *sizes, uint32_t n,
                                                   uint32_t *slots_out);
S14_API int32_t s14_loader_wait_all(s14_loader *loader);
S14_API uint32_t s14_loader_in_flight(const s14_loader *loader);
S14_API uint64_t s14_loader_stat_loads(const s14_loader *loader);
S14_API uint64_t s14_loader_stat_bytes(const s14_loader *loader);

/* Pinned host staging memory (GpuBuffer::new_staging, buffer.rs:56-75). */
S14_API int32_t s14_host_alloc_pinned(uint64_t bytes, void **out);
S14_API int32_t s14_host_free_pinned(void *ptr);

/* ---- page transactions: S14VulkanMoePages (s14_vulkan.rs:661-819) ------------ */
typedef struct {
    uint8_t layer;
    uint8_t kind; /* 0 = hash router, 1 = score router (RouterKind, contract.rs:27-31) */
    uint16_t expert_ids[S14_EXPERTS_PER_TOKEN];
    float weights[S14_EXPERTS_PER_TOKEN];
    uint32_t n; /* number of ids/weights supplied; must be 6 */
} s14_route_decision;

#define S14_PROFILE_S14_TOP6 0u
#define S14_PROFILE_FULL_DEPTH43_NATIVE_TOP6 1u

/* RouteDecision::validate_for (s14_runner/src/runner.rs:128-180) */
S14_API int32_t s14_route_validate_for(const s14_route_decision *route, uint32_t profile);

typedef struct s14_route_load_batch s14_route_load_batch;       /* RouteLoadBatch */
typedef struct s14_moe_compute_lease s14_moe_compute_lease;     /* S14MoeComputeLeaseBatch */

/* S14VulkanMoePages::new (s14_vulkan.rs:709-734) */
S14_API int32_t s14_moe_pages_create(s14_pool *routed_pool, s14_pool *shared_pool, uint32_t profile,
                                     s14_moe_pages **out);
/* The same with explicit minimum slot sizes (small test shapes; an MXFP4 shared
 * expert needs only S14_EXPERT_PAGE_BYTES). */
S14_API int32_t s14_moe_pages_create_ex(s14_pool *routed_pool, s14_pool *shared_pool, uint32_t profile,
                                        uint64_t min_routed_bytes, uint64_t min_shared_bytes,
                                        s14_moe_pages **out);
S14_API int32_t s14_moe_pages_destroy(s14_moe_pages *pages);
/* begin_after_official_route (:736-775).  On success *batch owns pins/reservations. */
S14_API int32_t s14_moe_pages_begin_after_official_route(s14_moe_pages *pages,
                                                         const s14_route_decision *route,
                                                         s14_route_load_batch **batch);
/* Pages of the batch that still need an upload (state Loading).  slots_out /
 * is_shared_out have room for 7 entries; returns the count in *count. */
S14_API int32_t s14_route_load_batch_missing(const s14_route_load_batch *batch,
                                             s14_loading_reservation *reservations_out,
                                             int32_t *is_shared_out, uint32_t *count);
/* publish_after_transfer_fence (:777-800); consumes the batch either way. */
S14_API int32_t s14_moe_pages_publish_after_transfer_fence(s14_moe_pages *pages,
                                                           s14_route_load_batch *batch,
                                                           s14_moe_compute_lease **lease);
/* routed_bindings / shared_binding / expert_ids / route_weights (:683-701) */
S14_API int32_t s14_moe_compute_lease_bindings(const s14_moe_compute_lease *lease,
                                               s14_slot_binding routed_out[S14_EXPERTS_PER_TOKEN],
                                               s14_slot_binding *shared_out,
                                               uint16_t ids_out[S14_EXPERTS_PER_TOKEN],
                                               float weights_out[S14_EXPERTS_PER_TOKEN]);
/* release_after_compute_fence (:802-812); consumes the lease on success. */
S14_API int32_t s14_moe_pages_release_after_compute_fence(s14_moe_pages *pages,
                                                          s14_moe_compute_lease *lease);
/* cancel (:814-818); consumes the batch. */
S14_API int32_t s14_moe_pages_cancel(s14_moe_pages *pages, s14_route_load_batch *batch);

#ifdef __cplusplus
}
#endif
#endif /* POLARIS_S14_CUDA_H */
