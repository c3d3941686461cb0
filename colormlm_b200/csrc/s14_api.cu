// C ABI of the S14 MoE path (include/polaris_s14_cuda.h): contexts, operator
// bind/cmd pairs, the fused layer, router, LM head, the page pool and the route
// page transaction.  No CPU fallback: every cmd_ call launches a CUDA kernel.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "s14_host.hpp"
#include "s14_internal.h"

using namespace s14;

// ---- error plumbing ---------------------------------------------------------

static thread_local std::string g_last_error;

static int32_t fail(int32_t code, const std::string &msg) {
    g_last_error = msg;
    return code;
}

static int32_t cuda_fail(cudaError_t e, const char *what) {
    return fail(S14_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

// a CUDA error inside host-side classes that report by exception
struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
static void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw CudaError(std::string(what) + ": " + cudaGetErrorString(e));
}

#define S14_TRY try {
#define S14_CATCH                                                      \
    }                                                                  \
    catch (const ContractError &e) { return fail(S14_ERR_CONTRACT, e.what()); } \
    catch (const PoolError &e) { return fail(S14_ERR_POOL, e.what()); }         \
    catch (const CudaError &e) { return fail(S14_ERR_CUDA, e.what()); }         \
    catch (const CodeError &e) { return fail(S14_ERR_CODE, e.what()); }         \
    catch (const std::bad_alloc &) { return fail(S14_ERR_CONTRACT, "out of host memory"); } \
    catch (const std::exception &e) { return fail(S14_ERR_CONTRACT, e.what()); }

#define CUDA_OK(call)                                      \
    do {                                                   \
        cudaError_t _e = (call);                           \
        if (_e != cudaSuccess) return cuda_fail(_e, #call); \
    } while (0)

extern "C" const char *s14_last_error(void) { return g_last_error.c_str(); }

// ---- context ----------------------------------------------------------------

static constexpr uint32_t kMaxDim = 4096;  // largest hidden / intermediate of the fused layer
static constexpr uint32_t kCounters = 2048; // [0]: router; [1 + token * 160 + slice]: down-phase row slices
static constexpr uint32_t kGlueTokens = 1024;   // most tokens of a hyper-connection / RMSNorm / hash-route call
static constexpr uint32_t kCtxCounters = 8192;  // a context's array also serves the tcgen05 phases (4609 used)

struct s14_ctx {
    int device = 0;
    int sm_count = 0;
    uint32_t mode = S14_ACCUM_PAIRWISE;
    cudaStream_t compute = nullptr, copy = nullptr;
    float *h = nullptr;       // [kMaxJobs, kMaxDim] activations between up and down
    float *d = nullptr;       // [kMaxJobs, kMaxDim] per-job down outputs before the mix
    float *scores = nullptr;  // [kMaxTokens, 256]
    float *select = nullptr;  // [kMaxTokens, 256]
    JobTable *dev_table = nullptr;
    float *x_stage = nullptr, *y_stage = nullptr;  // [kMaxTokens, kMaxDim]
    uint32_t *status = nullptr;
    uint64_t launches = 0;
    uint32_t last_path = 0;   // S14_LAYER_PATH_* of the last layer or stack call
    bool timing = false;  // per-kernel timing of routed layer calls (blocks after each call)
    KernelMarks marks{};
    double kernel_ms[4] = {0, 0, 0, 0};  // router, up, down, mix
    uint64_t timed_calls = 0;
    unsigned int *counters = nullptr;  // [kCtxCounters] arrival counters of the fused kernels, all zero at rest
    int32_t *ids_stage = nullptr;  // [8] route ids / weights staging of the host-buffer call
    float *weights_stage = nullptr;
    // Results of the routed host-buffer call: pinned host memory the kernels write through its
    // device address (16 KB + 64 B per step, posted writes), read by the CPU after the stream
    // synchronisation -- no device-to-host copy is enqueued.
    float *y_host = nullptr, *y_host_dev = nullptr;          // [kMaxDim]
    int32_t *ids_host = nullptr, *ids_host_dev = nullptr;    // [8]
    float *w_host = nullptr, *w_host_dev = nullptr;          // [8]
    // Expert-parallel exchange over peer memory: this rank's exchange buffer and the ranks' buffers
    // as mapped here (own buffer included); peers of other processes are opened CUDA IPC handles.
    struct {
        uint8_t *buf = nullptr;
        uint32_t rank = 0, world = 0, hidden = 0;
        uint8_t *peer[kMaxEpWorld] = {};
        bool opened[kMaxEpWorld] = {};
        bool connected = false;
        uint32_t wait_limit = 1u << 22;  // polls of about a microsecond: a few seconds
    } ep;
    float *glue = nullptr;    // [kGlueTokens, 25] dot products and mean squares of the hyper-connection calls
    uint16_t *glue16 = nullptr;  // [4, 8192] BF16 vectors between the steps of the executor calls
    UmmaScratch umma{nullptr, nullptr, nullptr};  // scratch of the tcgen05 layer kernel
    bool use_umma = true;                // S14_TENSOR_PATH=off in the environment turns it off
    const UmmaScratch *umma_scratch() const { return use_umma ? &umma : nullptr; }
};

static cudaStream_t stream_of(s14_ctx *ctx, void *stream) {
    return stream ? (cudaStream_t)stream : ctx->compute;
}

extern "C" int32_t s14_ctx_create(int32_t device, s14_ctx **out) {
    if (!out) return fail(S14_ERR_CONTRACT, "s14_ctx_create: out is NULL");
    *out = nullptr;
    int count = 0;
    CUDA_OK(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count)
        return fail(S14_ERR_CONTRACT, "s14_ctx_create: no CUDA device " + std::to_string(device));
    CUDA_OK(cudaSetDevice(device));
    cudaDeviceProp prop;
    CUDA_OK(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(S14_ERR_CONTRACT, "s14_ctx_create: the kernels are built for sm_100a only; device is sm_" +
                                          std::to_string(prop.major * 10 + prop.minor));
    std::unique_ptr<s14_ctx> ctx(new s14_ctx());
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    CUDA_OK(cudaStreamCreateWithFlags(&ctx->compute, cudaStreamNonBlocking));
    CUDA_OK(cudaStreamCreateWithFlags(&ctx->copy, cudaStreamNonBlocking));
    CUDA_OK(cudaMalloc(&ctx->h, sizeof(float) * kMaxJobs * kMaxDim));
    CUDA_OK(cudaMalloc(&ctx->d, sizeof(float) * kMaxJobs * kMaxDim));
    CUDA_OK(cudaMalloc(&ctx->scores, sizeof(float) * kMaxTokens * S14_N_ROUTED_EXPERTS));
    CUDA_OK(cudaMalloc(&ctx->select, sizeof(float) * kMaxTokens * S14_N_ROUTED_EXPERTS));
    CUDA_OK(cudaMalloc(&ctx->dev_table, sizeof(JobTable)));
    CUDA_OK(cudaMalloc(&ctx->glue, sizeof(float) * kGlueTokens * 25));
    CUDA_OK(cudaMalloc(&ctx->glue16, sizeof(uint16_t) * 4 * 8192));
    CUDA_OK(cudaMalloc(&ctx->x_stage, sizeof(float) * kMaxTokens * kMaxDim));
    CUDA_OK(cudaMalloc(&ctx->y_stage, sizeof(float) * kMaxTokens * kMaxDim));
    CUDA_OK(cudaMalloc(&ctx->status, sizeof(uint32_t)));
    CUDA_OK(cudaMemset(ctx->status, 0, sizeof(uint32_t)));
    CUDA_OK(cudaMalloc(&ctx->counters, sizeof(unsigned int) * kCtxCounters));
    CUDA_OK(cudaMemset(ctx->counters, 0, sizeof(unsigned int) * kCtxCounters));
    CUDA_OK(cudaMalloc(&ctx->ids_stage, sizeof(int32_t) * 8));
    CUDA_OK(cudaMalloc(&ctx->weights_stage, sizeof(float) * 8));
    CUDA_OK(cudaHostAlloc(&ctx->y_host, sizeof(float) * kMaxDim, cudaHostAllocMapped));
    CUDA_OK(cudaHostAlloc(&ctx->ids_host, sizeof(int32_t) * 8, cudaHostAllocMapped));
    CUDA_OK(cudaHostAlloc(&ctx->w_host, sizeof(float) * 8, cudaHostAllocMapped));
    CUDA_OK(cudaHostGetDevicePointer(&ctx->y_host_dev, ctx->y_host, 0));
    CUDA_OK(cudaHostGetDevicePointer(&ctx->ids_host_dev, ctx->ids_host, 0));
    CUDA_OK(cudaHostGetDevicePointer(&ctx->w_host_dev, ctx->w_host, 0));
    CUDA_OK(cudaMalloc(&ctx->umma.tiles, umma_scratch_bytes()));
    CUDA_OK(cudaMemset(ctx->umma.tiles, 0, umma_scratch_bytes()));  // no word carries a stamp yet
    ctx->umma.status = ctx->status;
    if (const char *path = getenv("S14_TENSOR_PATH")) ctx->use_umma = strcmp(path, "off") != 0;
    for (auto &e : ctx->marks.ev) CUDA_OK(cudaEventCreate(&e));
    *out = ctx.release();
    return S14_OK;
}

extern "C" int32_t s14_ctx_destroy(s14_ctx *ctx) {
    if (!ctx) return S14_OK;
    // a context whose expert-parallel exchange is still connected is not destroyed: its peers may
    // still write into its buffer (see s14_ep_exchange_disconnect for the order of a teardown)
    if (ctx->ep.connected)
        return fail(S14_ERR_CONTRACT,
                    "s14_ctx_destroy: the expert-parallel exchange is still connected; every rank calls "
                    "s14_ep_exchange_disconnect, the ranks pass a host barrier, then the contexts are destroyed");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->compute);
    cudaStreamSynchronize(ctx->copy);
    cudaFree(ctx->h);
    cudaFree(ctx->d);
    cudaFree(ctx->scores);
    cudaFree(ctx->select);
    cudaFree(ctx->glue);
    cudaFree(ctx->glue16);
    cudaFree(ctx->dev_table);
    cudaFree(ctx->x_stage);
    cudaFree(ctx->y_stage);
    cudaFree(ctx->status);
    cudaFree(ctx->counters);
    cudaFree(ctx->ids_stage);
    cudaFree(ctx->weights_stage);
    cudaFree(ctx->umma.tiles);
    cudaFree(ctx->umma.trace);
    s14_ep_exchange_destroy(ctx);
    cudaFreeHost(ctx->y_host);
    cudaFreeHost(ctx->ids_host);
    cudaFreeHost(ctx->w_host);
    for (auto &e : ctx->marks.ev)
        if (e) cudaEventDestroy(e);
    cudaStreamDestroy(ctx->compute);
    cudaStreamDestroy(ctx->copy);
    delete ctx;
    return S14_OK;
}

extern "C" void *s14_ctx_compute_stream(s14_ctx *ctx) { return ctx ? ctx->compute : nullptr; }
extern "C" void *s14_ctx_copy_stream(s14_ctx *ctx) { return ctx ? ctx->copy : nullptr; }

extern "C" int32_t s14_ctx_synchronize(s14_ctx *ctx) {
    if (!ctx) return fail(S14_ERR_CONTRACT, "ctx is NULL");
    CUDA_OK(cudaStreamSynchronize(ctx->compute));
    CUDA_OK(cudaStreamSynchronize(ctx->copy));
    return S14_OK;
}

extern "C" int32_t s14_ctx_set_accumulation(s14_ctx *ctx, uint32_t mode) {
    if (!ctx) return fail(S14_ERR_CONTRACT, "ctx is NULL");
    if (mode != S14_ACCUM_PAIRWISE && mode != S14_ACCUM_REFERENCE)
        return fail(S14_ERR_CONTRACT, "unknown accumulation mode " + std::to_string(mode));
    ctx->mode = mode;
    return S14_OK;
}

extern "C" uint32_t s14_ctx_accumulation(const s14_ctx *ctx) { return ctx ? ctx->mode : 0; }
extern "C" int32_t s14_ctx_sm_count(const s14_ctx *ctx) { return ctx ? ctx->sm_count : 0; }
extern "C" uint64_t s14_ctx_launch_count(const s14_ctx *ctx) { return ctx ? ctx->launches : 0; }
extern "C" uint32_t s14_ctx_last_layer_path(const s14_ctx *ctx) { return ctx ? ctx->last_path : 0; }

extern "C" int32_t s14_ctx_device_status(s14_ctx *ctx, uint32_t *status) {
    if (!ctx || !status) return fail(S14_ERR_CONTRACT, "ctx or status is NULL");
    CUDA_OK(cudaStreamSynchronize(ctx->compute));
    CUDA_OK(cudaMemcpy(status, ctx->status, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (*status != 0) CUDA_OK(cudaMemset(ctx->status, 0, sizeof(uint32_t)));
    return S14_OK;
}

extern "C" int32_t s14_ctx_set_layer_trace(s14_ctx *ctx, int32_t enable) {
    if (!ctx) return fail(S14_ERR_CONTRACT, "ctx is NULL");
    CUDA_OK(cudaStreamSynchronize(ctx->compute));
    if (enable && !ctx->umma.trace) {
        CUDA_OK(cudaMalloc(&ctx->umma.trace, umma_trace_bytes(ctx->sm_count)));
        CUDA_OK(cudaMemset(ctx->umma.trace, 0, umma_trace_bytes(ctx->sm_count)));
    } else if (!enable && ctx->umma.trace) {
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaFree(ctx->umma.trace));
        ctx->umma.trace = nullptr;
    }
    return S14_OK;
}

extern "C" int32_t s14_ctx_read_layer_trace(s14_ctx *ctx, uint64_t *out, uint32_t cap_words, uint32_t *n_ctas,
                                            uint32_t *words_per_cta) {
    if (!ctx || !out || !n_ctas || !words_per_cta) return fail(S14_ERR_CONTRACT, "s14_ctx_read_layer_trace: NULL argument");
    if (!ctx->umma.trace) return fail(S14_ERR_CONTRACT, "s14_ctx_read_layer_trace: the trace is not enabled");
    *n_ctas = (uint32_t)ctx->sm_count;
    *words_per_cta = umma_trace_words();
    const size_t words = (size_t)ctx->sm_count * umma_trace_words();
    if (cap_words < words) return fail(S14_ERR_CONTRACT, "s14_ctx_read_layer_trace: buffer too small");
    CUDA_OK(cudaDeviceSynchronize());
    CUDA_OK(cudaMemcpy(out, ctx->umma.trace, words * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return S14_OK;
}

extern "C" int32_t s14_ctx_set_kernel_timing(s14_ctx *ctx, int32_t enable) {
    if (!ctx) return fail(S14_ERR_CONTRACT, "ctx is NULL");
    ctx->timing = enable != 0;
    for (double &v : ctx->kernel_ms) v = 0.0;
    ctx->timed_calls = 0;
    return S14_OK;
}

extern "C" int32_t s14_ctx_kernel_times(s14_ctx *ctx, double ms_out[4], uint64_t *calls) {
    if (!ctx || !ms_out || !calls) return fail(S14_ERR_CONTRACT, "s14_ctx_kernel_times: NULL argument");
    for (int i = 0; i < 4; ++i) ms_out[i] = ctx->kernel_ms[i];
    *calls = ctx->timed_calls;
    return S14_OK;
}

// ---- byte contracts -----------------------------------------------------------

static S14MatvecShape shape_of(s14_matvec_shape s) {
    S14MatvecShape out;
    out.n = s.n;
    out.k = s.k;
    return out;
}

extern "C" int32_t s14_shape_new(uint32_t n, uint32_t k, s14_matvec_shape *out) {
    S14_TRY
    const S14MatvecShape s = S14MatvecShape::make(n, k);
    if (out) {
        out->n = s.n;
        out->k = s.k;
    }
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_shape_validate_mxfp4(s14_matvec_shape shape) {
    S14_TRY
    shape_of(shape).validate_mxfp4();
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_shape_validate_fp8(s14_matvec_shape shape) {
    S14_TRY
    shape_of(shape).validate_fp8();
    return S14_OK;
    S14_CATCH
}

#define SHAPE_BYTES_FN(name, method)                                              \
    extern "C" int32_t name(s14_matvec_shape shape, uint64_t *out) {              \
        S14_TRY                                                                   \
        if (!out) throw ContractError(#name ": out is NULL");                     \
        *out = shape_of(shape).method();                                          \
        return S14_OK;                                                            \
        S14_CATCH                                                                 \
    }
SHAPE_BYTES_FN(s14_shape_fp32_input_bytes, fp32_input_bytes)
SHAPE_BYTES_FN(s14_shape_fp32_output_bytes, fp32_output_bytes)
SHAPE_BYTES_FN(s14_shape_mxfp4_weight_bytes, mxfp4_weight_bytes)
SHAPE_BYTES_FN(s14_shape_mxfp4_scale_bytes, mxfp4_scale_bytes)
SHAPE_BYTES_FN(s14_shape_fp8_weight_bytes, fp8_weight_bytes)
SHAPE_BYTES_FN(s14_shape_fp8_scale_bytes, fp8_scale_bytes)

extern "C" int32_t s14_mxfp4_expert_page_from_tensors(uint32_t hidden, uint32_t inter, const uint8_t *tensor_page,
                                                      uint8_t *page) {
    S14_TRY
    mxfp4_expert_page_from_tensors(hidden, inter, tensor_page, page);
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_mxfp4_expert_page_to_tensors(uint32_t hidden, uint32_t inter, const uint8_t *page,
                                                    uint8_t *tensor_page) {
    S14_TRY
    mxfp4_expert_page_to_tensors(hidden, inter, page, tensor_page);
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_validate_ue8m0_codes(const uint8_t *codes, uint64_t len, uint64_t *bad_index) {
    try {
        validate_ue8m0_codes(codes, len);
    } catch (const CodeError &e) {
        if (bad_index) *bad_index = e.index;
        return fail(S14_ERR_CODE, e.what());
    }
    return S14_OK;
}

extern "C" int32_t s14_validate_e4m3fn_codes(const uint8_t *codes, uint64_t len, uint64_t *bad_index) {
    try {
        validate_e4m3fn_codes(codes, len);
    } catch (const CodeError &e) {
        if (bad_index) *bad_index = e.index;
        return fail(S14_ERR_CODE, e.what());
    }
    return S14_OK;
}

// ---- primitive operators --------------------------------------------------------

static void require_capacity(const s14_buffer *b, uint64_t required, const char *label) {
    if (!b || !b->ptr) throw ContractError(std::string(label) + " buffer is NULL");
    if (b->size < required)
        throw ContractError(std::string(label) + " buffer is " + std::to_string(b->size) +
                            " B, requires at least " + std::to_string(required) + " B");
}

static void require_aligned(const void *p, uint64_t a, const char *label) {
    if (reinterpret_cast<uintptr_t>(p) % a != 0)
        throw ContractError(std::string(label) + " must be aligned to " + std::to_string(a) + " bytes");
}

extern "C" int32_t s14_bind_mxfp4(s14_ctx *ctx, s14_matvec_shape shape, const s14_buffer *x,
                                  const s14_buffer *packed_weight, const s14_buffer *weight_scale,
                                  const s14_buffer *y, s14_mxfp4_dispatch *out) {
    S14_TRY
    if (!ctx || !out) throw ContractError("s14_bind_mxfp4: ctx or out is NULL");
    const S14MatvecShape s = shape_of(shape).validate_mxfp4();
    require_capacity(x, s.fp32_input_bytes(), "S14 MXFP4 input");
    require_capacity(packed_weight, storage_bytes(s.mxfp4_weight_bytes()), "S14 MXFP4 weight");
    require_capacity(weight_scale, storage_bytes(s.mxfp4_scale_bytes()), "S14 MXFP4 scale");
    require_capacity(y, s.fp32_output_bytes(), "S14 MXFP4 output");
    require_aligned(x->ptr, 16, "S14 MXFP4 input");
    require_aligned(packed_weight->ptr, 16, "S14 MXFP4 weight");
    require_aligned(weight_scale->ptr, 4, "S14 MXFP4 scale");
    out->shape = shape;
    out->x = (const float *)x->ptr;
    out->packed_weight = (const uint8_t *)packed_weight->ptr;
    out->weight_scale = (const uint8_t *)weight_scale->ptr;
    out->y = (float *)y->ptr;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_mxfp4_matvec(s14_ctx *ctx, void *stream, const s14_mxfp4_dispatch *dsp) {
    if (!ctx || !dsp) return fail(S14_ERR_CONTRACT, "s14_cmd_mxfp4_matvec: NULL argument");
    CUDA_OK(launch_mxfp4_matvec(stream_of(ctx, stream), ctx->mode, ctx->sm_count, dsp->x,
                                dsp->packed_weight, dsp->weight_scale, dsp->y, dsp->shape.n,
                                dsp->shape.k));
    ctx->launches += 1;
    return S14_OK;
}

extern "C" int32_t s14_bind_fp8_ex(s14_ctx *ctx, s14_matvec_shape shape, uint32_t scale_format,
                                   uint32_t n_tokens, const s14_buffer *x, const s14_buffer *weight,
                                   const s14_buffer *weight_scale, const s14_buffer *y,
                                   s14_fp8_dispatch *out) {
    S14_TRY
    if (!ctx || !out) throw ContractError("s14_bind_fp8: ctx or out is NULL");
    const S14MatvecShape s = shape_of(shape).validate_fp8();
    if (scale_format != S14_SCALE_UE8M0 && scale_format != S14_SCALE_F32)
        throw ContractError("S14 FP8 scale format must be UE8M0 or F32");
    if (n_tokens == 0 || n_tokens > kMaxTokens)
        throw ContractError("S14 FP8 matvec takes 1..8 tokens per weight pass");
    const uint64_t scale_elem = scale_format == S14_SCALE_F32 ? 4 : 1;
    require_capacity(x, s.fp32_input_bytes() * n_tokens, "S14 FP8 input");
    require_capacity(weight, storage_bytes(s.fp8_weight_bytes()), "S14 FP8 weight");
    require_capacity(weight_scale, storage_bytes(s.fp8_scale_bytes() * scale_elem), "S14 FP8 scale");
    require_capacity(y, s.fp32_output_bytes() * n_tokens, "S14 FP8 output");
    if (scale_format == S14_SCALE_F32) require_aligned(weight_scale->ptr, 4, "S14 FP8 scale");
    require_aligned(x->ptr, 4, "S14 FP8 input");
    out->shape = shape;
    out->scale_format = scale_format;
    out->n_tokens = n_tokens;
    out->x = (const float *)x->ptr;
    out->weight = (const uint8_t *)weight->ptr;
    out->weight_scale = weight_scale->ptr;
    out->y = (float *)y->ptr;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_bind_fp8(s14_ctx *ctx, s14_matvec_shape shape, const s14_buffer *x,
                                const s14_buffer *weight, const s14_buffer *weight_scale,
                                const s14_buffer *y, s14_fp8_dispatch *out) {
    return s14_bind_fp8_ex(ctx, shape, S14_SCALE_UE8M0, 1, x, weight, weight_scale, y, out);
}

extern "C" int32_t s14_cmd_fp8_matvec(s14_ctx *ctx, void *stream, const s14_fp8_dispatch *dsp) {
    if (!ctx || !dsp) return fail(S14_ERR_CONTRACT, "s14_cmd_fp8_matvec: NULL argument");
    CUDA_OK(launch_fp8_matvec(stream_of(ctx, stream), ctx->mode, ctx->sm_count, dsp->scale_format,
                              dsp->n_tokens, dsp->x, dsp->weight, dsp->weight_scale, dsp->y,
                              dsp->shape.n, dsp->shape.k));
    ctx->launches += 1;
    return S14_OK;
}

extern "C" int32_t s14_bind_swiglu_limit(s14_ctx *ctx, uint32_t n, const s14_buffer *gate,
                                         const s14_buffer *up, const s14_buffer *y,
                                         s14_swiglu_limit_dispatch *out) {
    S14_TRY
    if (!ctx || !out) throw ContractError("s14_bind_swiglu_limit: ctx or out is NULL");
    if (n == 0) throw ContractError("S14 SwiGLU requires non-zero length");
    const uint64_t bytes = (uint64_t)n * 4;
    require_capacity(gate, bytes, "S14 SwiGLU gate");
    require_capacity(up, bytes, "S14 SwiGLU up");
    require_capacity(y, bytes, "S14 SwiGLU output");
    out->n = n;
    out->gate = (const float *)gate->ptr;
    out->up = (const float *)up->ptr;
    out->y = (float *)y->ptr;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_swiglu_limit(s14_ctx *ctx, void *stream,
                                        const s14_swiglu_limit_dispatch *dsp) {
    if (!ctx || !dsp) return fail(S14_ERR_CONTRACT, "s14_cmd_swiglu_limit: NULL argument");
    CUDA_OK(launch_swiglu_limit(stream_of(ctx, stream), dsp->gate, dsp->up, dsp->y, dsp->n));
    ctx->launches += 1;
    return S14_OK;
}

extern "C" int32_t s14_bind_route_mix(s14_ctx *ctx, uint32_t n, float route_weight,
                                      const s14_buffer *expert, const s14_buffer *routed,
                                      s14_route_mix_dispatch *out) {
    S14_TRY
    if (!ctx || !out) throw ContractError("s14_bind_route_mix: ctx or out is NULL");
    if (n == 0 || !std::isfinite(route_weight) || route_weight < 0.0f)
        throw ContractError("S14 route mix requires non-zero length and finite non-negative weight");
    const uint64_t bytes = (uint64_t)n * 4;
    require_capacity(expert, bytes, "S14 route mix expert");
    require_capacity(routed, bytes, "S14 route mix output");
    out->n = n;
    out->route_weight = route_weight;
    out->expert = (const float *)expert->ptr;
    out->routed = (float *)routed->ptr;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_route_mix(s14_ctx *ctx, void *stream, const s14_route_mix_dispatch *dsp) {
    if (!ctx || !dsp) return fail(S14_ERR_CONTRACT, "s14_cmd_route_mix: NULL argument");
    CUDA_OK(launch_route_mix(stream_of(ctx, stream), dsp->expert, dsp->routed, dsp->n,
                             dsp->route_weight));
    ctx->launches += 1;
    return S14_OK;
}

extern "C" int32_t s14_bind_moe_accumulate(s14_ctx *ctx, uint32_t n, float weight,
                                           const s14_buffer *expert, const s14_buffer *accumulator,
                                           s14_moe_accumulate_dispatch *out) {
    S14_TRY
    if (!ctx || !out) throw ContractError("s14_bind_moe_accumulate: ctx or out is NULL");
    if (n == 0 || !std::isfinite(weight) || weight < 0.0f)
        throw ContractError("S14 MoE accumulate requires non-zero length and finite non-negative weight");
    const uint64_t bytes = (uint64_t)n * 4;
    require_capacity(expert, bytes, "S14 MoE accumulate expert");
    require_capacity(accumulator, bytes, "S14 MoE accumulator");
    out->n = n;
    out->weight = weight;
    out->expert = (const float *)expert->ptr;
    out->accumulator = (float *)accumulator->ptr;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_moe_accumulate(s14_ctx *ctx, void *stream,
                                          const s14_moe_accumulate_dispatch *dsp) {
    if (!ctx || !dsp) return fail(S14_ERR_CONTRACT, "s14_cmd_moe_accumulate: NULL argument");
    CUDA_OK(launch_moe_accumulate(stream_of(ctx, stream), dsp->expert, dsp->accumulator, dsp->n,
                                  dsp->weight));
    ctx->launches += 1;
    return S14_OK;
}

// ---- fused layer ------------------------------------------------------------------

static bool fused_dim_ok(uint32_t v) { return v == 1024 || v == 2048 || v == 4096; }

// Groups the (expert, token) pairs so that pairs of one expert are adjacent, shared
// expert pairs last; token_jobs keeps each token's mix order.
static void build_job_table(const s14_moe_layer_desc &desc, JobTable &tab) {
    if (desc.n_tokens == 0 || desc.n_tokens > kMaxTokens)
        throw ContractError("S14 MoE layer takes 1..8 tokens");
    if (!fused_dim_ok(desc.hidden) || !fused_dim_ok(desc.inter))
        throw ContractError("S14 MoE layer: hidden and intermediate must be 1024, 2048 or 4096");
    if (!desc.routes) throw ContractError("S14 MoE layer: routes is NULL");
    if (desc.shared_page && desc.shared_kind != S14_PAGE_MXFP4 && desc.shared_kind != S14_PAGE_FP8)
        throw ContractError("S14 MoE layer: unknown shared page kind");
    std::memset(&tab, 0, sizeof(tab));
    struct Pair {
        uint32_t token, slot;
        uint16_t expert;
    };
    std::vector<Pair> pairs;
    for (uint32_t t = 0; t < desc.n_tokens; ++t) {
        const s14_token_route &r = desc.routes[t];
        if (r.n_routed > S14_EXPERTS_PER_TOKEN)
            throw ContractError("S14 MoE layer: a token has more than 6 routed experts");
        if (r.n_routed == 0 && !desc.shared_page)
            throw ContractError("S14 MoE layer: a token has no expert at all");
        for (uint32_t j = 0; j < r.n_routed; ++j) {
            if (!r.pages[j]) throw ContractError("S14 MoE layer: routed page address is NULL");
            if (reinterpret_cast<uintptr_t>(r.pages[j]) % 16 != 0)
                throw ContractError("S14 MoE layer: page addresses must be 16-byte aligned");
            if (!std::isfinite(r.weights[j]) || r.weights[j] < 0.0f)
                throw ContractError("S14 MoE layer: route weight must be finite and non-negative");
            for (uint32_t i = 0; i < j; ++i)
                if (r.expert_ids[i] == r.expert_ids[j])
                    throw ContractError("S14 MoE layer: route expert repeated");
            pairs.push_back({t, j, r.expert_ids[j]});
        }
    }
    // stable order: by expert id, then token
    std::vector<uint32_t> order(pairs.size());
    for (uint32_t i = 0; i < order.size(); ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
        return pairs[a].expert < pairs[b].expert;
    });
    std::vector<std::vector<uint8_t>> per_token(desc.n_tokens,
                                                std::vector<uint8_t>(S14_EXPERTS_PER_TOKEN + 1, 0xff));
    uint32_t n = 0;
    for (uint32_t idx : order) {
        const Pair &p = pairs[idx];
        const s14_token_route &r = desc.routes[p.token];
        Job jb;
        jb.page = r.pages[p.slot];
        jb.kind = S14_PAGE_MXFP4;
        jb.token = p.token;
        jb.weight = r.weights[p.slot];
        jb.is_shared = 0;
        jb.out_index = n;
        tab.jobs[n] = jb;
        per_token[p.token][p.slot] = (uint8_t)n;
        ++n;
    }
    if (desc.shared_page) {
        if (reinterpret_cast<uintptr_t>(desc.shared_page) % 16 != 0)
            throw ContractError("S14 MoE layer: page addresses must be 16-byte aligned");
        for (uint32_t t = 0; t < desc.n_tokens; ++t) {
            Job jb;
            jb.page = desc.shared_page;
            jb.kind = desc.shared_kind;
            jb.token = t;
            jb.weight = 1.0f;
            jb.is_shared = 1;
            jb.out_index = n;
            tab.jobs[n] = jb;
            per_token[t][desc.routes[t].n_routed] = (uint8_t)n;
            ++n;
        }
    }
    tab.n_jobs = n;
    tab.n_tokens = desc.n_tokens;
    uint32_t pos = 0;
    for (uint32_t t = 0; t < desc.n_tokens; ++t) {
        tab.token_job_begin[t] = pos;
        const uint32_t cnt = desc.routes[t].n_routed + (desc.shared_page ? 1u : 0u);
        for (uint32_t j = 0; j < cnt; ++j) tab.token_jobs[pos++] = per_token[t][j];
    }
    tab.token_job_begin[desc.n_tokens] = pos;
}

static int32_t enqueue_layer(s14_ctx *ctx, cudaStream_t st, const s14_moe_layer_desc &desc,
                             const float *x, float *y) {
    S14_TRY
    JobTable tab;
    build_job_table(desc, tab);
    if (!x || !y) throw ContractError("S14 MoE layer: x or y is NULL");
    require_aligned(x, 16, "S14 MoE layer x");
    cudaError_t err;
    bool all_mxfp4 = true;
    for (uint32_t j = 0; j < tab.n_jobs; ++j) all_mxfp4 = all_mxfp4 && tab.jobs[j].kind == S14_PAGE_MXFP4;
    const int launched = launch_moe_layer(st, ctx->mode, ctx->sm_count, nullptr, tab, tab.n_tokens,
                                          tab.n_jobs, desc.hidden, desc.inter, x, ctx->h, ctx->d, y,
                                          &err, nullptr, all_mxfp4, ctx->counters, ctx->umma_scratch());
    ctx->last_path = last_layer_path();
    ctx->launches += launched;
    if (err != cudaSuccess) return cuda_fail(err, "S14 MoE layer launch");
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_layer_work_list(uint32_t cta, uint32_t n_ctas, uint32_t n_jobs, uint32_t n_early_jobs,
                                       uint32_t hidden, uint32_t inter, uint32_t *items_out, uint32_t cap,
                                       uint32_t *count) {
    if (!count || (cap && !items_out)) return fail(S14_ERR_CONTRACT, "s14_layer_work_list: NULL argument");
    if (n_ctas == 0 || cta >= n_ctas || (hidden & 511u) || (inter & 511u) || hidden == 0 || inter == 0)
        return fail(S14_ERR_CONTRACT, "s14_layer_work_list: cta outside the grid, or sizes that are not multiples of 512");
    *count = layer_work_list(cta, n_ctas, n_jobs, inter >> 6, hidden >> 7, hidden >> 8, inter >> 8, items_out, cap,
                             n_early_jobs);
    return S14_OK;
}

extern "C" int32_t s14_cmd_moe_layer(s14_ctx *ctx, void *stream, const s14_moe_layer_desc *desc) {
    if (!ctx || !desc) return fail(S14_ERR_CONTRACT, "s14_cmd_moe_layer: NULL argument");
    return enqueue_layer(ctx, stream_of(ctx, stream), *desc, desc->x, desc->y);
}

// ---- allocation-free layer ----------------------------------------------------------
//
// Scratch of s14_moe_layer_noalloc: the hidden vectors between the up and down phases, the
// per-expert down outputs before the mix, and the arrival counters of the fused mix.  File
// scope, so every GPU that loads this library holds kNoAllocBytes of it until the process exits.
static constexpr uint32_t kNoAllocJobs = S14_EXPERTS_PER_TOKEN + 1;  // one token: 6 routed + shared
static __device__ __align__(256) float g_noalloc_h[kNoAllocJobs * kMaxDim];
static __device__ __align__(256) float g_noalloc_d[kNoAllocJobs * kMaxDim];
static __device__ __align__(256) unsigned int g_noalloc_counters[kCounters];

struct NoAllocDevice {
    std::once_flag once;    // several host threads may make a device's first call together
    int32_t rc = S14_OK;    // what the one initialisation returned
    int sm_count = 0;
    float *h = nullptr, *d = nullptr;
    unsigned int *counters = nullptr;
};
static NoAllocDevice g_noalloc[64];

// Resolves the device addresses of the scratch arrays for `device`, which is current.  In host
// code the array names are only handles; the kernels need what cudaGetSymbolAddress returns.
static int32_t noalloc_resolve(int device, NoAllocDevice &nd) {
    cudaDeviceProp prop;
    CUDA_OK(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(S14_ERR_CONTRACT, "s14_moe_layer_noalloc: the kernels are built for sm_100a only");
    CUDA_OK(cudaGetSymbolAddress((void **)&nd.h, g_noalloc_h));
    CUDA_OK(cudaGetSymbolAddress((void **)&nd.d, g_noalloc_d));
    CUDA_OK(cudaGetSymbolAddress((void **)&nd.counters, g_noalloc_counters));
    nd.sm_count = prop.multiProcessorCount;
    return S14_OK;
}

// Once per device and process; every later call (and every thread that lost the race) reads the
// result of that one initialisation.
static int32_t noalloc_setup(int device, NoAllocDevice **out) {
    if (device < 0 || device >= 64) return fail(S14_ERR_CONTRACT, "s14_moe_layer_noalloc: device out of range");
    NoAllocDevice &nd = g_noalloc[device];
    std::call_once(nd.once, [&] { nd.rc = noalloc_resolve(device, nd); });
    if (nd.rc != S14_OK) return fail(nd.rc, "s14_moe_layer_noalloc: the device could not be set up on its first call");
    *out = &nd;
    return S14_OK;
}

// Makes `device` current for the duration of a call and puts the caller's device back afterwards.
struct DeviceScope {
    int previous = -1;
    bool switched = false;
    cudaError_t enter(int device) {
        cudaError_t e = cudaGetDevice(&previous);
        if (e != cudaSuccess) return e;
        if (previous != device) {
            e = cudaSetDevice(device);
            switched = e == cudaSuccess;
        }
        return e;
    }
    ~DeviceScope() {
        if (switched) cudaSetDevice(previous);
    }
};

extern "C" int32_t s14_moe_layer_noalloc(int32_t device, void *stream, uint32_t accumulation,
                                         const s14_moe_layer_desc *desc) {
    S14_TRY
    if (!desc) throw ContractError("s14_moe_layer_noalloc: desc is NULL");
    if (accumulation != S14_ACCUM_PAIRWISE && accumulation != S14_ACCUM_REFERENCE)
        throw ContractError("s14_moe_layer_noalloc: unknown accumulation mode");
    if (desc->n_tokens != 1)
        throw ContractError("s14_moe_layer_noalloc: the static scratch holds one token (6 routed + shared "
                            "experts); got " + std::to_string(desc->n_tokens) + " tokens");
    if (!fused_dim_ok(desc->hidden) || !fused_dim_ok(desc->inter))
        throw ContractError("s14_moe_layer_noalloc: hidden and intermediate must be 1024, 2048 or 4096");
    DeviceScope scope;  // the caller's current device is restored on every way out
    CUDA_OK(scope.enter(device));
    NoAllocDevice *nd = nullptr;
    const int32_t rc = noalloc_setup(device, &nd);
    if (rc != S14_OK) return rc;
    JobTable tab;
    build_job_table(*desc, tab);
    if (!desc->x || !desc->y) throw ContractError("s14_moe_layer_noalloc: x or y is NULL");
    require_aligned(desc->x, 16, "S14 MoE layer x");
    bool all_mxfp4 = true;
    for (uint32_t j = 0; j < tab.n_jobs; ++j) all_mxfp4 = all_mxfp4 && tab.jobs[j].kind == S14_PAGE_MXFP4;
    cudaStream_t st = (cudaStream_t)stream;
    // every call shares the scratch: the counters must start at zero whatever an earlier,
    // interrupted call left behind; h and d are fully overwritten before they are read
    CUDA_OK(cudaMemsetAsync(nd->counters, 0, sizeof(unsigned int) * kCounters, st));
    cudaError_t err;
    launch_moe_layer(st, accumulation, nd->sm_count, nullptr, tab, tab.n_tokens, tab.n_jobs, desc->hidden,
                     desc->inter, desc->x, nd->h, nd->d, desc->y, &err, nullptr, all_mxfp4, nd->counters);
    if (err != cudaSuccess) return cuda_fail(err, "S14 MoE layer launch");
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_moe_layer_host(s14_ctx *ctx, const s14_moe_layer_desc *desc,
                                      const float *host_x, float *host_y) {
    if (!ctx || !desc || !host_x || !host_y)
        return fail(S14_ERR_CONTRACT, "s14_moe_layer_host: NULL argument");
    if (desc->n_tokens == 0 || desc->n_tokens > kMaxTokens || desc->hidden > kMaxDim)
        return fail(S14_ERR_CONTRACT, "s14_moe_layer_host: token count or hidden size out of range");
    const size_t bytes = sizeof(float) * desc->n_tokens * desc->hidden;
    CUDA_OK(cudaMemcpyAsync(ctx->x_stage, host_x, bytes, cudaMemcpyHostToDevice, ctx->compute));
    const int32_t rc = enqueue_layer(ctx, ctx->compute, *desc, ctx->x_stage, ctx->y_stage);
    if (rc != S14_OK) return rc;
    CUDA_OK(cudaMemcpyAsync(host_y, ctx->y_stage, bytes, cudaMemcpyDeviceToHost, ctx->compute));
    CUDA_OK(cudaStreamSynchronize(ctx->compute));
    return S14_OK;
}

static void validate_router(const s14_router_desc &r, bool need_outputs) {
    if (r.n_experts == 0 || r.n_experts > S14_N_ROUTED_EXPERTS)
        throw ContractError("S14 router: 1..256 experts");
    if (r.hidden == 0 || r.hidden % 256 != 0) throw ContractError("S14 router: hidden must be a multiple of 256");
    if (r.n_tokens == 0 || r.n_tokens > kMaxTokens) throw ContractError("S14 router: 1..8 tokens");
    if (r.top_k == 0 || r.top_k > 8 || r.top_k > r.n_experts) throw ContractError("S14 router: top_k must be 1..8");
    if (r.score_fn != S14_SCORE_SIGMOID && r.score_fn != S14_SCORE_SQRT_SOFTPLUS)
        throw ContractError("S14 router: unknown score function");
    if (!std::isfinite(r.route_scale) || r.route_scale <= 0.0f)
        throw ContractError("S14 router: route_scale must be finite and positive");
    if (!r.x || !r.router_weight_bf16) throw ContractError("S14 router: x or weight is NULL");
    if (need_outputs && (!r.ids_out || !r.weights_out))
        throw ContractError("S14 router: ids_out or weights_out is NULL");
    require_aligned(r.x, 16, "S14 router x");
    require_aligned(r.router_weight_bf16, 16, "S14 router weight");
}

extern "C" int32_t s14_cmd_router(s14_ctx *ctx, void *stream, const s14_router_desc *desc) {
    S14_TRY
    if (!ctx || !desc) throw ContractError("s14_cmd_router: NULL argument");
    validate_router(*desc, true);
    cudaError_t err;
    ctx->launches += launch_router(stream_of(ctx, stream), *desc, ctx->scores, ctx->select, nullptr,
                                   nullptr, nullptr, 0, ctx->counters, &err);
    if (err != cudaSuccess) return cuda_fail(err, "S14 router launch");
    return S14_OK;
    S14_CATCH
}

// The router's side of a routed layer call, for launch_moe_layer (which scores the experts inside
// the layer kernel when that kernel can, and launches k_router otherwise).
static FusedRouter router_of(const s14_ctx *ctx, const s14_routed_layer_desc *desc, uint32_t ep_rank,
                             uint32_t ep_world, uint32_t shared_owner) {
    const s14_router_desc &r = desc->router;
    FusedRouter f = {};
    f.weight = r.router_weight_bf16;
    f.bias = r.bias;
    f.scores = ctx->scores;
    f.select = ctx->select;
    f.n_experts = r.n_experts;
    f.score_fn = r.score_fn;
    f.top_k = r.top_k;
    f.route_scale = r.route_scale;
    f.ids_out = r.ids_out;
    f.weights_out = r.weights_out;
    f.table_out = ctx->dev_table;
    f.page_table = desc->page_table;
    f.shared_page = desc->shared_page;
    f.shared_kind = desc->shared_kind;
    f.ep_rank = ep_rank;
    f.ep_world = ep_world;
    f.shared_owner = shared_owner;
    return f;
}

extern "C" int32_t s14_cmd_routed_moe_layer(s14_ctx *ctx, void *stream,
                                            const s14_routed_layer_desc *desc) {
    S14_TRY
    if (!ctx || !desc) throw ContractError("s14_cmd_routed_moe_layer: NULL argument");
    const s14_router_desc &r = desc->router;
    validate_router(r, false);
    if (r.n_tokens != 1) throw ContractError("S14 routed layer: one decode token per call");
    if (r.top_k > S14_EXPERTS_PER_TOKEN) throw ContractError("S14 routed layer: top_k must be <= 6");
    if (!fused_dim_ok(r.hidden) || !fused_dim_ok(desc->inter))
        throw ContractError("S14 routed layer: hidden and intermediate must be 1024, 2048 or 4096");
    if (!desc->page_table || !desc->y) throw ContractError("S14 routed layer: page_table or y is NULL");
    if (desc->shared_page && desc->shared_kind != S14_PAGE_MXFP4 && desc->shared_kind != S14_PAGE_FP8)
        throw ContractError("S14 routed layer: unknown shared page kind");
    cudaStream_t st = stream_of(ctx, stream);
    cudaError_t err;
    const KernelMarks *km = ctx->timing ? &ctx->marks : nullptr;
    const FusedRouter fr = router_of(ctx, desc, 0, 1, 0);
    JobTable unused;
    unused.n_jobs = 0;
    const uint32_t n_jobs = r.top_k + (desc->shared_page ? 1u : 0u);
    ctx->launches += launch_moe_layer(st, ctx->mode, ctx->sm_count, ctx->dev_table, unused, 1, n_jobs,
                                      r.hidden, desc->inter, r.x, ctx->h, ctx->d, desc->y, &err, km,
                                      !desc->shared_page || desc->shared_kind == S14_PAGE_MXFP4, ctx->counters,
                                      ctx->umma_scratch(), &fr);
    ctx->last_path = last_layer_path();
    if (err != cudaSuccess) return cuda_fail(err, "S14 routed MoE layer launch");
    if (km) {
        CUDA_OK(cudaStreamSynchronize(st));
        for (int i = 0; i < 4; ++i) {
            float ms = 0.0f;
            CUDA_OK(cudaEventElapsedTime(&ms, km->ev[i], km->ev[i + 1]));
            ctx->kernel_ms[i] += ms;
        }
        ctx->timed_calls += 1;
    }
    return S14_OK;
    S14_CATCH
}

// ---- decode stack ---------------------------------------------------------------------

struct s14_stack {
    s14_ctx *ctx = nullptr;
    s14_stack_config cfg{};
    std::vector<StackLayer> layers;
    StackLayer *dev_layers = nullptr;
    float *hbuf = nullptr;  // [2][hidden]: the tokens between layers
    float *ybuf = nullptr;  // [hidden]: a layer's output when the layers are launched one by one
};

extern "C" int32_t s14_stack_create(s14_ctx *ctx, const s14_stack_config *config, const s14_stack_layer *layers,
                                    s14_stack **out) {
    S14_TRY
    if (!ctx || !config || !layers || !out) throw ContractError("s14_stack_create: NULL argument");
    *out = nullptr;
    const s14_stack_config &c = *config;
    if (c.n_layers == 0 || c.n_layers > 62) throw ContractError("S14 stack: 1..62 layers");
    if (c.n_experts == 0 || c.n_experts > S14_N_ROUTED_EXPERTS) throw ContractError("S14 stack: 1..256 experts");
    if (!fused_dim_ok(c.hidden) || !fused_dim_ok(c.inter))
        throw ContractError("S14 stack: hidden and intermediate must be 1024, 2048 or 4096");
    if (c.top_k == 0 || c.top_k > S14_EXPERTS_PER_TOKEN || c.top_k > c.n_experts)
        throw ContractError("S14 stack: top_k must be 1..6");
    if (c.score_fn != S14_SCORE_SIGMOID && c.score_fn != S14_SCORE_SQRT_SOFTPLUS)
        throw ContractError("S14 stack: unknown score function");
    if (!std::isfinite(c.route_scale) || c.route_scale <= 0.0f)
        throw ContractError("S14 stack: route_scale must be finite and positive");
    if (c.shared_kind != S14_PAGE_MXFP4 && c.shared_kind != S14_PAGE_FP8)
        throw ContractError("S14 stack: unknown shared page kind");
    std::unique_ptr<s14_stack> st(new s14_stack());
    st->ctx = ctx;
    st->cfg = c;
    const bool has_shared = layers[0].shared_page != nullptr;
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        const s14_stack_layer &in = layers[l];
        if (!in.router_weight_bf16 || !in.page_table) throw ContractError("S14 stack: router weight or page table is NULL");
        if ((in.shared_page != nullptr) != has_shared)
            throw ContractError("S14 stack: either every layer has a shared expert or none has");
        require_aligned(in.router_weight_bf16, 16, "S14 stack router weight");
        if (in.shared_page) require_aligned(in.shared_page, 16, "S14 stack shared page");
        StackLayer v;
        v.router_weight = in.router_weight_bf16;
        v.bias = in.bias;
        v.page_table = in.page_table;
        v.shared_page = in.shared_page;
        v.ids_out = in.ids_out;
        v.weights_out = in.weights_out;
        v.y_out = in.y_out;
        st->layers.push_back(v);
    }
    CUDA_OK(cudaSetDevice(ctx->device));
    CUDA_OK(cudaMalloc(&st->dev_layers, sizeof(StackLayer) * c.n_layers));
    CUDA_OK(cudaMemcpy(st->dev_layers, st->layers.data(), sizeof(StackLayer) * c.n_layers, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMalloc(&st->hbuf, sizeof(float) * 2 * c.hidden));
    CUDA_OK(cudaMalloc(&st->ybuf, sizeof(float) * c.hidden));
    *out = st.release();
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_stack_destroy(s14_stack *stack) {
    if (!stack) return S14_OK;
    if (stack->ctx) {
        cudaSetDevice(stack->ctx->device);
        cudaStreamSynchronize(stack->ctx->compute);
    }
    cudaFree(stack->dev_layers);
    cudaFree(stack->hbuf);
    cudaFree(stack->ybuf);
    delete stack;
    return S14_OK;
}

static FusedRouter stack_router(const s14_ctx *ctx, const s14_stack *stack, uint32_t layer) {
    const s14_stack_config &c = stack->cfg;
    const StackLayer &ly = stack->layers[layer];
    FusedRouter f = {};
    f.weight = ly.router_weight;
    f.bias = ly.bias;
    f.scores = ctx->scores;
    f.select = ctx->select;
    f.n_experts = c.n_experts;
    f.score_fn = c.score_fn;
    f.top_k = c.top_k;
    f.route_scale = c.route_scale;
    f.ids_out = ly.ids_out;
    f.weights_out = ly.weights_out;
    f.table_out = ctx->dev_table;
    f.page_table = ly.page_table;
    f.shared_page = ly.shared_page;
    f.shared_kind = c.shared_kind;
    f.ep_rank = 0;
    f.ep_world = 1;
    f.shared_owner = 0;
    f.has_shared = ly.shared_page != nullptr;
    return f;
}

extern "C" int32_t s14_cmd_stack_decode(s14_ctx *ctx, void *stream, s14_stack *stack, const float *x, float *h_out) {
    S14_TRY
    if (!ctx || !stack || !x || !h_out) throw ContractError("s14_cmd_stack_decode: NULL argument");
    if (stack->ctx != ctx) throw ContractError("S14 stack: created for another context");
    require_aligned(x, 16, "S14 stack x");
    const s14_stack_config &c = stack->cfg;
    cudaStream_t st = stream_of(ctx, stream);
    const bool has_shared = stack->layers[0].shared_page != nullptr;
    const uint32_t n_jobs = c.top_k + (has_shared ? 1u : 0u);
    JobTable unused;
    unused.n_jobs = 0;
    const bool tensor_path = ctx->mode == S14_ACCUM_PAIRWISE && ctx->use_umma && (!has_shared || c.shared_kind == S14_PAGE_MXFP4) &&
                             umma_layer_ok(ctx->sm_count, 1, n_jobs, c.hidden, c.inter) &&
                             umma_router_ok(ctx->sm_count, c.n_experts);
    if (tensor_path) {
        FusedRouter fr = stack_router(ctx, stack, 0);
        fr.has_shared = has_shared;
        const cudaError_t err = launch_moe_layer_umma(st, ctx->sm_count, nullptr, unused, x, ctx->d, h_out, ctx->umma.tiles,
                                                      ctx->counters, ctx->status, c.hidden, c.inter, &fr, nullptr,
                                                      ctx->umma.trace, stack->dev_layers, c.n_layers, stack->hbuf,
                                                      c.residual != 0);
        ctx->launches += 1;
        ctx->last_path = S14_LAYER_PATH_TENSOR_STACK;
        if (err != cudaSuccess) return cuda_fail(err, "S14 stack launch");
        return S14_OK;
    }
    // the layers one by one: router and layer kernels into ybuf, then the step to the next token
    const float *cur = x;
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        const FusedRouter fr = stack_router(ctx, stack, l);
        cudaError_t err;
        ctx->launches += launch_moe_layer(st, ctx->mode, ctx->sm_count, ctx->dev_table, unused, 1, n_jobs, c.hidden, c.inter,
                                          cur, ctx->h, ctx->d, stack->ybuf, &err, nullptr,
                                          !has_shared || c.shared_kind == S14_PAGE_MXFP4, ctx->counters, ctx->umma_scratch(), &fr);
        ctx->last_path = last_layer_path();
        if (err != cudaSuccess) return cuda_fail(err, "S14 stack layer launch");
        float *next = (l + 1 == c.n_layers) ? h_out : stack->hbuf + (size_t)((l + 1) & 1u) * c.hidden;
        CUDA_OK(launch_stack_step(st, cur, stack->ybuf, next, stack->layers[l].y_out, c.hidden, c.residual != 0));
        ctx->launches += 1;
        cur = next;
    }
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_stack_decode_host(s14_ctx *ctx, s14_stack *stack, const float *host_x, float *host_h) {
    if (!ctx || !stack || !host_x || !host_h) return fail(S14_ERR_CONTRACT, "s14_stack_decode_host: NULL argument");
    const size_t bytes = sizeof(float) * stack->cfg.hidden;
    CUDA_OK(cudaMemcpyAsync(ctx->x_stage, host_x, bytes, cudaMemcpyHostToDevice, ctx->compute));
    const int32_t rc = s14_cmd_stack_decode(ctx, ctx->compute, stack, ctx->x_stage, ctx->y_host_dev);
    if (rc != S14_OK) return rc;
    CUDA_OK(cudaStreamSynchronize(ctx->compute));
    std::memcpy(host_h, ctx->y_host, bytes);
    return S14_OK;
}

extern "C" int32_t s14_cmd_routed_moe_experts_ep(s14_ctx *ctx, void *stream,
                                                 const s14_routed_layer_desc *desc, uint32_t ep_rank,
                                                 uint32_t ep_world, uint32_t shared_owner,
                                                 float *slots_out) {
    S14_TRY
    if (!ctx || !desc || !slots_out) throw ContractError("s14_cmd_routed_moe_experts_ep: NULL argument");
    const s14_router_desc &r = desc->router;
    validate_router(r, true);
    if (r.n_tokens != 1) throw ContractError("S14 expert-parallel layer: one decode token per call");
    if (r.top_k > S14_EXPERTS_PER_TOKEN) throw ContractError("S14 expert-parallel layer: top_k must be <= 6");
    if (ep_world == 0 || ep_rank >= ep_world || shared_owner >= ep_world)
        throw ContractError("S14 expert-parallel layer: rank / owner outside the world");
    if (!fused_dim_ok(r.hidden) || !fused_dim_ok(desc->inter))
        throw ContractError("S14 expert-parallel layer: hidden and intermediate must be 1024, 2048 or 4096");
    if (!desc->page_table) throw ContractError("S14 expert-parallel layer: page_table is NULL");
    if (desc->shared_page && desc->shared_kind != S14_PAGE_MXFP4 && desc->shared_kind != S14_PAGE_FP8)
        throw ContractError("S14 expert-parallel layer: unknown shared page kind");
    cudaStream_t st = stream_of(ctx, stream);
    const uint32_t n_slots = r.top_k + (desc->shared_page ? 1u : 0u);
    // slots this rank does not own stay zero, so that the ranks' buffers add up exactly
    CUDA_OK(cudaMemsetAsync(slots_out, 0, sizeof(float) * n_slots * r.hidden, st));
    cudaError_t err;
    const FusedRouter fr = router_of(ctx, desc, ep_rank, ep_world, shared_owner);
    JobTable unused;
    unused.n_jobs = 0;
    ctx->launches += launch_moe_layer(st, ctx->mode, ctx->sm_count, ctx->dev_table, unused, 1, n_slots,
                                      r.hidden, desc->inter, r.x, ctx->h, slots_out, nullptr, &err, nullptr,
                                      !desc->shared_page || desc->shared_kind == S14_PAGE_MXFP4,
                                      ctx->counters, ctx->umma_scratch(), &fr);
    ctx->last_path = last_layer_path();
    if (err != cudaSuccess) return cuda_fail(err, "S14 routed MoE layer launch");
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_moe_mix_slots(s14_ctx *ctx, void *stream, const float *slots,
                                         const float *weights_dev, uint32_t n_routed, int32_t has_shared,
                                         float *y, uint32_t hidden) {
    if (!ctx || !slots || !weights_dev || !y || hidden == 0 || n_routed > S14_EXPERTS_PER_TOKEN)
        return fail(S14_ERR_CONTRACT, "s14_cmd_moe_mix_slots: NULL or out-of-range argument");
    CUDA_OK(launch_mix_slots(stream_of(ctx, stream), slots, weights_dev, n_routed, has_shared, y, hidden));
    ctx->launches += 1;
    return S14_OK;
}

// ---- expert-parallel exchange over peer memory ------------------------------------------

// Teardown of the exchange is a contract between the ranks, because every rank's layer kernel stores
// into every other rank's buffer and freeing memory that a peer still has mapped, or still writes
// to, is undefined:
//   1. every rank calls s14_ep_exchange_disconnect: it waits for all work of its device (its own
//      steps, whatever stream they ran on) and closes its mappings of the other ranks' buffers;
//   2. a host barrier over the ranks: after it no rank writes into, or maps, another rank's buffer;
//   3. every rank calls s14_ep_exchange_destroy (or s14_ctx_destroy), which frees its own buffer.
// destroy refuses (S14_ERR_CONTRACT) while the exchange is still connected.
extern "C" int32_t s14_ep_exchange_disconnect(s14_ctx *ctx) {
    if (!ctx) return fail(S14_ERR_CONTRACT, "s14_ep_exchange_disconnect: ctx is NULL");
    if (!ctx->ep.buf) return S14_OK;
    CUDA_OK(cudaSetDevice(ctx->device));
    CUDA_OK(cudaDeviceSynchronize());  // steps may have run on the caller's streams
    for (uint32_t p = 0; p < kMaxEpWorld; ++p) {
        if (ctx->ep.opened[p]) CUDA_OK(cudaIpcCloseMemHandle(ctx->ep.peer[p]));
        ctx->ep.opened[p] = false;
        ctx->ep.peer[p] = nullptr;
    }
    ctx->ep.connected = false;
    return S14_OK;
}

extern "C" int32_t s14_ep_exchange_destroy(s14_ctx *ctx) {
    if (!ctx) return S14_OK;
    if (ctx->ep.connected)
        return fail(S14_ERR_CONTRACT,
                    "S14 expert-parallel exchange: still connected; every rank calls s14_ep_exchange_disconnect, the "
                    "ranks pass a host barrier, and only then is a buffer freed");
    if (ctx->ep.buf) {
        CUDA_OK(cudaSetDevice(ctx->device));
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaFree(ctx->ep.buf));
    }
    ctx->ep.buf = nullptr;
    ctx->ep.world = 0;
    return S14_OK;
}

extern "C" int32_t s14_ep_exchange_create(s14_ctx *ctx, uint32_t rank, uint32_t world, uint32_t hidden,
                                          uint8_t *handle_out) {
    S14_TRY
    if (!ctx) throw ContractError("s14_ep_exchange_create: ctx is NULL");
    if (world < 2 || world > kMaxEpWorld || rank >= world)
        throw ContractError("S14 expert-parallel exchange: 2..8 ranks, rank inside the world");
    if (!fused_dim_ok(hidden)) throw ContractError("S14 expert-parallel exchange: hidden must be 1024, 2048 or 4096");
    if (ctx->ep.buf) throw ContractError("S14 expert-parallel exchange: already created for this context");
    CUDA_OK(cudaSetDevice(ctx->device));
    const size_t bytes = ep_exchange_bytes(hidden);
    CUDA_OK(cudaMalloc(&ctx->ep.buf, bytes));
    CUDA_OK(cudaMemset(ctx->ep.buf, 0, bytes));
    CUDA_OK(cudaDeviceSynchronize());
    ctx->ep.rank = rank;
    ctx->ep.world = world;
    ctx->ep.hidden = hidden;
    if (handle_out) {
        cudaIpcMemHandle_t h;
        static_assert(sizeof(h) == S14_EP_HANDLE_BYTES, "IPC handle size");
        CUDA_OK(cudaIpcGetMemHandle(&h, ctx->ep.buf));
        std::memcpy(handle_out, &h, sizeof(h));
    }
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_ep_exchange_connect(s14_ctx *ctx, const uint8_t *handles) {
    S14_TRY
    if (!ctx || !handles) throw ContractError("s14_ep_exchange_connect: NULL argument");
    if (!ctx->ep.buf) throw ContractError("S14 expert-parallel exchange: create it first");
    if (ctx->ep.connected) throw ContractError("S14 expert-parallel exchange: already connected");
    CUDA_OK(cudaSetDevice(ctx->device));
    for (uint32_t p = 0; p < ctx->ep.world; ++p) {
        if (p == ctx->ep.rank) {
            ctx->ep.peer[p] = ctx->ep.buf;
            continue;
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + (size_t)p * S14_EP_HANDLE_BYTES, sizeof(h));
        void *base = nullptr;
        CUDA_OK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
        ctx->ep.peer[p] = (uint8_t *)base;
        ctx->ep.opened[p] = true;
    }
    ctx->ep.connected = true;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_ep_exchange_connect_local(s14_ctx *ctx, s14_ctx *const *ranks) {
    S14_TRY
    if (!ctx || !ranks) throw ContractError("s14_ep_exchange_connect_local: NULL argument");
    if (!ctx->ep.buf) throw ContractError("S14 expert-parallel exchange: create it first");
    if (ctx->ep.connected) throw ContractError("S14 expert-parallel exchange: already connected");
    for (uint32_t p = 0; p < ctx->ep.world; ++p) {
        const s14_ctx *o = ranks[p];
        if (!o || !o->ep.buf || o->ep.world != ctx->ep.world || o->ep.rank != p || o->ep.hidden != ctx->ep.hidden ||
            o->device != ctx->device)
            throw ContractError("S14 expert-parallel exchange: rank " + std::to_string(p) +
                                " is not an exchange of the same world, hidden size and device");
        ctx->ep.peer[p] = o->ep.buf;
    }
    ctx->ep.connected = true;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_ep_exchange_set_wait_limit(s14_ctx *ctx, uint32_t polls) {
    if (!ctx || polls == 0) return fail(S14_ERR_CONTRACT, "s14_ep_exchange_set_wait_limit: NULL context or zero polls");
    ctx->ep.wait_limit = polls;
    return S14_OK;
}

extern "C" int32_t s14_cmd_routed_moe_layer_ep(s14_ctx *ctx, void *stream, const s14_routed_layer_desc *desc,
                                               uint32_t shared_owner, int32_t wait_and_mix) {
    S14_TRY
    if (!ctx || !desc) throw ContractError("s14_cmd_routed_moe_layer_ep: NULL argument");
    if (!ctx->ep.connected) throw ContractError("S14 expert-parallel layer: the exchange is not connected");
    const s14_router_desc &r = desc->router;
    validate_router(r, false);
    if (r.n_tokens != 1) throw ContractError("S14 expert-parallel layer: one decode token per call");
    if (r.top_k > S14_EXPERTS_PER_TOKEN) throw ContractError("S14 expert-parallel layer: top_k must be <= 6");
    if (shared_owner >= ctx->ep.world) throw ContractError("S14 expert-parallel layer: owner outside the world");
    if (r.hidden != ctx->ep.hidden || !fused_dim_ok(desc->inter))
        throw ContractError("S14 expert-parallel layer: hidden must be the exchange's, intermediate 1024, 2048 or 4096");
    if (!desc->page_table || (wait_and_mix && !desc->y))
        throw ContractError("S14 expert-parallel layer: page_table or y is NULL");
    if (desc->shared_page && desc->shared_kind != S14_PAGE_MXFP4)
        throw ContractError("S14 expert-parallel layer: the exchange over peer memory takes MXFP4 pages only");
    if (ctx->mode != S14_ACCUM_PAIRWISE || !ctx->use_umma)
        throw ContractError("S14 expert-parallel layer: the exchange over peer memory is part of the pairwise tensor-core kernel");
    cudaStream_t st = stream_of(ctx, stream);
    const uint32_t n_slots = r.top_k + (desc->shared_page ? 1u : 0u);
    const FusedRouter fr = router_of(ctx, desc, ctx->ep.rank, ctx->ep.world, shared_owner);
    EpExchange ex = {};
    for (uint32_t p = 0; p < ctx->ep.world; ++p)
        ex.slots[p] = reinterpret_cast<unsigned long long *>(ctx->ep.peer[p]);
    ex.step = reinterpret_cast<uint32_t *>(ctx->ep.buf + ep_exchange_slot_bytes(ctx->ep.hidden));
    ex.world = ctx->ep.world;
    ex.rank = ctx->ep.rank;
    ex.n_slots = n_slots;
    ex.wait_and_mix = wait_and_mix ? 1u : 0u;
    ex.wait_limit = ctx->ep.wait_limit;
    JobTable unused;
    unused.n_jobs = 0;
    cudaError_t err;
    ctx->launches += launch_moe_layer(st, ctx->mode, ctx->sm_count, ctx->dev_table, unused, 1, n_slots, r.hidden,
                                      desc->inter, r.x, ctx->h, ctx->d, desc->y, &err, nullptr, true, ctx->counters,
                                      ctx->umma_scratch(), &fr, &ex);
    ctx->last_path = last_layer_path();
    if (err != cudaSuccess) return cuda_fail(err, "S14 expert-parallel layer launch");
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_routed_moe_layer_host(s14_ctx *ctx, const s14_routed_layer_desc *desc,
                                             const float *host_x, float *host_y, int32_t *host_ids,
                                             float *host_weights) {
    if (!ctx || !desc || !host_x || !host_y)
        return fail(S14_ERR_CONTRACT, "s14_routed_moe_layer_host: NULL argument");
    if (desc->router.hidden == 0 || desc->router.hidden > kMaxDim || desc->router.top_k > 8)
        return fail(S14_ERR_CONTRACT, "s14_routed_moe_layer_host: hidden size or top_k out of range");
    const size_t bytes = sizeof(float) * desc->router.hidden;
    s14_routed_layer_desc d = *desc;
    d.router.x = ctx->x_stage;
    d.router.n_tokens = 1;
    d.router.ids_out = ctx->ids_host_dev;
    d.router.weights_out = ctx->w_host_dev;
    d.y = ctx->y_host_dev;
    CUDA_OK(cudaMemcpyAsync(ctx->x_stage, host_x, bytes, cudaMemcpyHostToDevice, ctx->compute));
    const int32_t rc = s14_cmd_routed_moe_layer(ctx, ctx->compute, &d);
    if (rc != S14_OK) return rc;
    CUDA_OK(cudaStreamSynchronize(ctx->compute));
    std::memcpy(host_y, ctx->y_host, bytes);
    if (host_ids) std::memcpy(host_ids, ctx->ids_host, sizeof(int32_t) * d.router.top_k);
    if (host_weights) std::memcpy(host_weights, ctx->w_host, sizeof(float) * d.router.top_k);
    return S14_OK;
}

extern "C" int32_t s14_cmd_head_logits(s14_ctx *ctx, void *stream, const float *x, uint32_t n_tokens,
                                       const uint16_t *weight_bf16, uint32_t n_rows, uint32_t hidden,
                                       float *logits_out, uint32_t logits_stride) {
    S14_TRY
    if (!ctx || !x || !weight_bf16 || !logits_out) throw ContractError("s14_cmd_head_logits: NULL argument");
    if (n_tokens == 0 || n_tokens > kMaxTokens) throw ContractError("S14 head: 1..8 tokens");
    if (n_rows == 0 || hidden == 0 || hidden % 8 != 0)
        throw ContractError("S14 head: rows must be non-zero and hidden a multiple of 8");
    if (n_tokens > 1 && logits_stride < n_rows) throw ContractError("S14 head: logits stride < rows");
    require_aligned(x, 16, "S14 head x");
    require_aligned(weight_bf16, 16, "S14 head weight");
    CUDA_OK(launch_head_logits(stream_of(ctx, stream), ctx->sm_count, x, n_tokens, weight_bf16, n_rows,
                               hidden, logits_out, logits_stride));
    ctx->launches += 1;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_greedy_argmax(s14_ctx *ctx, void *stream, const float *logits,
                                         uint32_t vocab, int64_t *result) {
    if (!ctx || !logits || !result || vocab == 0)
        return fail(S14_ERR_CONTRACT, "s14_cmd_greedy_argmax: NULL or empty argument");
    CUDA_OK(launch_greedy_argmax(stream_of(ctx, stream), logits, vocab, result));
    ctx->launches += 1;
    return S14_OK;
}

// ---- page pool ----------------------------------------------------------------------

struct s14_pool {
    s14_ctx *ctx = nullptr;
    uint8_t *device_base = nullptr;
    std::vector<uint8_t> host_base;  // s14_pool_create_host
    std::unique_ptr<VramPool> pool;
    cudaEvent_t transfer_fence = nullptr;
    bool fence_recorded = false;
};

static ExpertKey key_of(s14_expert_key k) { return ExpertKey{k.layer, k.kind, k.slot}; }
static s14_expert_key key_to_c(const ExpertKey &k) {
    s14_expert_key o;
    std::memset(&o, 0, sizeof(o));
    o.layer = k.layer;
    o.kind = k.kind;
    o.slot = k.slot;
    return o;
}
static SlotBinding binding_of(s14_slot_binding b) { return SlotBinding{key_of(b.key), b.slot, b.generation}; }
static s14_slot_binding binding_to_c(const SlotBinding &b) {
    s14_slot_binding o;
    std::memset(&o, 0, sizeof(o));
    o.key = key_to_c(b.key);
    o.slot = b.slot;
    o.generation = b.generation;
    return o;
}
static LoadingReservation reservation_of(const s14_loading_reservation &r) {
    LoadingReservation o;
    o.key = key_of(r.key);
    o.slot = r.slot;
    o.generation = r.generation;
    if (r.has_evicted) o.evicted = key_of(r.evicted);
    return o;
}
static s14_loading_reservation reservation_to_c(const LoadingReservation &r) {
    s14_loading_reservation o;
    std::memset(&o, 0, sizeof(o));
    o.key = key_to_c(r.key);
    o.slot = r.slot;
    o.generation = r.generation;
    o.has_evicted = r.evicted.has_value() ? 1 : 0;
    if (r.evicted) o.evicted = key_to_c(*r.evicted);
    return o;
}

extern "C" int32_t s14_pool_create(s14_ctx *ctx, uint32_t n_slots, uint64_t slot_bytes, s14_pool **out) {
    S14_TRY
    if (!out) throw ContractError("s14_pool_create: out is NULL");
    *out = nullptr;
    std::unique_ptr<s14_pool> p(new s14_pool());
    p->pool.reset(new VramPool(n_slots, slot_bytes, nullptr));  // validates sizes first
    if (ctx) {
        if (slot_bytes % 16 != 0) throw PoolError("VRAM slot size must be a multiple of 16 bytes");
        CUDA_OK(cudaSetDevice(ctx->device));
        void *base = nullptr;
        CUDA_OK(cudaMalloc(&base, (size_t)n_slots * slot_bytes));
        p->device_base = (uint8_t *)base;
        p->pool.reset(new VramPool(n_slots, slot_bytes, p->device_base));
        p->ctx = ctx;
        CUDA_OK(cudaEventCreateWithFlags(&p->transfer_fence, cudaEventDisableTiming));
    }
    *out = p.release();
    return S14_OK;
    S14_CATCH
}

// A pool whose slots are host memory: the bookkeeping of s14_pool_create with memory a CPU test can
// read (the expert loader's tests); no kernel can use it.
extern "C" int32_t s14_pool_create_host(uint32_t n_slots, uint64_t slot_bytes, s14_pool **out) {
    S14_TRY
    if (!out) throw ContractError("s14_pool_create_host: out is NULL");
    *out = nullptr;
    std::unique_ptr<s14_pool> p(new s14_pool());
    p->pool.reset(new VramPool(n_slots, slot_bytes, nullptr));  // validates sizes first
    p->host_base.assign((size_t)n_slots * slot_bytes, 0);
    p->pool.reset(new VramPool(n_slots, slot_bytes, p->host_base.data()));
    *out = p.release();
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_destroy(s14_pool *pool) {
    if (!pool) return S14_OK;
    if (pool->ctx) {
        cudaSetDevice(pool->ctx->device);
        cudaStreamSynchronize(pool->ctx->copy);
        cudaStreamSynchronize(pool->ctx->compute);
        if (pool->transfer_fence) cudaEventDestroy(pool->transfer_fence);
        cudaFree(pool->device_base);
    }
    delete pool;
    return S14_OK;
}

extern "C" uint32_t s14_pool_capacity(const s14_pool *p) { return p ? p->pool->capacity() : 0; }
extern "C" uint64_t s14_pool_slot_bytes(const s14_pool *p) { return p ? p->pool->slot_bytes() : 0; }
extern "C" uint32_t s14_pool_n_loaded(const s14_pool *p) { return p ? p->pool->n_loaded() : 0; }
extern "C" uint64_t s14_pool_total_bytes(const s14_pool *p) { return p ? p->pool->total_bytes() : 0; }
extern "C" uint64_t s14_pool_slot_offset(const s14_pool *p, uint32_t slot) {
    return p ? p->pool->slot_offset(slot) : 0;
}
extern "C" void *s14_pool_slot_ptr(const s14_pool *p, uint32_t slot) {
    return (p && slot < p->pool->capacity()) ? p->pool->slot_ptr(slot) : nullptr;
}

extern "C" int32_t s14_pool_lookup(s14_pool *p, s14_expert_key key, int32_t *found, uint32_t *slot) {
    S14_TRY
    if (!p || !found) throw ContractError("s14_pool_lookup: NULL argument");
    auto r = p->pool->lookup(key_of(key));
    *found = r ? 1 : 0;
    if (r && slot) *slot = *r;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_lookup_and_pin(s14_pool *p, s14_expert_key key, int32_t *found,
                                           s14_slot_binding *lease) {
    S14_TRY
    if (!p || !found || !lease) throw ContractError("s14_pool_lookup_and_pin: NULL argument");
    auto r = p->pool->lookup_and_pin(key_of(key));
    *found = r ? 1 : 0;
    if (r) *lease = binding_to_c(*r);
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_reserve_loading_generation(s14_pool *p, s14_expert_key key,
                                                       s14_loading_reservation *out) {
    S14_TRY
    if (!p || !out) throw ContractError("s14_pool_reserve_loading_generation: NULL argument");
    *out = reservation_to_c(p->pool->reserve_loading_generation(key_of(key)));
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_mark_ready(s14_pool *p, uint32_t slot, s14_expert_key key) {
    S14_TRY
    if (!p) throw ContractError("s14_pool_mark_ready: NULL argument");
    p->pool->mark_ready(slot, key_of(key));
    return S14_OK;
    S14_CATCH
}

static std::vector<LoadingReservation> reservations_of(const s14_loading_reservation *r, uint32_t n) {
    std::vector<LoadingReservation> v;
    for (uint32_t i = 0; i < n; ++i) v.push_back(reservation_of(r[i]));
    return v;
}

extern "C" int32_t s14_pool_validate_publish_batch(const s14_pool *p, const s14_loading_reservation *r,
                                                   uint32_t count) {
    S14_TRY
    if (!p || (count && !r)) throw ContractError("s14_pool_validate_publish_batch: NULL argument");
    p->pool->validate_publish_batch(reservations_of(r, count));
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_publish_batch_and_pin(s14_pool *p, const s14_loading_reservation *r,
                                                  uint32_t count, s14_slot_binding *leases_out) {
    S14_TRY
    if (!p || (count && (!r || !leases_out)))
        throw ContractError("s14_pool_publish_batch_and_pin: NULL argument");
    auto leases = p->pool->publish_batch_and_pin(reservations_of(r, count));
    for (size_t i = 0; i < leases.size(); ++i) leases_out[i] = binding_to_c(leases[i]);
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_validate_binding(const s14_pool *p, s14_slot_binding binding) {
    S14_TRY
    if (!p) throw ContractError("s14_pool_validate_binding: NULL argument");
    p->pool->validate_binding(binding_of(binding));
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_release_after_compute_fence(s14_pool *p, s14_slot_binding lease) {
    S14_TRY
    if (!p) throw ContractError("s14_pool_release_after_compute_fence: NULL argument");
    p->pool->release_after_compute_fence(binding_of(lease));
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_cancel_loading(s14_pool *p, uint32_t slot, s14_expert_key key) {
    S14_TRY
    if (!p) throw ContractError("s14_pool_cancel_loading: NULL argument");
    p->pool->cancel_loading(slot, key_of(key));
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_cancel_reservation(s14_pool *p, s14_loading_reservation reservation) {
    S14_TRY
    if (!p) throw ContractError("s14_pool_cancel_reservation: NULL argument");
    p->pool->cancel_reservation(reservation_of(reservation));
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_upload_page_async(s14_pool *p, const s14_loading_reservation *reservation,
                                              const void *host_bytes, uint64_t bytes) {
    S14_TRY
    if (!p || !reservation || !host_bytes) throw ContractError("s14_pool_upload_page_async: NULL argument");
    if (!p->ctx) throw PoolError("this pool has no device memory (bookkeeping-only pool)");
    if (bytes > p->pool->slot_bytes())
        throw PoolError("expert page is too large for VRAM slot: " + std::to_string(bytes) + " > " +
                        std::to_string(p->pool->slot_bytes()) + " bytes");
    // the reservation must still be the live one: same slot, key and generation
    p->pool->validate_publish_batch({reservation_of(*reservation)});
    CUDA_OK(cudaMemcpyAsync(p->pool->slot_ptr(reservation->slot), host_bytes, bytes,
                            cudaMemcpyHostToDevice, p->ctx->copy));
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_pool_transfer_fence(s14_pool *p) {
    if (!p || !p->ctx) return fail(S14_ERR_POOL, "pool has no device");
    CUDA_OK(cudaEventRecord(p->transfer_fence, p->ctx->copy));
    p->fence_recorded = true;
    return S14_OK;
}

extern "C" int32_t s14_pool_wait_transfer_fence(s14_pool *p) {
    if (!p || !p->ctx) return fail(S14_ERR_POOL, "pool has no device");
    if (!p->fence_recorded) return S14_OK;
    CUDA_OK(cudaEventSynchronize(p->transfer_fence));
    return S14_OK;
}

extern "C" int32_t s14_pool_compute_wait_transfer(s14_pool *p, void *compute_stream) {
    if (!p || !p->ctx) return fail(S14_ERR_POOL, "pool has no device");
    if (!p->fence_recorded) return S14_OK;
    CUDA_OK(cudaStreamWaitEvent(stream_of(p->ctx, compute_stream), p->transfer_fence, 0));
    return S14_OK;
}

extern "C" int32_t s14_host_alloc_pinned(uint64_t bytes, void **out) {
    if (!out || bytes == 0) return fail(S14_ERR_CONTRACT, "s14_host_alloc_pinned: bad argument");
    CUDA_OK(cudaHostAlloc(out, bytes, cudaHostAllocDefault));
    return S14_OK;
}

extern "C" int32_t s14_host_free_pinned(void *ptr) {
    if (ptr) CUDA_OK(cudaFreeHost(ptr));
    return S14_OK;
}

// ---- expert loader ------------------------------------------------------------------

// Pinned staging buffers, one cudaMemcpyAsync per page on the context's copy stream, one event per
// ring entry.
struct CudaTransferEngine : TransferEngine {
    s14_ctx *ctx;
    std::vector<uint8_t *> bufs;
    std::vector<cudaEvent_t> fences;
    CudaTransferEngine(s14_ctx *c, uint32_t depth, uint64_t bytes) : ctx(c) {
        cuda_check(cudaSetDevice(c->device), "expert loader");
        for (uint32_t i = 0; i < depth; ++i) {
            void *p = nullptr;
            cuda_check(cudaHostAlloc(&p, bytes, cudaHostAllocDefault), "expert loader staging buffer");
            bufs.push_back((uint8_t *)p);
            cudaEvent_t e = nullptr;
            cuda_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "expert loader fence");
            fences.push_back(e);
        }
    }
    ~CudaTransferEngine() override {
        for (auto e : fences) cudaEventDestroy(e);
        for (auto b : bufs) cudaFreeHost(b);
    }
    uint8_t *staging(uint32_t entry) override { return bufs[entry]; }
    void submit(uint32_t entry, uint8_t *dst, uint64_t bytes) override {
        cuda_check(cudaMemcpyAsync(dst, bufs[entry], bytes, cudaMemcpyHostToDevice, ctx->copy), "expert page upload");
        cuda_check(cudaEventRecord(fences[entry], ctx->copy), "expert page fence");
    }
    void wait(uint32_t entry) override { cuda_check(cudaEventSynchronize(fences[entry]), "expert page fence wait"); }
};

// For a pool in host memory (s14_pool_create_host; tests without a GPU): the copy runs when it is
// waited for, the latest moment a real transfer may still read its staging buffer.
struct HostTransferEngine : TransferEngine {
    struct Job {
        uint8_t *dst = nullptr;
        uint64_t bytes = 0;
    };
    std::vector<std::vector<uint8_t>> bufs;
    std::vector<Job> jobs;
    HostTransferEngine(uint32_t depth, uint64_t bytes) : bufs(depth, std::vector<uint8_t>(bytes)), jobs(depth) {}
    uint8_t *staging(uint32_t entry) override { return bufs[entry].data(); }
    void submit(uint32_t entry, uint8_t *dst, uint64_t bytes) override {
        if (!dst) throw PoolError("this pool has no memory (bookkeeping-only pool)");
        jobs[entry] = Job{dst, bytes};
    }
    void wait(uint32_t entry) override {
        if (jobs[entry].dst) std::memcpy(jobs[entry].dst, bufs[entry].data(), jobs[entry].bytes);
        jobs[entry] = Job{};
    }
};

struct s14_loader {
    s14_pool *pool = nullptr;
    std::unique_ptr<TransferEngine> engine;
    std::unique_ptr<ExpertLoader> loader;
};

extern "C" int32_t s14_loader_create(s14_pool *pool, uint32_t pipeline_depth, s14_loader **out) {
    S14_TRY
    if (!pool || !out) throw ContractError("s14_loader_create: NULL argument");
    *out = nullptr;
    if (pipeline_depth == 0 || pipeline_depth > 64) throw PoolError("expert loader: pipeline depth must be 1..64");
    if (!pool->pool->base()) throw PoolError("this pool has no memory (bookkeeping-only pool)");
    std::unique_ptr<s14_loader> l(new s14_loader());
    l->pool = pool;
    if (pool->ctx) l->engine.reset(new CudaTransferEngine(pool->ctx, pipeline_depth, pool->pool->slot_bytes()));
    else l->engine.reset(new HostTransferEngine(pipeline_depth, pool->pool->slot_bytes()));
    l->loader.reset(new ExpertLoader(*pool->pool, *l->engine, pipeline_depth, pool->pool->slot_bytes()));
    *out = l.release();
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_loader_destroy(s14_loader *loader) {
    if (!loader) return S14_OK;
    S14_TRY
    std::unique_ptr<s14_loader> own(loader);
    own->loader->wait_all();  // only submitted transfers are waited for
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_loader_enqueue_from_buf(s14_loader *loader, s14_expert_key key, const void *data, uint64_t bytes,
                                               uint32_t *slot_out) {
    S14_TRY
    if (!loader || !slot_out) throw ContractError("s14_loader_enqueue_from_buf: NULL argument");
    *slot_out = loader->loader->enqueue_from_buf(key_of(key), (const uint8_t *)data, bytes);
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_loader_batch_enqueue_from_bufs(s14_loader *loader, const s14_expert_key *keys,
                                                      const void *const *datas, const uint64_t *sizes, uint32_t n,
                                                      uint32_t *slots_out) {
    S14_TRY
    if (!loader || (n && (!keys || !datas || !sizes || !slots_out)))
        throw ContractError("s14_loader_batch_enqueue_from_bufs: NULL argument");
    std::vector<ExpertKey> k;
    std::vector<const uint8_t *> d;
    std::vector<uint64_t> z;
    for (uint32_t i = 0; i < n; ++i) {
        k.push_back(key_of(keys[i]));
        d.push_back((const uint8_t *)datas[i]);
        z.push_back(sizes[i]);
    }
    const std::vector<uint32_t> slots = loader->loader->batch_enqueue_from_bufs(k, d, z);
    for (uint32_t i = 0; i < n; ++i) slots_out[i] = slots[i];
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_loader_wait_all(s14_loader *loader) {
    S14_TRY
    if (!loader) throw ContractError("s14_loader_wait_all: loader is NULL");
    loader->loader->wait_all();
    return S14_OK;
    S14_CATCH
}

extern "C" uint32_t s14_loader_in_flight(const s14_loader *loader) { return loader ? loader->loader->in_flight() : 0; }
extern "C" uint64_t s14_loader_stat_loads(const s14_loader *loader) { return loader ? loader->loader->stat_loads : 0; }
extern "C" uint64_t s14_loader_stat_bytes(const s14_loader *loader) { return loader ? loader->loader->stat_bytes : 0; }

// ---- route page transaction ---------------------------------------------------------

struct s14_moe_pages {
    std::unique_ptr<S14MoePages> pages;
};
struct s14_route_load_batch {
    RouteLoadBatch batch;
};
struct s14_moe_compute_lease {
    S14MoeComputeLeaseBatch lease;
};

static RouteDecision route_of(const s14_route_decision &r) {
    RouteDecision d;
    d.layer = r.layer;
    d.kind = r.kind == 0 ? RouterKind::Hash : RouterKind::Score;
    const uint32_t n = r.n > S14_EXPERTS_PER_TOKEN ? S14_EXPERTS_PER_TOKEN : r.n;
    d.expert_ids.assign(r.expert_ids, r.expert_ids + n);
    d.weights.assign(r.weights, r.weights + n);
    return d;
}

extern "C" int32_t s14_route_validate_for(const s14_route_decision *route, uint32_t profile) {
    S14_TRY
    if (!route) throw ContractError("s14_route_validate_for: route is NULL");
    if (profile > 1) throw ContractError("unknown graph profile");
    if (route->n != S14_EXPERTS_PER_TOKEN) throw ContractError("profile requires top-6 ids and weights");
    route_of(*route).validate_for((GraphProfile)profile);
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_moe_pages_create_ex(s14_pool *routed_pool, s14_pool *shared_pool,
                                           uint32_t profile, uint64_t min_routed_bytes,
                                           uint64_t min_shared_bytes, s14_moe_pages **out) {
    S14_TRY
    if (!routed_pool || !shared_pool || !out) throw ContractError("s14_moe_pages_create: NULL argument");
    if (profile > 1) throw ContractError("unknown graph profile");
    std::unique_ptr<s14_moe_pages> p(new s14_moe_pages());
    p->pages.reset(new S14MoePages(*routed_pool->pool, *shared_pool->pool, (GraphProfile)profile,
                                   min_routed_bytes, min_shared_bytes));
    *out = p.release();
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_moe_pages_create(s14_pool *routed_pool, s14_pool *shared_pool, uint32_t profile,
                                        s14_moe_pages **out) {
    return s14_moe_pages_create_ex(routed_pool, shared_pool, profile, S14_EXPERT_PAGE_BYTES,
                                   S14_SHARED_EXPERT_PAGE_BYTES, out);
}

extern "C" int32_t s14_moe_pages_destroy(s14_moe_pages *pages) {
    delete pages;
    return S14_OK;
}

extern "C" int32_t s14_moe_pages_begin_after_official_route(s14_moe_pages *pages,
                                                            const s14_route_decision *route,
                                                            s14_route_load_batch **batch) {
    S14_TRY
    if (!pages || !route || !batch) throw ContractError("begin_after_official_route: NULL argument");
    *batch = nullptr;
    if (route->n != S14_EXPERTS_PER_TOKEN) throw ContractError("profile requires top-6 ids and weights");
    std::unique_ptr<s14_route_load_batch> b(new s14_route_load_batch());
    b->batch = pages->pages->begin_after_official_route(route_of(*route));
    *batch = b.release();
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_route_load_batch_missing(const s14_route_load_batch *batch,
                                                s14_loading_reservation *reservations_out,
                                                int32_t *is_shared_out, uint32_t *count) {
    if (!batch || !reservations_out || !is_shared_out || !count)
        return fail(S14_ERR_CONTRACT, "s14_route_load_batch_missing: NULL argument");
    uint32_t n = 0;
    for (const PageState &p : batch->batch.routed_pages)
        if (p.loading) {
            reservations_out[n] = reservation_to_c(p.reservation);
            is_shared_out[n] = 0;
            ++n;
        }
    if (batch->batch.shared_page.loading) {
        reservations_out[n] = reservation_to_c(batch->batch.shared_page.reservation);
        is_shared_out[n] = 1;
        ++n;
    }
    *count = n;
    return S14_OK;
}

extern "C" int32_t s14_moe_pages_publish_after_transfer_fence(s14_moe_pages *pages,
                                                              s14_route_load_batch *batch,
                                                              s14_moe_compute_lease **lease) {
    if (!pages || !batch || !lease) return fail(S14_ERR_CONTRACT, "publish_after_transfer_fence: NULL argument");
    *lease = nullptr;
    std::unique_ptr<s14_route_load_batch> owned(batch);  // consumed either way
    S14_TRY
    std::unique_ptr<s14_moe_compute_lease> l(new s14_moe_compute_lease());
    l->lease = pages->pages->publish_after_transfer_fence(std::move(owned->batch));
    *lease = l.release();
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_moe_compute_lease_bindings(const s14_moe_compute_lease *lease,
                                                  s14_slot_binding routed_out[S14_EXPERTS_PER_TOKEN],
                                                  s14_slot_binding *shared_out,
                                                  uint16_t ids_out[S14_EXPERTS_PER_TOKEN],
                                                  float weights_out[S14_EXPERTS_PER_TOKEN]) {
    if (!lease) return fail(S14_ERR_CONTRACT, "s14_moe_compute_lease_bindings: lease is NULL");
    const S14MoeComputeLeaseBatch &l = lease->lease;
    for (size_t i = 0; i < l.routed.size() && i < S14_EXPERTS_PER_TOKEN; ++i) {
        if (routed_out) routed_out[i] = binding_to_c(l.routed[i]);
        if (ids_out) ids_out[i] = l.expert_ids[i];
        if (weights_out) weights_out[i] = l.route_weights[i];
    }
    if (shared_out) *shared_out = binding_to_c(l.shared);
    return S14_OK;
}

extern "C" int32_t s14_moe_pages_release_after_compute_fence(s14_moe_pages *pages,
                                                             s14_moe_compute_lease *lease) {
    S14_TRY
    if (!pages || !lease) throw ContractError("release_after_compute_fence: NULL argument");
    pages->pages->release_after_compute_fence(lease->lease);
    delete lease;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_moe_pages_cancel(s14_moe_pages *pages, s14_route_load_batch *batch) {
    if (!pages || !batch) return fail(S14_ERR_CONTRACT, "s14_moe_pages_cancel: NULL argument");
    std::unique_ptr<s14_route_load_batch> owned(batch);
    S14_TRY
    pages->pages->cancel(std::move(owned->batch));
    return S14_OK;
    S14_CATCH
}

// ---- a block of tokens through one layer, grouped by expert ----------------------------
//
// The workspace of the grouped tensor-core kernels (s14_moe_block.cu) for up to max_tokens tokens:
// chunk and item tables, the tokens' and the (token, route) pairs' digit tiles, the pairs' expert
// outputs, router scratch, and a pinned staging buffer for routes that come from the host.
struct s14_block {
    s14_ctx *ctx = nullptr;
    int device = 0;           // the context's device (the object may outlive the context; its calls may not)
    uint32_t hidden = 0, inter = 0, max_tokens = 0;
    BlockWork w{};
    float *scores = nullptr, *select = nullptr;   // [max_tokens, 256]
    unsigned int *counter = nullptr;              // the router kernel's arrival counter
    int32_t *ids = nullptr;                       // [max_tokens, 6] routes of the host-route call, on the device
    float *weights = nullptr;
    const uint8_t **pages = nullptr;
    uint8_t *stage = nullptr;                     // pinned: ids | weights | pages of one call
    cudaEvent_t staged = nullptr;                 // the staging buffer's last copy has left it
    bool stage_busy = false;
    bool residual = false;                        // y = x + moe(x)
    bool official = false;                        // the official expert arithmetic (s14_block_set_semantics)
    // expert-parallel exchange inside the block kernels: this rank's buffer (two pair buffers, then two rows of
    // flag words) and the ranks' buffers as mapped here
    struct {
        uint8_t *buf = nullptr;
        size_t pair_bytes = 0;
        uint32_t rank = 0, world = 0, calls = 0, wait_limit = 1u << 22;
        uint8_t *peer[kMaxEpWorld] = {};
        bool opened[kMaxEpWorld] = {};
        bool connected = false;
        unsigned int *counter = nullptr;
    } ep;
};

static constexpr uint32_t kBlockMaxTokens = 1024;

extern "C" int32_t s14_block_destroy(s14_block *blk) {
    if (!blk) return S14_OK;
    if (blk->ep.connected)
        return fail(S14_ERR_CONTRACT,
                    "s14_block_destroy: the expert-parallel exchange is still connected; every rank calls "
                    "s14_block_ep_disconnect, the ranks pass a host barrier, then the objects are destroyed");
    cudaSetDevice(blk->device);
    cudaDeviceSynchronize();
    cudaFree(blk->w.chunks);
    cudaFree(blk->w.counts);
    cudaFree(blk->w.xdig);
    cudaFree(blk->w.xexp);
    cudaFree(blk->w.hdig);
    cudaFree(blk->w.hexp);
    cudaFree(blk->w.d);
    cudaFree(blk->w.hval);
    cudaFree(blk->scores);
    cudaFree(blk->select);
    cudaFree(blk->counter);
    cudaFree(blk->ids);
    cudaFree(blk->weights);
    cudaFree(blk->pages);
    cudaFreeHost(blk->stage);
    cudaFree(blk->ep.buf);
    cudaFree(blk->ep.counter);
    if (blk->staged) cudaEventDestroy(blk->staged);
    delete blk;
    return S14_OK;
}

extern "C" int32_t s14_block_create(s14_ctx *ctx, uint32_t hidden, uint32_t inter, uint32_t max_tokens, s14_block **out) {
    if (!ctx || !out) return fail(S14_ERR_CONTRACT, "s14_block_create: NULL argument");
    *out = nullptr;
    if (max_tokens == 0 || max_tokens > kBlockMaxTokens)
        return fail(S14_ERR_CONTRACT, "s14_block_create: 1..1024 tokens");
    CUDA_OK(cudaSetDevice(ctx->device));
    if (!moe_block_ok(ctx->sm_count, hidden, inter, S14_N_ROUTED_EXPERTS, S14_EXPERTS_PER_TOKEN))
        return fail(S14_ERR_CONTRACT, "s14_block_create: hidden and intermediate must be multiples of 512 up to 4096");
    std::unique_ptr<s14_block, int32_t (*)(s14_block *)> blk(new s14_block(), s14_block_destroy);
    blk->ctx = ctx;
    blk->device = ctx->device;
    blk->hidden = hidden;
    blk->inter = inter;
    blk->max_tokens = max_tokens;
    const size_t T = max_tokens, P = T * (S14_EXPERTS_PER_TOKEN + 1), C = moe_block_max_chunks(max_tokens);
    const size_t R = S14_EXPERTS_PER_TOKEN;
    CUDA_OK(cudaMalloc((void **)&blk->w.chunks, C * sizeof(BlockChunk)));
    CUDA_OK(cudaMalloc((void **)&blk->w.counts, 64));
    CUDA_OK(cudaMalloc((void **)&blk->w.xdig, T * (hidden >> 8) * 2048u));
    CUDA_OK(cudaMalloc((void **)&blk->w.xexp, T * (hidden >> 5)));
    CUDA_OK(cudaMalloc((void **)&blk->w.hdig, P * (inter >> 8) * 2048u));
    CUDA_OK(cudaMalloc((void **)&blk->w.hexp, P * (inter >> 5)));
    CUDA_OK(cudaMalloc((void **)&blk->w.d, P * hidden * sizeof(float)));
    // the pairs' hidden values as F32 (large blocks and the official arithmetic); zero, so that the slot of a
    // pair without a route always holds a finite value
    CUDA_OK(cudaMalloc((void **)&blk->w.hval, P * inter * sizeof(float)));
    CUDA_OK(cudaMemset(blk->w.hval, 0, P * inter * sizeof(float)));
    CUDA_OK(cudaMalloc((void **)&blk->scores, T * S14_N_ROUTED_EXPERTS * sizeof(float)));
    CUDA_OK(cudaMalloc((void **)&blk->select, T * S14_N_ROUTED_EXPERTS * sizeof(float)));
    CUDA_OK(cudaMalloc((void **)&blk->counter, 64));
    CUDA_OK(cudaMalloc((void **)&blk->ids, T * R * sizeof(int32_t)));
    CUDA_OK(cudaMalloc((void **)&blk->weights, T * R * sizeof(float)));
    CUDA_OK(cudaMalloc((void **)&blk->pages, T * R * sizeof(uint8_t *)));
    CUDA_OK(cudaHostAlloc((void **)&blk->stage, T * R * 16u, cudaHostAllocDefault));
    CUDA_OK(cudaEventCreateWithFlags(&blk->staged, cudaEventDisableTiming));
    CUDA_OK(cudaMemset(blk->w.counts, 0, 64));
    CUDA_OK(cudaMemset(blk->counter, 0, 64));
    *out = blk.release();
    return S14_OK;
}

// After the stream is synchronised: counts[3] of the last call (an expert id outside the table).
static int32_t block_launch(s14_block *blk, cudaStream_t st, const float *x, float *y, const int32_t *ids,
                            const float *weights, const uint8_t *const *pages, const uint8_t *const *page_table,
                            const uint8_t *shared_page, uint32_t n_tokens, uint32_t top_k, uint32_t n_experts) {
    s14_ctx *ctx = blk->ctx;
    cudaError_t err;
    ctx->launches += launch_moe_block(st, ctx->sm_count, blk->w, x, y, ids, weights, pages, page_table, shared_page, n_tokens,
                                      top_k, n_experts, blk->hidden, blk->inter, ctx->status, &err, 0, blk->residual, 0, 1, nullptr,
                                      nullptr, false, blk->official);
    ctx->last_path = S14_LAYER_PATH_TENSOR_BLOCK;
    if (err != cudaSuccess) return cuda_fail(err, "S14 MoE block launch");
    return S14_OK;
}

extern "C" int32_t s14_cmd_moe_block(s14_ctx *ctx, void *stream, s14_block *blk, const s14_moe_layer_desc *desc) {
    S14_TRY
    if (!ctx || !blk || !desc) throw ContractError("s14_cmd_moe_block: NULL argument");
    if (blk->ctx != ctx) throw ContractError("s14_cmd_moe_block: the block object belongs to another context");
    if (desc->hidden != blk->hidden || desc->inter != blk->inter)
        throw ContractError("s14_cmd_moe_block: sizes differ from the block object's");
    if (desc->n_tokens == 0 || desc->n_tokens > blk->max_tokens)
        throw ContractError("s14_cmd_moe_block: more tokens than the block object was created for");
    if (!desc->routes || !desc->x || !desc->y) throw ContractError("s14_cmd_moe_block: routes, x or y is NULL");
    if (desc->shared_page && desc->shared_kind != S14_PAGE_MXFP4)
        throw ContractError("s14_cmd_moe_block: the grouped kernels take MXFP4 pages only");
    require_aligned(desc->x, 16, "S14 MoE block x");
    if (desc->shared_page) require_aligned(desc->shared_page, 16, "S14 MoE block shared page");
    const uint32_t T = desc->n_tokens, R = S14_EXPERTS_PER_TOKEN;
    CUDA_OK(cudaSetDevice(ctx->device));
    if (blk->stage_busy) CUDA_OK(cudaEventSynchronize(blk->staged));
    int32_t *h_ids = reinterpret_cast<int32_t *>(blk->stage);
    float *h_w = reinterpret_cast<float *>(blk->stage + (size_t)T * R * 4u);
    const uint8_t **h_pages = reinterpret_cast<const uint8_t **>(blk->stage + (size_t)T * R * 8u);
    for (uint32_t t = 0; t < T; ++t) {
        const s14_token_route &r = desc->routes[t];
        if (r.n_routed > R) throw ContractError("s14_cmd_moe_block: a token has more than 6 routed experts");
        if (r.n_routed == 0 && !desc->shared_page) throw ContractError("s14_cmd_moe_block: a token has no expert at all");
        for (uint32_t j = 0; j < R; ++j) {
            h_ids[t * R + j] = -1;
            h_w[t * R + j] = 0.0f;
            h_pages[t * R + j] = nullptr;
            if (j >= r.n_routed) continue;
            if (!r.pages[j] || reinterpret_cast<uintptr_t>(r.pages[j]) % 16 != 0)
                throw ContractError("s14_cmd_moe_block: a routed page address is NULL or not 16-byte aligned");
            if (!std::isfinite(r.weights[j]) || r.weights[j] < 0.0f)
                throw ContractError("s14_cmd_moe_block: route weight must be finite and non-negative");
            if (r.expert_ids[j] >= S14_N_ROUTED_EXPERTS) throw ContractError("s14_cmd_moe_block: expert id above 255");
            for (uint32_t i = 0; i < j; ++i)
                if (r.expert_ids[i] == r.expert_ids[j]) throw ContractError("s14_cmd_moe_block: route expert repeated");
            h_ids[t * R + j] = r.expert_ids[j];
            h_w[t * R + j] = r.weights[j];
            h_pages[t * R + j] = r.pages[j];
        }
    }
    cudaStream_t st = stream_of(ctx, stream);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    CUDA_OK(cudaStreamIsCapturing(st, &cap));
    if (cap != cudaStreamCaptureStatusNone)
        throw ContractError("s14_cmd_moe_block: the routes are staged through one host buffer per block object, so the call "
                            "cannot be captured into a CUDA graph; s14_cmd_routed_moe_block can");
    CUDA_OK(cudaMemcpyAsync(blk->ids, h_ids, (size_t)T * R * 4u, cudaMemcpyHostToDevice, st));
    CUDA_OK(cudaMemcpyAsync(blk->weights, h_w, (size_t)T * R * 4u, cudaMemcpyHostToDevice, st));
    CUDA_OK(cudaMemcpyAsync(blk->pages, h_pages, (size_t)T * R * 8u, cudaMemcpyHostToDevice, st));
    CUDA_OK(cudaEventRecord(blk->staged, st));
    blk->stage_busy = true;
    return block_launch(blk, st, desc->x, desc->y, blk->ids, blk->weights, blk->pages, nullptr, desc->shared_page, T, R,
                        S14_N_ROUTED_EXPERTS);
    S14_CATCH
}

// What the routed block calls share: checks, the router's two launches; rd receives the router with its outputs set.
static int32_t routed_block_router(s14_ctx *ctx, cudaStream_t st, s14_block *blk, const s14_routed_layer_desc *desc,
                                   s14_router_desc *rd, bool need_outputs) {
    S14_TRY
    if (blk->ctx != ctx) throw ContractError("S14 MoE block: the block object belongs to another context");
    const s14_router_desc &r = desc->router;
    if (r.hidden != blk->hidden || desc->inter != blk->inter) throw ContractError("S14 MoE block: sizes differ from the block object's");
    if (r.hidden > 8192u) throw ContractError("S14 MoE block: hidden above 8192");
    if (r.n_tokens == 0 || r.n_tokens > blk->max_tokens)
        throw ContractError("S14 MoE block: more tokens than the block object was created for");
    if (r.n_experts == 0 || r.n_experts > S14_N_ROUTED_EXPERTS) throw ContractError("S14 router: 1..256 experts");
    if (r.top_k == 0 || r.top_k > S14_EXPERTS_PER_TOKEN || r.top_k > r.n_experts)
        throw ContractError("S14 MoE block: top_k must be 1..6");
    if (r.score_fn != S14_SCORE_SIGMOID && r.score_fn != S14_SCORE_SQRT_SOFTPLUS)
        throw ContractError("S14 router: unknown score function");
    if (!std::isfinite(r.route_scale) || r.route_scale <= 0.0f)
        throw ContractError("S14 router: route_scale must be finite and positive");
    if (!r.x || !r.router_weight_bf16 || !desc->page_table) throw ContractError("S14 MoE block: x, router weight or page table is NULL");
    if (need_outputs && (!r.ids_out || !r.weights_out)) throw ContractError("S14 MoE block: ids_out or weights_out is NULL");
    if (desc->shared_page && desc->shared_kind != S14_PAGE_MXFP4)
        throw ContractError("S14 MoE block: the grouped kernels take MXFP4 pages only");
    require_aligned(r.x, 16, "S14 router x");
    require_aligned(r.router_weight_bf16, 16, "S14 router weight");
    CUDA_OK(cudaSetDevice(ctx->device));
    *rd = r;
    if (!rd->ids_out) rd->ids_out = blk->ids;
    if (!rd->weights_out) rd->weights_out = blk->weights;
    cudaError_t err;
    ctx->launches += launch_router_batch(st, *rd, blk->scores, blk->select, &err);
    if (err != cudaSuccess) return cuda_fail(err, "S14 router launch");
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_routed_moe_block(s14_ctx *ctx, void *stream, s14_block *blk, const s14_routed_layer_desc *desc) {
    if (!ctx || !blk || !desc) return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block: NULL argument");
    if (!desc->y) return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block: y is NULL");
    cudaStream_t st = stream_of(ctx, stream);
    s14_router_desc rd;
    const int32_t rc = routed_block_router(ctx, st, blk, desc, &rd, false);
    if (rc != S14_OK) return rc;
    return block_launch(blk, st, rd.x, desc->y, rd.ids_out, rd.weights_out, nullptr, desc->page_table, desc->shared_page,
                        rd.n_tokens, rd.top_k, rd.n_experts);
}

// Expert parallel: the block's pairs of the experts this rank owns (expert e on rank e mod world, the shared
// expert on shared_owner) into pairs_out [n_tokens * 7, hidden], zeros elsewhere; no mix.
extern "C" int32_t s14_cmd_routed_moe_block_experts_ep(s14_ctx *ctx, void *stream, s14_block *blk,
                                                       const s14_routed_layer_desc *desc, uint32_t ep_rank, uint32_t ep_world,
                                                       uint32_t shared_owner, float *pairs_out) {
    if (!ctx || !blk || !desc || !pairs_out) return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block_experts_ep: NULL argument");
    if (blk->official) return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block_experts_ep: the official arithmetic runs on one GPU");
    const bool by_token = shared_owner == S14_EP_SHARED_BY_TOKEN;
    if (ep_world == 0 || ep_world > kMaxEpWorld || ep_rank >= ep_world || (!by_token && shared_owner >= ep_world))
        return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block_experts_ep: rank or shared owner outside the world (1..8 ranks)");
    cudaStream_t st = stream_of(ctx, stream);
    s14_router_desc rd;
    const int32_t rc = routed_block_router(ctx, st, blk, desc, &rd, true);
    if (rc != S14_OK) return rc;
    cudaError_t err;
    ctx->launches += launch_moe_block(st, ctx->sm_count, blk->w, rd.x, nullptr, rd.ids_out, rd.weights_out, nullptr, desc->page_table,
                                      (by_token || shared_owner == ep_rank) ? desc->shared_page : nullptr, rd.n_tokens, rd.top_k,
                                      rd.n_experts, blk->hidden, blk->inter, ctx->status, &err, 0, false, ep_rank, ep_world, pairs_out,
                                      nullptr, by_token);
    ctx->last_path = S14_LAYER_PATH_TENSOR_BLOCK;
    if (err != cudaSuccess) return cuda_fail(err, "S14 MoE block launch");
    return S14_OK;
}

// ---- expert parallel with the exchange inside the block kernels ----
static size_t block_ep_bytes(const s14_block *blk) { return 2u * blk->ep.pair_bytes + 2u * 8u * kMaxEpWorld; }

extern "C" int32_t s14_block_ep_create(s14_block *blk, uint32_t rank, uint32_t world, uint8_t *handle_out) {
    S14_TRY
    if (!blk) throw ContractError("s14_block_ep_create: blk is NULL");
    if (world < 2 || world > kMaxEpWorld || rank >= world) throw ContractError("s14_block_ep_create: 2..8 ranks, rank inside the world");
    if (blk->ep.buf) throw ContractError("s14_block_ep_create: already created for this block object");
    if (blk->official) throw ContractError("s14_block_ep_create: the official arithmetic runs on one GPU");
    CUDA_OK(cudaSetDevice(blk->device));
    blk->ep.pair_bytes = ((size_t)blk->max_tokens * (S14_EXPERTS_PER_TOKEN + 1) * blk->hidden * sizeof(float) + 255u) & ~(size_t)255u;
    CUDA_OK(cudaMalloc(&blk->ep.buf, block_ep_bytes(blk)));
    CUDA_OK(cudaMemset(blk->ep.buf, 0, block_ep_bytes(blk)));
    CUDA_OK(cudaMalloc(&blk->ep.counter, 64));
    CUDA_OK(cudaMemset(blk->ep.counter, 0, 64));
    CUDA_OK(cudaDeviceSynchronize());
    blk->ep.rank = rank;
    blk->ep.world = world;
    blk->ep.calls = 0;
    if (handle_out) {
        cudaIpcMemHandle_t h;
        static_assert(sizeof(h) == S14_EP_HANDLE_BYTES, "IPC handle size");
        CUDA_OK(cudaIpcGetMemHandle(&h, blk->ep.buf));
        std::memcpy(handle_out, &h, sizeof(h));
    }
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_block_ep_connect(s14_block *blk, const uint8_t *handles) {
    S14_TRY
    if (!blk || !handles) throw ContractError("s14_block_ep_connect: NULL argument");
    if (!blk->ep.buf) throw ContractError("s14_block_ep_connect: create the exchange first");
    if (blk->ep.connected) throw ContractError("s14_block_ep_connect: already connected");
    CUDA_OK(cudaSetDevice(blk->device));
    for (uint32_t p = 0; p < blk->ep.world; ++p) {
        if (p == blk->ep.rank) {
            blk->ep.peer[p] = blk->ep.buf;
            continue;
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + (size_t)p * S14_EP_HANDLE_BYTES, sizeof(h));
        void *base = nullptr;
        CUDA_OK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
        blk->ep.peer[p] = (uint8_t *)base;
        blk->ep.opened[p] = true;
    }
    blk->ep.connected = true;
    return S14_OK;
    S14_CATCH
}

// The ranks are block objects of this process on the same GPU (tests: every rank but the last runs with
// wait_and_mix = 0 - it publishes and returns - so that no launch waits for a later launch of the same GPU).
extern "C" int32_t s14_block_ep_connect_local(s14_block *blk, s14_block *const *ranks) {
    S14_TRY
    if (!blk || !ranks) throw ContractError("s14_block_ep_connect_local: NULL argument");
    if (!blk->ep.buf) throw ContractError("s14_block_ep_connect_local: create the exchange first");
    for (uint32_t p = 0; p < blk->ep.world; ++p) {
        if (!ranks[p] || !ranks[p]->ep.buf || ranks[p]->ep.world != blk->ep.world || ranks[p]->ep.rank != p ||
            ranks[p]->device != blk->device || ranks[p]->ep.pair_bytes != blk->ep.pair_bytes)
            throw ContractError("s14_block_ep_connect_local: the ranks' objects must be created alike, in rank order, on this GPU");
        blk->ep.peer[p] = ranks[p]->ep.buf;
    }
    blk->ep.connected = true;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_block_ep_set_wait_limit(s14_block *blk, uint32_t polls) {
    if (!blk || polls == 0) return fail(S14_ERR_CONTRACT, "s14_block_ep_set_wait_limit: NULL object or zero polls");
    blk->ep.wait_limit = polls;
    return S14_OK;
}

// Teardown as for the one-token exchange: every rank disconnects (waits for its device's work, closes its mappings),
// the ranks pass a host barrier, then the objects are destroyed.
extern "C" int32_t s14_block_ep_disconnect(s14_block *blk) {
    if (!blk) return fail(S14_ERR_CONTRACT, "s14_block_ep_disconnect: blk is NULL");
    if (!blk->ep.buf) return S14_OK;
    CUDA_OK(cudaSetDevice(blk->device));
    CUDA_OK(cudaDeviceSynchronize());
    for (uint32_t p = 0; p < kMaxEpWorld; ++p) {
        if (blk->ep.opened[p]) CUDA_OK(cudaIpcCloseMemHandle(blk->ep.peer[p]));
        blk->ep.opened[p] = false;
        blk->ep.peer[p] = nullptr;
    }
    blk->ep.connected = false;
    return S14_OK;
}

// One call per rank and block: router, grouping of the owned experts' pairs, the two contractions - the down kernel
// stores its rows into every rank's pair buffer and publishes the call's number -, and (wait_and_mix) the mix,
// which waits (bounded; status 0x5508 and no result if it runs out) for every rank's number.
extern "C" int32_t s14_cmd_routed_moe_block_ep(s14_ctx *ctx, void *stream, s14_block *blk, const s14_routed_layer_desc *desc,
                                               uint32_t shared_owner, int32_t wait_and_mix) {
    if (!ctx || !blk || !desc) return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block_ep: NULL argument");
    if (!blk->ep.connected) return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block_ep: the exchange is not connected");
    const bool by_token = shared_owner == S14_EP_SHARED_BY_TOKEN;
    if (!by_token && shared_owner >= blk->ep.world)
        return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block_ep: shared owner outside the world");
    if (wait_and_mix && !desc->y) return fail(S14_ERR_CONTRACT, "s14_cmd_routed_moe_block_ep: y is NULL");
    cudaStream_t st = stream_of(ctx, stream);
    s14_router_desc rd;
    const int32_t rc = routed_block_router(ctx, st, blk, desc, &rd, false);
    if (rc != S14_OK) return rc;
    const uint32_t call = ++blk->ep.calls, parity = call & 1u;
    BlockEp ep = {};
    for (uint32_t p = 0; p < blk->ep.world; ++p) {
        ep.pairs_peer[p] = reinterpret_cast<float *>(blk->ep.peer[p] + parity * blk->ep.pair_bytes);
        ep.flags_peer[p] = reinterpret_cast<unsigned long long *>(blk->ep.peer[p] + 2u * blk->ep.pair_bytes + parity * 8u * kMaxEpWorld);
    }
    ep.flags = ep.flags_peer[blk->ep.rank];
    ep.counter = blk->ep.counter;
    ep.world = blk->ep.world;
    ep.rank = blk->ep.rank;
    ep.call = call;
    ep.wait_limit = blk->ep.wait_limit;
    cudaError_t err;
    ctx->launches += launch_moe_block(st, ctx->sm_count, blk->w, rd.x, nullptr, rd.ids_out, rd.weights_out, nullptr, desc->page_table,
                                      (by_token || shared_owner == blk->ep.rank) ? desc->shared_page : nullptr, rd.n_tokens, rd.top_k,
                                      rd.n_experts, blk->hidden, blk->inter, ctx->status, &err, 0, false, blk->ep.rank, blk->ep.world,
                                      ep.pairs_peer[blk->ep.rank], &ep, by_token);
    ctx->last_path = S14_LAYER_PATH_TENSOR_BLOCK;
    if (err != cudaSuccess) return cuda_fail(err, "S14 MoE block launch");
    if (!wait_and_mix) return S14_OK;
    err = launch_block_mix(st, ep.pairs_peer[blk->ep.rank], rd.ids_out, rd.weights_out, rd.n_tokens, rd.top_k, desc->shared_page != nullptr,
                           blk->residual ? rd.x : nullptr, desc->y, blk->hidden, blk->w.counts, &ep, ctx->status);
    ctx->launches += 1;
    if (err != cudaSuccess) return cuda_fail(err, "S14 MoE block mix launch");
    return S14_OK;
}

// The ordered mix of a block from a pairs buffer (after the ranks' buffers have been added up).
extern "C" int32_t s14_cmd_moe_block_mix(s14_ctx *ctx, void *stream, s14_block *blk, const float *pairs, const int32_t *ids,
                                         const float *weights, uint32_t n_tokens, uint32_t top_k, int32_t has_shared,
                                         const float *x_residual, float *y) {
    if (!ctx || !blk || !pairs || !ids || !weights || !y) return fail(S14_ERR_CONTRACT, "s14_cmd_moe_block_mix: NULL argument");
    if (n_tokens == 0 || n_tokens > blk->max_tokens || top_k == 0 || top_k > S14_EXPERTS_PER_TOKEN)
        return fail(S14_ERR_CONTRACT, "s14_cmd_moe_block_mix: token count or top_k out of range");
    CUDA_OK(cudaSetDevice(ctx->device));
    const cudaError_t err = launch_block_mix(stream_of(ctx, stream), pairs, ids, weights, n_tokens, top_k, has_shared != 0, x_residual, y,
                                             blk->hidden, blk->w.counts);
    ctx->launches += 1;
    if (err != cudaSuccess) return cuda_fail(err, "S14 MoE block mix launch");
    return S14_OK;
}

// The arithmetic of the block's experts: this library's (F32 values, exact sums, one rounding per matvec) or
// the official one of s14_first_real_token/executor.py:712-743.
extern "C" int32_t s14_block_set_semantics(s14_block *blk, uint32_t semantics) {
    S14_TRY
    if (!blk) return fail(S14_ERR_CONTRACT, "s14_block_set_semantics: blk is NULL");
    if (semantics != S14_BLOCK_SEMANTICS_F32 && semantics != S14_BLOCK_SEMANTICS_OFFICIAL)
        return fail(S14_ERR_CONTRACT, "s14_block_set_semantics: unknown semantics");
    if (semantics == S14_BLOCK_SEMANTICS_OFFICIAL) {
        if (blk->ep.buf) return fail(S14_ERR_CONTRACT, "s14_block_set_semantics: the official arithmetic runs on one GPU (the block has an exchange)");
    }
    blk->official = semantics == S14_BLOCK_SEMANTICS_OFFICIAL;
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_block_set_residual(s14_block *blk, int32_t residual) {
    if (!blk) return fail(S14_ERR_CONTRACT, "s14_block_set_residual: blk is NULL");
    blk->residual = residual != 0;
    return S14_OK;
}

// counts of the last call's grouping (after the stream is synchronised): chunks, up items, down
// items, and 1 if an expert id was outside the table (the call then did nothing).
extern "C" int32_t s14_block_last_counts(s14_block *blk, uint32_t counts_out[4]) {
    if (!blk || !counts_out) return fail(S14_ERR_CONTRACT, "s14_block_last_counts: NULL argument");
    CUDA_OK(cudaSetDevice(blk->device));
    CUDA_OK(cudaMemcpy(counts_out, blk->w.counts, 16, cudaMemcpyDeviceToHost));
    return S14_OK;
}


// ---- the steps on either side of the MoE inside one layer ---------------------------------------
static void check_streams(const char *what, uint32_t n_tokens, uint32_t hc, uint32_t hidden, uint32_t dtype) {
    if (n_tokens == 0 || n_tokens > kGlueTokens) throw ContractError(std::string(what) + ": 1..1024 tokens");
    if (hc != 4) throw ContractError(std::string(what) + ": the state has four streams");
    if (hidden == 0 || hidden % 256 != 0 || hidden > 8192) throw ContractError(std::string(what) + ": hidden must be a multiple of 256 up to 8192");
    if (dtype != S14_STREAM_F32 && dtype != S14_STREAM_BF16) throw ContractError(std::string(what) + ": unknown stream type");
}

static int32_t hc_reduce_call(s14_ctx *ctx, void *stream, const s14_hc_params *p, bool head, const void *x, void *reduced,
                              float *post, float *comb, float *pre, const char *what) {
    S14_TRY
    if (!ctx || !p || !x || !reduced) throw ContractError(std::string(what) + ": NULL argument");
    check_streams(what, p->n_tokens, p->hc, p->hidden, p->dtype);
    if (!p->hc_fn || !p->hc_scale || !p->hc_base) throw ContractError(std::string(what) + ": hc_fn, hc_scale or hc_base is NULL");
    if (!head && (!post || !comb)) throw ContractError(std::string(what) + ": post or comb is NULL");
    if (head && !pre) throw ContractError(std::string(what) + ": pre is NULL");
    if (!head && p->sinkhorn_iters == 0) throw ContractError(std::string(what) + ": at least one Sinkhorn round");
    if (!std::isfinite(p->norm_eps) || p->norm_eps <= 0.0f || !std::isfinite(p->hc_eps) || p->hc_eps <= 0.0f)
        throw ContractError(std::string(what) + ": norm_eps and hc_eps must be finite and positive");
    CUDA_OK(cudaSetDevice(ctx->device));
    cudaError_t err;
    ctx->launches += launch_hc_pre(stream_of(ctx, stream), p->dtype == S14_STREAM_BF16, head, p->n_tokens, p->hidden, x, p->hc_fn,
                                   p->hc_scale, p->hc_base, p->norm_eps, p->sinkhorn_iters, p->hc_eps, ctx->glue,
                                   ctx->glue + (size_t)kGlueTokens * 24, reduced, post, comb, pre, &err);
    if (err != cudaSuccess) return cuda_fail(err, what);
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_hc_pre(s14_ctx *ctx, void *stream, const s14_hc_params *params, const void *x, void *reduced,
                                  float *post, float *comb) {
    return hc_reduce_call(ctx, stream, params, false, x, reduced, post, comb, nullptr, "s14_cmd_hc_pre");
}

extern "C" int32_t s14_cmd_hc_head_reduce(s14_ctx *ctx, void *stream, const s14_hc_params *params, const void *x, void *reduced,
                                          float *pre) {
    return hc_reduce_call(ctx, stream, params, true, x, reduced, nullptr, nullptr, pre, "s14_cmd_hc_head_reduce");
}

extern "C" int32_t s14_cmd_hc_post(s14_ctx *ctx, void *stream, uint32_t n_tokens, uint32_t hc, uint32_t hidden, uint32_t dtype,
                                   const void *branch, const void *residual, const float *post, const float *comb, void *merged) {
    S14_TRY
    if (!ctx || !branch || !residual || !post || !comb || !merged) throw ContractError("s14_cmd_hc_post: NULL argument");
    check_streams("s14_cmd_hc_post", n_tokens, hc, hidden, dtype);
    CUDA_OK(cudaSetDevice(ctx->device));
    const cudaError_t err = launch_hc_post(stream_of(ctx, stream), dtype == S14_STREAM_BF16, n_tokens, hidden, branch, residual, post,
                                           comb, merged);
    ctx->launches += 1;
    if (err != cudaSuccess) return cuda_fail(err, "s14_cmd_hc_post");
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_rms_norm(s14_ctx *ctx, void *stream, uint32_t n_tokens, uint32_t hidden, uint32_t dtype, const void *x,
                                    const float *weight, float eps, void *out) {
    S14_TRY
    if (!ctx || !x || !weight || !out) throw ContractError("s14_cmd_rms_norm: NULL argument");
    check_streams("s14_cmd_rms_norm", n_tokens, 4, hidden, dtype);
    if (!std::isfinite(eps) || eps <= 0.0f) throw ContractError("s14_cmd_rms_norm: eps must be finite and positive");
    CUDA_OK(cudaSetDevice(ctx->device));
    const cudaError_t err = launch_rms_norm(stream_of(ctx, stream), dtype == S14_STREAM_BF16, n_tokens, hidden, x, weight, eps, out);
    ctx->launches += 1;
    if (err != cudaSuccess) return cuda_fail(err, "s14_cmd_rms_norm");
    return S14_OK;
    S14_CATCH
}

extern "C" int32_t s14_cmd_router_hash(s14_ctx *ctx, void *stream, const s14_router_desc *desc, const int64_t *tid2eid_rows) {
    S14_TRY
    if (!ctx || !desc || !tid2eid_rows) throw ContractError("s14_cmd_router_hash: NULL argument");
    const s14_router_desc &r = *desc;
    if (r.n_experts == 0 || r.n_experts > S14_N_ROUTED_EXPERTS) throw ContractError("S14 router: 1..256 experts");
    if (r.hidden == 0 || r.hidden % 256 != 0) throw ContractError("S14 router: hidden must be a multiple of 256");
    if (r.n_tokens == 0 || r.n_tokens > kGlueTokens) throw ContractError("s14_cmd_router_hash: 1..1024 tokens");
    if (r.top_k == 0 || r.top_k > 8) throw ContractError("S14 router: top_k must be 1..8");
    if (r.score_fn != S14_SCORE_SIGMOID && r.score_fn != S14_SCORE_SQRT_SOFTPLUS) throw ContractError("S14 router: unknown score function");
    if (!std::isfinite(r.route_scale) || r.route_scale <= 0.0f) throw ContractError("S14 router: route_scale must be finite and positive");
    if (!r.x || !r.router_weight_bf16 || !r.ids_out || !r.weights_out) throw ContractError("S14 router: x, weight, ids_out or weights_out is NULL");
    CUDA_OK(cudaSetDevice(ctx->device));
    const cudaError_t err = launch_router_hash(stream_of(ctx, stream), r, tid2eid_rows);
    ctx->launches += 1;
    if (err != cudaSuccess) return cuda_fail(err, "s14_cmd_router_hash");
    return S14_OK;
    S14_CATCH
}


// ---- the executor's two device steps (s14_runner/src/runner.rs:86-118) as single calls ------------
//
// NativeS14Executor::routed_and_shared_moe_then_hc_post: the FFN site's input (BF16, after hc_pre and
// RMSNorm) through the routed and shared experts, the branch rounded to BF16, expanded into the four
// streams with the site's post / comb.  One token.
extern "C" int32_t s14_exec_routed_and_shared_moe_then_hc_post(s14_ctx *ctx, void *stream, const s14_exec_moe_desc *d) {
    S14_TRY
    if (!ctx || !d) throw ContractError("s14_exec_routed_and_shared_moe_then_hc_post: NULL argument");
    if (!d->route || !d->ffn_input_bf16 || !d->residual_bf16 || !d->post || !d->comb || !d->state_out_bf16)
        throw ContractError("s14_exec_routed_and_shared_moe_then_hc_post: NULL pointer in the descriptor");
    if (!fused_dim_ok(d->hidden) || !fused_dim_ok(d->inter))
        throw ContractError("s14_exec_routed_and_shared_moe_then_hc_post: hidden and intermediate must be 1024, 2048 or 4096");
    CUDA_OK(cudaSetDevice(ctx->device));
    cudaStream_t st = stream_of(ctx, stream);
    CUDA_OK(launch_bf16_to_f32(st, d->ffn_input_bf16, ctx->x_stage, d->hidden));
    s14_moe_layer_desc ld = {};
    ld.hidden = d->hidden;
    ld.inter = d->inter;
    ld.n_tokens = 1;
    ld.shared_kind = d->shared_kind;
    ld.shared_page = d->shared_page;
    ld.routes = d->route;
    const int32_t rc = enqueue_layer(ctx, st, ld, ctx->x_stage, ctx->y_stage);
    if (rc != S14_OK) return rc;
    uint16_t *branch = d->moe_branch_out_bf16 ? d->moe_branch_out_bf16 : ctx->glue16;
    CUDA_OK(launch_f32_to_bf16(st, ctx->y_stage, branch, d->hidden));
    CUDA_OK(launch_hc_post(st, true, 1, d->hidden, branch, d->residual_bf16, d->post, d->comb, d->state_out_bf16));
    ctx->launches += 3;
    return S14_OK;
    S14_CATCH
}

// NativeS14Executor::hc_head_norm_full_logits (final_head.py:152-191): the head's reduce of the four
// streams, RMSNorm, the BF16 head's logits for rows [row_begin, row_begin + n_rows) of the vocabulary.
extern "C" int32_t s14_exec_hc_head_norm_full_logits(s14_ctx *ctx, void *stream, const s14_hc_params *head, const float *norm_weight,
                                                     const uint16_t *head_weight_bf16, uint32_t n_rows, const uint16_t *state_bf16,
                                                     float *logits_out) {
    S14_TRY
    if (!ctx || !head || !norm_weight || !head_weight_bf16 || !state_bf16 || !logits_out)
        throw ContractError("s14_exec_hc_head_norm_full_logits: NULL argument");
    if (head->n_tokens != 1 || head->dtype != S14_STREAM_BF16)
        throw ContractError("s14_exec_hc_head_norm_full_logits: one token, BF16 state");
    if (n_rows == 0) throw ContractError("s14_exec_hc_head_norm_full_logits: no vocabulary rows");
    if (head->hidden > kMaxDim) throw ContractError("s14_exec_hc_head_norm_full_logits: hidden above 4096");
    uint16_t *reduced = ctx->glue16 + 8192, *normed = ctx->glue16 + 2 * 8192;
    float *pre = ctx->glue + (size_t)kGlueTokens * 24 + 512;
    int32_t rc = hc_reduce_call(ctx, stream, head, true, state_bf16, reduced, nullptr, nullptr, pre, "s14_exec_hc_head_norm_full_logits");
    if (rc != S14_OK) return rc;
    cudaStream_t st = stream_of(ctx, stream);
    CUDA_OK(launch_rms_norm(st, true, 1, head->hidden, reduced, norm_weight, head->norm_eps, normed));
    CUDA_OK(launch_bf16_to_f32(st, normed, ctx->x_stage, head->hidden));
    CUDA_OK(launch_head_logits(st, ctx->sm_count, ctx->x_stage, 1, head_weight_bf16, n_rows, head->hidden, logits_out, n_rows));
    ctx->launches += 3;
    return S14_OK;
    S14_CATCH
}
