/*
 * CPU oracle for the S14 MoE expert hot path.  TEST INFRASTRUCTURE ONLY: nothing
 * in the shipped library or in the Python package may link, load or call this
 * file; only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg use it, and there only as the checker or as the timed CPU reference.
 *
 * Every function restates, in plain C, the F32 CPU reference that the
 * reference project keeps in
 *   scheduler/ssd_inference/examples/s14_vulkan_numeric.rs
 * (cited per function below as "numeric.rs:<lines>").  The evaluation order is
 * kept exactly: one output row at a time, k ascending, two separate
 * multiply-then-add steps per packed byte, `(x * decode) * scale` association,
 * no fused multiply-add (build with -ffp-contract=off), correctly rounded F32 exp for SiLU
 * (see s14o_swiglu_limit).
 * Rows are independent, so the OpenMP loop over rows (the reference uses a
 * rayon parallel iterator over rows, numeric.rs:1678, 1701) does not change any
 * result bit.
 *
 * The "_f64" matvecs and the "_acc64" layer accumulate the same exact products in
 * double (the accumulator option of the reference's Python code) and serve as the
 * order-independent value when reporting how far either F32 summation order is
 * from it.
 *
 * The router and LM-head functions restate the Python reference
 *   fast16/research/polaris_meridian_v1/s14_first_real_token/executor.py:638-668
 *   fast16/research/polaris_meridian_v1/local_s14_primitives/final_head.py:113-149
 * with one stated deviation: logits are accumulated in double (the Python code
 * leaves the F32 summation order to the BLAS it happens to run on), rounded to
 * F32 once, so that selection is reproducible on any device.
 *
 * Parity pin: the decode tables and matvecs are checked against the reference's
 * own known-answer vectors (local_s14_primitives/tests/test_primitives.py:37-112)
 * and against outputs of the importable Python reference committed under
 * tests/golden/.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define S14O_API __attribute__((visibility("default")))

/* numeric.rs:1716-1724 */
S14O_API float s14o_e2m1(uint8_t code) {
    static const float magnitude[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float value = magnitude[code & 7];
    return (code & 8) ? -value : value;
}

/* numeric.rs:1726-1728: 2^(code-127); code 0 gives the subnormal 2^-127, 0xFF is
 * rejected by the caller before any decode (s14_vulkan.rs:143-148). */
S14O_API float s14o_ue8m0(uint8_t code) { return ldexpf(1.0f, (int)code - 127); }

/* numeric.rs:1730-1743 */
S14O_API float s14o_e4m3fn(uint8_t code) {
    unsigned exponent = (code >> 3) & 0x0f;
    unsigned mantissa = code & 7;
    float magnitude;
    if (exponent == 0) {
        magnitude = (float)mantissa * ldexpf(1.0f, -9);
    } else {
        magnitude = (1.0f + (float)mantissa / 8.0f) * ldexpf(1.0f, (int)exponent - 7);
    }
    return (code & 0x80) ? -magnitude : magnitude;
}

S14O_API int s14o_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

S14O_API void s14o_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* numeric.rs:1669-1696.  W [n, k/2] bytes (low nibble = even k), S [n, k/32]. */
S14O_API void s14o_mxfp4_matvec(const float *x, const uint8_t *packed_weight,
                                const uint8_t *scale, uint32_t n_rows, uint32_t k,
                                float *y) {
    const size_t packed_k = k / 2, groups = k / 32;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)n_rows; ++n) {
        float sum = 0.0f;
        for (size_t group = 0; group < groups; ++group) {
            const float s = s14o_ue8m0(scale[n * groups + group]);
            const size_t pair_base = group * 16;
            for (size_t pair_in_group = 0; pair_in_group < 16; ++pair_in_group) {
                const size_t pair = pair_base + pair_in_group;
                const uint8_t codes = packed_weight[n * packed_k + pair];
                const size_t k0 = pair * 2;
                sum += x[k0] * s14o_e2m1(codes & 0x0f) * s;
                sum += x[k0 + 1] * s14o_e2m1(codes >> 4) * s;
            }
        }
        y[n] = sum;
    }
}

/* Same products, double accumulation, double result ("truth"). */
S14O_API void s14o_mxfp4_matvec_f64(const double *x, const uint8_t *packed_weight,
                                    const uint8_t *scale, uint32_t n_rows, uint32_t k,
                                    double *y) {
    const size_t packed_k = k / 2, groups = k / 32;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)n_rows; ++n) {
        double sum = 0.0;
        for (size_t group = 0; group < groups; ++group) {
            const double s = ldexp(1.0, (int)scale[n * groups + group] - 127);
            double part = 0.0;
            for (size_t pair = group * 16; pair < group * 16 + 16; ++pair) {
                const uint8_t codes = packed_weight[n * packed_k + pair];
                part += x[pair * 2] * (double)s14o_e2m1(codes & 0x0f);
                part += x[pair * 2 + 1] * (double)s14o_e2m1(codes >> 4);
            }
            sum += part * s;
        }
        y[n] = sum;
    }
}

/* numeric.rs:1698-1714.  W [n, k] bytes, S [ceil(n/128), ceil(k/128)] UE8M0. */
S14O_API void s14o_fp8_matvec(const float *x, const uint8_t *weight, const uint8_t *scale,
                              uint32_t n_rows, uint32_t k, float *y) {
    const size_t k_groups = ((size_t)k + 127) / 128;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)n_rows; ++n) {
        const size_t scale_row = ((size_t)n / 128) * k_groups;
        const size_t weight_row = (size_t)n * k;
        float sum = 0.0f;
        for (size_t k_index = 0; k_index < k; ++k_index) {
            const float s = s14o_ue8m0(scale[scale_row + k_index / 128]);
            sum += x[k_index] * s14o_e4m3fn(weight[weight_row + k_index]) * s;
        }
        y[n] = sum;
    }
}

/* The same loop with one F32 scale per 128x128 block instead of a UE8M0 byte
 * (the Python reference accepts either, local_s14_primitives/fp8.py:37-46). */
S14O_API void s14o_fp8_matvec_f32scale(const float *x, const uint8_t *weight,
                                       const float *scale, uint32_t n_rows, uint32_t k,
                                       float *y) {
    const size_t k_groups = ((size_t)k + 127) / 128;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)n_rows; ++n) {
        const size_t scale_row = ((size_t)n / 128) * k_groups;
        const size_t weight_row = (size_t)n * k;
        float sum = 0.0f;
        for (size_t k_index = 0; k_index < k; ++k_index) {
            const float s = scale[scale_row + k_index / 128];
            sum += x[k_index] * s14o_e4m3fn(weight[weight_row + k_index]) * s;
        }
        y[n] = sum;
    }
}

/* Double-accumulated FP8 matvec; scale_is_f32 selects the scale format. */
S14O_API void s14o_fp8_matvec_f64(const double *x, const uint8_t *weight, const void *scale,
                                  int scale_is_f32, uint32_t n_rows, uint32_t k, double *y) {
    const size_t k_groups = ((size_t)k + 127) / 128;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < (int64_t)n_rows; ++n) {
        const size_t scale_row = ((size_t)n / 128) * k_groups;
        const size_t weight_row = (size_t)n * k;
        double sum = 0.0;
        for (size_t kg = 0; kg < k_groups; ++kg) {
            const double s = scale_is_f32
                                 ? (double)((const float *)scale)[scale_row + kg]
                                 : ldexp(1.0, (int)((const uint8_t *)scale)[scale_row + kg] - 127);
            const size_t k_end = (kg * 128 + 128 < k) ? kg * 128 + 128 : k;
            double part = 0.0;
            for (size_t k_index = kg * 128; k_index < k_end; ++k_index)
                part += x[k_index] * (double)s14o_e4m3fn(weight[weight_row + k_index]);
            sum += part * s;
        }
        y[n] = sum;
    }
}

/* numeric.rs:1543-1556: gate is limited from above only, up on both sides.  The
 * reference calls its platform's F32 exp, whose last bit differs between C libraries
 * (glibc's expf returns a value other than the correctly rounded one for about 80
 * arguments per million).  The oracle pins the platform-independent definition: the
 * correctly rounded F32 exponential, obtained as a double exp rounded once.
 * s14o_swiglu_limit_libm keeps the libm call to measure that difference. */
S14O_API void s14o_swiglu_limit(const float *gate, const float *up, uint32_t n, float *y) {
    for (uint32_t i = 0; i < n; ++i) {
        float g = gate[i] < 10.0f ? gate[i] : 10.0f;
        float u = up[i];
        if (u < -10.0f) u = -10.0f;
        if (u > 10.0f) u = 10.0f;
        const float e = (float)exp(-(double)g);
        y[i] = (g / (1.0f + e)) * u;
    }
}

S14O_API void s14o_swiglu_limit_libm(const float *gate, const float *up, uint32_t n, float *y) {
    for (uint32_t i = 0; i < n; ++i) {
        float g = gate[i] < 10.0f ? gate[i] : 10.0f;
        float u = up[i];
        if (u < -10.0f) u = -10.0f;
        if (u > 10.0f) u = 10.0f;
        y[i] = (g / (1.0f + expf(-g))) * u;
    }
}

/* One expert page as the library lays it out in a pool slot:
 *   [w1 codes n_i*k_h/2][w3 codes][w2 codes n_h*k_i/2][s1][s3][s2]  (MXFP4)
 *   [w1 n_i*k_h][w3][w2][s1][s3][s2]                                (FP8, UE8M0 128x128)
 * hidden = k_h, intermediate = n_i. */
typedef struct {
    const uint8_t *w1, *w3, *w2, *s1, *s3, *s2;
} s14o_expert_view;

static s14o_expert_view mxfp4_view(const uint8_t *page, uint32_t hidden, uint32_t inter) {
    s14o_expert_view v;
    const size_t wb = (size_t)hidden * inter / 2, sb = (size_t)hidden * inter / 32;
    v.w1 = page;
    v.w3 = page + wb;
    v.w2 = page + 2 * wb;
    v.s1 = page + 3 * wb;
    v.s3 = v.s1 + sb;
    v.s2 = v.s3 + sb;
    return v;
}

static size_t fp8_scale_bytes(uint32_t n, uint32_t k) {
    return (((size_t)n + 127) / 128) * (((size_t)k + 127) / 128);
}

static s14o_expert_view fp8_view(const uint8_t *page, uint32_t hidden, uint32_t inter) {
    s14o_expert_view v;
    const size_t wb = (size_t)hidden * inter;
    v.w1 = page;
    v.w3 = page + wb;
    v.w2 = page + 2 * wb;
    v.s1 = page + 3 * wb;
    v.s3 = v.s1 + fp8_scale_bytes(inter, hidden);
    v.s2 = v.s3 + fp8_scale_bytes(inter, hidden);
    return v;
}

/* numeric.rs:1296-1300 (single-expert chain): w1,w3 -> limited SwiGLU -> w2 ->
 * multiply by the route weight.  work must hold 3*inter floats. */
S14O_API void s14o_expert_chain_mxfp4(const float *x, const uint8_t *page, uint32_t hidden,
                                      uint32_t inter, float route_weight, float *work,
                                      float *down_out, float *y) {
    s14o_expert_view v = mxfp4_view(page, hidden, inter);
    float *gate = work, *up = work + inter, *h = work + 2 * (size_t)inter;
    s14o_mxfp4_matvec(x, v.w1, v.s1, inter, hidden, gate);
    s14o_mxfp4_matvec(x, v.w3, v.s3, inter, hidden, up);
    s14o_swiglu_limit(gate, up, inter, h);
    s14o_mxfp4_matvec(h, v.w2, v.s2, hidden, inter, down_out);
    if (y)
        for (uint32_t i = 0; i < hidden; ++i) y[i] = route_weight * down_out[i];
}

/* numeric.rs:929-947 (layer): acc = 0; for each routed expert in route order
 * acc += w_e * down_e; then acc += down_shared (weight 1).  shared_kind: 0 =
 * MXFP4 page, 1 = FP8 page (the reference's shared expert), 2 = no shared expert.
 * work must hold 3*inter + hidden floats. */
S14O_API void s14o_moe_layer(const float *x, const uint8_t *const *routed_pages,
                             const float *route_weights, uint32_t n_routed,
                             const uint8_t *shared_page, int shared_kind, uint32_t hidden,
                             uint32_t inter, float *work, float *y) {
    float *down = work + 3 * (size_t)inter;
    for (uint32_t i = 0; i < hidden; ++i) y[i] = 0.0f;
    for (uint32_t e = 0; e < n_routed; ++e) {
        s14o_expert_chain_mxfp4(x, routed_pages[e], hidden, inter, 0.0f, work, down, NULL);
        for (uint32_t i = 0; i < hidden; ++i) y[i] += route_weights[e] * down[i];
    }
    if (shared_kind == 0) {
        s14o_expert_chain_mxfp4(x, shared_page, hidden, inter, 0.0f, work, down, NULL);
        for (uint32_t i = 0; i < hidden; ++i) y[i] += down[i];
    } else if (shared_kind == 1) {
        s14o_expert_view v = fp8_view(shared_page, hidden, inter);
        float *gate = work, *up = work + inter, *h = work + 2 * (size_t)inter;
        s14o_fp8_matvec(x, v.w1, v.s1, inter, hidden, gate);
        s14o_fp8_matvec(x, v.w3, v.s3, inter, hidden, up);
        s14o_swiglu_limit(gate, up, inter, h);
        s14o_fp8_matvec(h, v.w2, v.s2, hidden, inter, down);
        for (uint32_t i = 0; i < hidden; ++i) y[i] += down[i];
    }
}

/* The reference's layer with the accumulator of every matvec widened to double: each
 * matvec sums its exact products in double and rounds the row result to F32 once; gate,
 * up, the SwiGLU, the hidden vector and the ordered mix stay F32 exactly as in
 * numeric.rs:929-947.  This is what the reference's Python code computes with
 * accumulation_dtype=float64 (local_s14_primitives/mxfp4.py:172-275) and it is free of
 * the summation-order noise of either F32 order.  work: 3*inter + hidden floats,
 * work64: 2*max(hidden, inter) doubles. */
static void matvec_acc64(const float *x, const uint8_t *w, const void *s, int kind, uint32_t n,
                         uint32_t k, double *xd, double *yd, float *y) {
    for (uint32_t i = 0; i < k; ++i) xd[i] = (double)x[i];
    if (kind == 0)
        s14o_mxfp4_matvec_f64(xd, w, (const uint8_t *)s, n, k, yd);
    else
        s14o_fp8_matvec_f64(xd, w, s, 0, n, k, yd);
    for (uint32_t i = 0; i < n; ++i) y[i] = (float)yd[i];
}

S14O_API void s14o_moe_layer_acc64(const float *x, const uint8_t *const *routed_pages,
                                   const float *route_weights, uint32_t n_routed,
                                   const uint8_t *shared_page, int shared_kind, uint32_t hidden,
                                   uint32_t inter, float *work, double *work64, float *y) {
    const uint32_t big = hidden > inter ? hidden : inter;
    float *gate = work, *up = work + inter, *h = work + 2 * (size_t)inter;
    float *down = work + 3 * (size_t)inter;
    double *xd = work64, *yd = work64 + big;
    for (uint32_t i = 0; i < hidden; ++i) y[i] = 0.0f;
    for (uint32_t e = 0; e <= n_routed; ++e) {
        const int is_shared = (e == n_routed);
        if (is_shared && shared_kind == 2) break;
        const uint8_t *page = is_shared ? shared_page : routed_pages[e];
        const int kind = (is_shared && shared_kind == 1) ? 1 : 0;
        s14o_expert_view v = kind ? fp8_view(page, hidden, inter) : mxfp4_view(page, hidden, inter);
        matvec_acc64(x, v.w1, v.s1, kind, inter, hidden, xd, yd, gate);
        matvec_acc64(x, v.w3, v.s3, kind, inter, hidden, xd, yd, up);
        s14o_swiglu_limit(gate, up, inter, h);
        matvec_acc64(h, v.w2, v.s2, kind, hidden, inter, xd, yd, down);
        if (is_shared)
            for (uint32_t i = 0; i < hidden; ++i) y[i] += down[i];
        else
            for (uint32_t i = 0; i < hidden; ++i) y[i] += route_weights[e] * down[i];
    }
}

/* torch's .to(torch.bfloat16).float(): nearest, ties to even (l42_reference.py:356-358). */
static float bf16_round(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return f;
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    memcpy(&f, &u, 4);
    return f;
}

/* The nearest E4M3FN value (ties to even) of |v| <= 448: three mantissa bits, subnormals are
 * multiples of 2^-9 below 2^-6 (torch's .to(torch.float8_e4m3fn).float()). */
static float e4m3fn_round(float v) {
    const float a = fabsf(v);
    float q;
    if (a < 0.015625f) {
        q = rintf(a * 512.0f) / 512.0f;
    } else {
        int e;
        (void)frexpf(a, &e); /* a = m * 2^e, m in [0.5, 1) */
        const float step = ldexpf(1.0f, e - 4);
        q = rintf(a / step) * step;
    }
    return copysignf(q, v);
}

/* l42_reference.py:389-403 (_activation_quant): per group of 128 elements amax = max(|x|, 1e-4),
 * scale = 2^ceil(log2(amax / 448)) with the F32 quotient and the F32 logarithm, the elements divided
 * by the scale, clipped to +-448, rounded to E4M3FN and multiplied by the scale again.  The F32
 * logarithm is taken as the double one rounded to F32 (numpy's log2 of a float32 is within an ulp of
 * that; the two can differ only where amax / 448 is within a few ulps of a power of two).  n must
 * be a multiple of 128. */
S14O_API void s14o_act_quant(const float *x, uint32_t n, float *out) {
    for (uint32_t g = 0; g + 128 <= n; g += 128) {
        float amax = 0.0f;
        for (uint32_t i = 0; i < 128; ++i) amax = fmaxf(amax, fabsf(x[g + i]));
        amax = fmaxf(amax, 1e-4f);
        const float r = amax / 448.0f;
        const float scale = ldexpf(1.0f, (int)ceilf((float)log2((double)r)));
        for (uint32_t i = 0; i < 128; ++i) {
            float v = x[g + i] / scale;
            v = fminf(fmaxf(v, -448.0f), 448.0f);
            out[g + i] = e4m3fn_round(v) * scale;
        }
    }
}

/* The official expert arithmetic of one token (s14_first_real_token/executor.py:712-743 finish_layer with
 * l42_reference.py:405-419 _linear_fp8 / _linear_fp4): every linear quantises its input per 128
 * elements (s14o_act_quant), multiplies with the dequantised weights and rounds the result to BF16;
 * hidden = limited SwiGLU of the BF16 gate and up in F32; a routed expert's hidden values are
 * multiplied by its route weight and rounded to BF16 BEFORE w2, the shared expert's are rounded
 * only; the BF16 outputs are added in F32 in route order, the shared expert last, and the sum is
 * rounded to BF16 (moe_branch).  The reference's product `activation @ weight.T` is a float32 BLAS
 * call whose summation order is the library's; here every dot product is summed in double and
 * rounded to F32 once (the quantised activations have four significant bits, the weights two: the
 * double sums are exact at the magnitudes of this path), then to BF16.  shared_kind: 0 MXFP4 page,
 * 1 FP8 page (the reference's), 2 none.  work: 2*hidden + 4*inter floats, work64: 2*max(hidden,
 * inter) doubles. */
S14O_API void s14o_official_moe_layer(const float *x, const uint8_t *const *routed_pages,
                                      const float *route_weights, uint32_t n_routed,
                                      const uint8_t *shared_page, int shared_kind, uint32_t hidden,
                                      uint32_t inter, float *work, double *work64, float *branch) {
    const uint32_t big = hidden > inter ? hidden : inter;
    float *gate = work, *up = work + inter, *h = work + 2 * (size_t)inter, *hq = work + 3 * (size_t)inter;
    float *xq = work + 4 * (size_t)inter, *down = xq + hidden;
    double *xd = work64, *yd = work64 + big;
    s14o_act_quant(x, hidden, xq);
    for (uint32_t i = 0; i < hidden; ++i) branch[i] = 0.0f;
    for (uint32_t e = 0; e <= n_routed; ++e) {
        const int is_shared = (e == n_routed);
        if (is_shared && shared_kind == 2) break;
        const uint8_t *page = is_shared ? shared_page : routed_pages[e];
        const int kind = (is_shared && shared_kind == 1) ? 1 : 0;
        s14o_expert_view v = kind ? fp8_view(page, hidden, inter) : mxfp4_view(page, hidden, inter);
        matvec_acc64(xq, v.w1, v.s1, kind, inter, hidden, xd, yd, gate);
        matvec_acc64(xq, v.w3, v.s3, kind, inter, hidden, xd, yd, up);
        for (uint32_t i = 0; i < inter; ++i) {
            gate[i] = bf16_round(gate[i]);
            up[i] = bf16_round(up[i]);
        }
        s14o_swiglu_limit(gate, up, inter, h);
        for (uint32_t i = 0; i < inter; ++i) h[i] = bf16_round(is_shared ? h[i] : h[i] * route_weights[e]);
        s14o_act_quant(h, inter, hq);
        matvec_acc64(hq, v.w2, v.s2, kind, hidden, inter, xd, yd, down);
        for (uint32_t i = 0; i < hidden; ++i) branch[i] += bf16_round(down[i]);
    }
    for (uint32_t i = 0; i < hidden; ++i) branch[i] = bf16_round(branch[i]);
}

static float bf16_to_f32(uint16_t bits) {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* executor.py:638-668.  Wr [n_experts, hidden] BF16 bits, bias [n_experts] F32 (may
 * be NULL).  score_fn 0: sigmoid(logit); 1: sqrt(softplus(logit)) (the reference's
 * router, softplus threshold 20 as in torch).  Selection: top_k largest of
 * score+bias, order = descending value, ties -> lowest index.  Weights: unbiased
 * score[idx] / sum(score[idx]) * route_scale, F32, summed in selection order.
 * scores_out / select_out (n_experts each) may be NULL. */
S14O_API void s14o_router(const float *x, const uint16_t *wr_bf16, const float *bias,
                          uint32_t n_experts, uint32_t hidden, int score_fn, uint32_t top_k,
                          float route_scale, int32_t *ids_out, float *weights_out,
                          float *scores_out, float *select_out) {
    float scores[4096], select[4096];
    uint8_t taken[4096];
    if (n_experts > 4096) n_experts = 4096;
#pragma omp parallel for schedule(static)
    for (int64_t e = 0; e < (int64_t)n_experts; ++e) {
        double acc = 0.0;
        const uint16_t *row = wr_bf16 + (size_t)e * hidden;
        for (uint32_t k = 0; k < hidden; ++k) acc += (double)x[k] * (double)bf16_to_f32(row[k]);
        const float logit = (float)acc;
        double s;
        if (score_fn == 0) {
            s = 1.0 / (1.0 + exp(-(double)logit));
        } else {
            const double l = (double)logit;
            s = sqrt(l > 20.0 ? l : log1p(exp(l)));
        }
        scores[e] = (float)s;
        select[e] = scores[e] + (bias ? bias[e] : 0.0f);
        taken[e] = 0;
    }
    for (uint32_t j = 0; j < top_k; ++j) {
        int32_t best = -1;
        for (uint32_t e = 0; e < n_experts; ++e) {
            if (taken[e]) continue;
            if (best < 0 || select[e] > select[best]) best = (int32_t)e;
        }
        taken[best] = 1;
        ids_out[j] = best;
    }
    float sum = 0.0f;
    for (uint32_t j = 0; j < top_k; ++j) sum += scores[ids_out[j]];
    for (uint32_t j = 0; j < top_k; ++j) weights_out[j] = scores[ids_out[j]] / sum * route_scale;
    if (scores_out) memcpy(scores_out, scores, n_experts * sizeof(float));
    if (select_out) memcpy(select_out, select, n_experts * sizeof(float));
}

/* final_head.py:113-149: logits[v] = sum_k x[k] * float(W_bf16[v,k]).  Accumulated
 * in double and rounded to F32 once (the reference leaves the F32 order to BLAS
 * and itself accepts rtol 2e-7 / atol 3e-7 between two chunkings,
 * tests/test_final_head.py:68-70). */
S14O_API void s14o_head_logits(const float *x, const uint16_t *w_bf16, uint32_t vocab,
                               uint32_t hidden, float *logits) {
#pragma omp parallel for schedule(static)
    for (int64_t v = 0; v < (int64_t)vocab; ++v) {
        double acc = 0.0;
        const uint16_t *row = w_bf16 + (size_t)v * hidden;
        for (uint32_t k = 0; k < hidden; ++k) acc += (double)x[k] * (double)bf16_to_f32(row[k]);
        logits[v] = (float)acc;
    }
}

/* scheduler/s14_runner/src/runner.rs:485-508: greedy argmax over all logits,
 * lowest id wins ties, any NaN rejects (-1). */
S14O_API int64_t s14o_greedy_argmax(const float *logits, uint32_t vocab) {
    int64_t best = -1;
    for (uint32_t v = 0; v < vocab; ++v) {
        if (isnan(logits[v])) return -1;
        if (best < 0 || logits[v] > logits[best]) best = v;
    }
    return best;
}

/* numeric.rs:1745-1771.  out = {max_abs, mean_abs, rmse, max_rel(|ref|>1e-5)};
 * returns -1 on a shape error or a non-finite value. */
S14O_API int s14o_error_stats(const float *actual, const float *expected, uint64_t n,
                              double out[4]) {
    if (n == 0) return -1;
    float max_abs = 0.0f, max_rel = 0.0f;
    double sum_abs = 0.0, sum_square = 0.0;
    for (uint64_t i = 0; i < n; ++i) {
        const float a = actual[i], e = expected[i];
        if (!isfinite(a) || !isfinite(e)) return -1;
        const float delta = fabsf(a - e);
        if (delta > max_abs) max_abs = delta;
        sum_abs += (double)delta;
        sum_square += (double)delta * (double)delta;
        if (fabsf(e) > 1.0e-5f) {
            const float rel = delta / fabsf(e);
            if (rel > max_rel) max_rel = rel;
        }
    }
    out[0] = max_abs;
    out[1] = sum_abs / (double)n;
    out[2] = sqrt(sum_square / (double)n);
    out[3] = max_rel;
    return 0;
}

/* ---- the steps on either side of the MoE inside one layer --------------------------------------
 * Hyper-connection reduce / expand, RMSNorm and the head's reduce, restating
 *   fast16/research/polaris_meridian_v1/local_s14_primitives/hc.py:19-148
 *   fast16/research/polaris_meridian_v1/local_s14_primitives/final_head.py:43-110
 * The Python code computes in F32 with torch's CPU kernels, whose summation order inside
 * F.linear / mean and whose exp are not fixed; here the long sums (mean of squares, the dot
 * products with hc_fn) are accumulated in double and rounded to F32 once, exp is evaluated in
 * double and rounded once, and everything else follows the Python expressions operation by
 * operation in F32 (sums over the four streams in stream order).  The golden vectors made by the
 * Python code itself are met within a few F32 ulps (tests/test_oracle_golden.py states the bound).
 * dtype 0: F32 streams; 1: BF16 streams (the reference's state is BF16 [1,1,4,4096]; results are
 * rounded to BF16 where the Python code casts back with .to(original_dtype) / type_as). */
static inline float stream_get(const void *p, size_t i, int dtype) {
    return dtype ? bf16_to_f32(((const uint16_t *)p)[i]) : ((const float *)p)[i];
}
static inline void stream_put(void *p, size_t i, int dtype, float v) {
    if (dtype) {
        const float r = bf16_round(v);
        uint32_t b;
        memcpy(&b, &r, 4);
        ((uint16_t *)p)[i] = (uint16_t)(b >> 16);
    } else {
        ((float *)p)[i] = v;
    }
}
static inline float sigmoid_f32(float v) { return (float)(1.0 / (1.0 + exp(-(double)v))); }

/* hc.py:19-84.  mixes [(2 + hc) * hc], scale [3], base like mixes -> pre [hc], post [hc], comb [hc][hc]. */
S14O_API void s14o_hc_split_sinkhorn(const float *mixes, const float *scale, const float *base, uint32_t hc,
                                     uint32_t iters, float eps, float *pre, float *post, float *comb) {
    for (uint32_t h = 0; h < hc; ++h) {
        pre[h] = sigmoid_f32(mixes[h] * scale[0] + base[h]) + eps;
        post[h] = 2.0f * sigmoid_f32(mixes[hc + h] * scale[1] + base[hc + h]);
    }
    for (uint32_t i = 0; i < hc * hc; ++i) comb[i] = mixes[2 * hc + i] * scale[2] + base[2 * hc + i];
    for (uint32_t i = 0; i < hc; ++i) { /* stable row softmax, + eps */
        float m = comb[i * hc];
        for (uint32_t j = 1; j < hc; ++j) m = comb[i * hc + j] > m ? comb[i * hc + j] : m;
        float s = 0.0f;
        for (uint32_t j = 0; j < hc; ++j) {
            comb[i * hc + j] = (float)exp((double)(comb[i * hc + j] - m));
            s += comb[i * hc + j];
        }
        for (uint32_t j = 0; j < hc; ++j) comb[i * hc + j] = comb[i * hc + j] / s + eps;
    }
    for (uint32_t it = 0; it < iters; ++it) {
        if (it) { /* rows */
            for (uint32_t i = 0; i < hc; ++i) {
                float s = 0.0f;
                for (uint32_t j = 0; j < hc; ++j) s += comb[i * hc + j];
                for (uint32_t j = 0; j < hc; ++j) comb[i * hc + j] = comb[i * hc + j] / (s + eps);
            }
        }
        for (uint32_t j = 0; j < hc; ++j) { /* columns */
            float s = 0.0f;
            for (uint32_t i = 0; i < hc; ++i) s += comb[i * hc + j];
            for (uint32_t i = 0; i < hc; ++i) comb[i * hc + j] = comb[i * hc + j] / (s + eps);
        }
    }
}

/* mixes[m] = (x_flat . fn[m]) * rsqrt(mean(x_flat^2) + norm_eps) for n_mix rows of fn [n_mix][hc * hidden]. */
static void hc_mixes(const void *x, int dtype, const float *fn, uint32_t n_mix, uint32_t n, float norm_eps, float *mixes) {
    double ss = 0.0;
    for (uint32_t i = 0; i < n; ++i) {
        const double v = (double)stream_get(x, i, dtype);
        ss += v * v;
    }
    const float ms = (float)(ss / (double)n);
    const float rs = (float)(1.0 / sqrt((double)(ms + norm_eps)));
    for (uint32_t m = 0; m < n_mix; ++m) {
        double acc = 0.0;
        for (uint32_t i = 0; i < n; ++i) acc += (double)stream_get(x, i, dtype) * (double)fn[(size_t)m * n + i];
        mixes[m] = (float)acc * rs;
    }
}

/* hc.py:87-124 for one token: x [hc][hidden] -> reduced [hidden] (stream dtype), post [hc], comb [hc][hc]. */
S14O_API void s14o_hc_pre(const void *x, int dtype, const float *hc_fn, const float *hc_scale, const float *hc_base,
                          uint32_t hc, uint32_t hidden, float norm_eps, uint32_t iters, float hc_eps, void *reduced,
                          float *post, float *comb) {
    float mixes[64], pre[8];
    if (hc > 6) return;
    hc_mixes(x, dtype, hc_fn, (2 + hc) * hc, hc * hidden, norm_eps, mixes);
    s14o_hc_split_sinkhorn(mixes, hc_scale, hc_base, hc, iters, hc_eps, pre, post, comb);
    for (uint32_t d = 0; d < hidden; ++d) {
        float acc = pre[0] * stream_get(x, d, dtype);
        for (uint32_t h = 1; h < hc; ++h) acc += pre[h] * stream_get(x, (size_t)h * hidden + d, dtype);
        stream_put(reduced, d, dtype, acc);
    }
}

/* hc.py:127-148 for one token: merged[h'] = post[h'] * branch + sum_h comb[h][h'] * residual[h]. */
S14O_API void s14o_hc_post(const void *branch, const void *residual, int dtype, const float *post, const float *comb,
                           uint32_t hc, uint32_t hidden, void *merged) {
    for (uint32_t o = 0; o < hc; ++o) {
        for (uint32_t d = 0; d < hidden; ++d) {
            float s = comb[o] * stream_get(residual, d, dtype);
            for (uint32_t h = 1; h < hc; ++h) s += comb[h * hc + o] * stream_get(residual, (size_t)h * hidden + d, dtype);
            const float v = post[o] * stream_get(branch, d, dtype) + s;
            stream_put(merged, (size_t)o * hidden + d, dtype, v);
        }
    }
}

/* final_head.py:84-110 (and l42_reference.py:421-426): out = w * (x * rsqrt(mean(x^2) + eps)). */
S14O_API void s14o_rms_norm(const void *x, int dtype, const float *w, uint32_t hidden, float eps, void *out) {
    double ss = 0.0;
    for (uint32_t i = 0; i < hidden; ++i) {
        const double v = (double)stream_get(x, i, dtype);
        ss += v * v;
    }
    const float ms = (float)(ss / (double)hidden);
    const float rs = (float)(1.0 / sqrt((double)(ms + eps)));
    for (uint32_t i = 0; i < hidden; ++i) stream_put(out, i, dtype, w[i] * (stream_get(x, i, dtype) * rs));
}

/* final_head.py:43-81 for one token: pre = sigmoid(mixes * scale + base) + eps, reduced = sum_h pre[h] x[h]. */
S14O_API void s14o_hc_head_reduce(const void *x, int dtype, const float *fn, const float *scale, const float *base,
                                  uint32_t hc, uint32_t hidden, float norm_eps, float hc_eps, void *reduced, float *pre) {
    float mixes[8];
    if (hc > 8) return;
    hc_mixes(x, dtype, fn, hc, hc * hidden, norm_eps, mixes);
    for (uint32_t h = 0; h < hc; ++h) pre[h] = sigmoid_f32(mixes[h] * scale[0] + base[h]) + hc_eps;
    for (uint32_t d = 0; d < hidden; ++d) {
        float acc = pre[0] * stream_get(x, d, dtype);
        for (uint32_t h = 1; h < hc; ++h) acc += pre[h] * stream_get(x, (size_t)h * hidden + d, dtype);
        stream_put(reduced, d, dtype, acc);
    }
}

/* executor.py:638-668 for the hash-routed layers (0-2): the ids come from the token's row of
 * tid2eid; the weights are the router's scores of those experts, normalised and scaled. */
S14O_API void s14o_router_hash(const float *x, const uint16_t *wr_bf16, uint32_t n_experts, uint32_t hidden, int score_fn,
                               uint32_t top_k, float route_scale, const int64_t *tid2eid_row, int32_t *ids_out,
                               float *weights_out) {
    float sc[8];
    float sum = 0.0f;
    for (uint32_t j = 0; j < top_k && j < 8; ++j) {
        const int64_t e = tid2eid_row[j];
        ids_out[j] = (int32_t)e;
        double acc = 0.0;
        if (e >= 0 && (uint64_t)e < n_experts) {
            const uint16_t *row = wr_bf16 + (size_t)e * hidden;
            for (uint32_t k = 0; k < hidden; ++k) acc += (double)x[k] * (double)bf16_to_f32(row[k]);
        }
        const double l = (double)(float)acc;
        sc[j] = (float)(score_fn == 0 ? 1.0 / (1.0 + exp(-l)) : sqrt(l > 20.0 ? l : log1p(exp(l))));
        sum += sc[j];
    }
    for (uint32_t j = 0; j < top_k && j < 8; ++j) weights_out[j] = sc[j] / sum * route_scale;
}
