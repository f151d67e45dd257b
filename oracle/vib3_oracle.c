/*
 * CPU oracle for the vib3 MoE decode hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU kernels (Rust, src/compute/kernels.rs) and of
 * the summation order of its CUDA router GEMV (cuda/src/kernels.cu).  The Rust toolchain is
 * not available where this is built, so the arithmetic is restated here operation by
 * operation: same loop order, same f32 rounding points, no fused multiply-add (the Rust code
 * compiles `acc += a * b` to a separate multiply and add; build this file with
 * -ffp-contract=off).  Only tests, the smoke check and the benchmark's CPU-baseline leg may
 * call it; the product library never links or loads it.
 *
 * Pinned against the known-answer vectors of the reference's own tests
 * (tests/integration_test.rs:1709-1785, :1788-1831, :420-451, :454-485, :2300-2374); everything
 * beyond those vectors (Kimi shapes, sigmoid routing, paging) has no fixture in the
 * reference and is pinned only by this restatement and by the reference's CUDA kernels
 * compiled unmodified into oracle/_ref.
 *
 * Each function cites the reference lines it follows.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define VO_API __attribute__((visibility("default")))

/* Row parallelism of the timed CPU baseline: the number of OpenMP threads the row loops use (the
 * reference's rayon pool takes every core).  A launcher that exports OMP_NUM_THREADS=1 to its children
 * would otherwise pin the baseline to one core.  Returns the thread count now in force. */
VO_API int vo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* The compiler flags this file was built with (recorded beside the timed baseline). */
#ifndef VO_CFLAGS
#define VO_CFLAGS "unknown"
#endif
VO_API const char* vo_build_flags(void) { return VO_CFLAGS; }

/* ── 16-bit float helpers (crate `half` 2.7.1 semantics: IEEE round-to-nearest-even) ── */

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

VO_API float vo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * (1.0f / 16777216.0f);
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

VO_API uint16_t vo_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x0200u | ((ax >> 13) & 0x3FFu) : 0));
    }
    if (ax >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (ax < 0x38800000u) { /* |f| < 2^-14: subnormal or zero in f16 */
        if (ax < 0x33000000u) return (uint16_t)sign; /* < 2^-25 -> 0 (ties at 2^-25 go to even = 0) */
        uint32_t e = ax >> 23;
        uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
        uint32_t shift = 126u - e; /* value = m * 2^(e-150); target unit 2^-24 -> shift = 126 - e */
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t e = (ax >> 23) - 112u;
    uint32_t m = ax & 0x7FFFFFu;
    uint32_t q = (e << 10) | (m >> 13);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

VO_API float vo_bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

VO_API uint16_t vo_f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

/* scale_format: 0 = BF16 (what the reference's CPU kernels decode, kernels.rs:2788-2790),
 *               1 = FP16 (what its CUDA kernels decode, kernels.cu:41-47, :140). */
static inline float decode_scale(uint16_t bits, int scale_format) {
    return scale_format == 0 ? vo_bf16_to_f32(bits) : vo_f16_to_f32(bits);
}

/* ── INT4 group-quantised row kernels ──────────────────────────────────────────────────── */

/* One output row of cpu_matmul_int4_grouped (kernels.rs:2768-2821): per-group 16-entry LUT
 * lut[n] = (n - 8) * scale, non-finite or non-positive scales replaced by 1/8
 * (kernels.rs:2791-2795), then a sequential f32 accumulate over the packed bytes, low nibble
 * = even column first.  `lut` is caller-provided scratch of num_groups*16 floats. */
static float int4_row_dot(const float* x, const uint8_t* row_packed, const uint8_t* row_scales,
                          int K, int group_size, int scale_format, float* lut) {
    int packed_k = (K + 1) / 2;
    int num_groups = (K + group_size - 1) / group_size;
    for (int g = 0; g < num_groups; g++) {
        uint16_t sb = (uint16_t)(row_scales[2 * g] | (row_scales[2 * g + 1] << 8));
        float s = decode_scale(sb, scale_format);
        if (!(isfinite(s) && s > 0.0f)) s = 1.0f / 8.0f;
        for (int n = 0; n < 16; n++) lut[g * 16 + n] = (float)(n - 8) * s;
    }
    float acc = 0.0f;
    for (int b = 0; b < packed_k; b++) {
        int col = 2 * b;
        if (col >= K) break;
        int g = col / group_size;
        if (g > num_groups - 1) g = num_groups - 1;
        uint8_t p = row_packed[b];
        acc += x[col] * lut[g * 16 + (p & 0x0F)];
        if (col + 1 < K) acc += x[col + 1] * lut[g * 16 + (p >> 4)];
    }
    return acc;
}

/* Raw f32 row sums of W_page * x for a page laid out [M*ceil(K/2) code bytes][M*groups u16
 * scales] (kernels.rs:2753-2760).  Rows are independent; the reference parallelises over rows
 * with rayon when M >= 64 (kernels.rs:2658, :2823), mirrored with OpenMP. */
VO_API void vo_matmul_int4_rows_f32(const float* x, const uint8_t* page, float* y, int K, int M,
                                    int group_size, int scale_format) {
    int packed_k = (K + 1) / 2;
    int num_groups = (K + group_size - 1) / group_size;
    const uint8_t* scales = page + (size_t)packed_k * M;
#pragma omp parallel if (M >= 64)
    {
        float* lut = (float*)malloc((size_t)num_groups * 16 * sizeof(float));
#pragma omp for schedule(static)
        for (int r = 0; r < M; r++) {
            y[r] = int4_row_dot(x, page + (size_t)r * packed_k, scales + (size_t)r * num_groups * 2,
                                K, group_size, scale_format, lut);
        }
        free(lut);
    }
}

/* cpu_matmul_int4_grouped (kernels.rs:2746-2832): f16 input, f16 output. */
VO_API void vo_matmul_int4(const uint16_t* x_f16, const uint8_t* page, uint16_t* y_f16, int K, int M,
                           int group_size, int scale_format) {
    float* x = (float*)malloc((size_t)K * sizeof(float));
    float* y = (float*)malloc((size_t)(M > 0 ? M : 1) * sizeof(float));
    for (int i = 0; i < K; i++) x[i] = vo_f16_to_f32(x_f16[i]);
    vo_matmul_int4_rows_f32(x, page, y, K, M, group_size, scale_format);
    for (int r = 0; r < M; r++) y_f16[r] = vo_f32_to_f16(y[r]);
    free(x);
    free(y);
}

/* cpu_swiglu_int4 (kernels.rs:2932-3054): up and gate rows accumulated in f32 in the same
 * byte loop, silu = g / (1 + exp(-g)), one f16 rounding of silu * up.  Because the two
 * accumulators never interact, running the row kernel twice gives the same bits. */
VO_API void vo_swiglu_int4_f32in(const float* x, const uint8_t* up_page, const uint8_t* gate_page,
                                 uint16_t* y_f16, int H, int M, int group_size, int scale_format) {
    float* up = (float*)malloc((size_t)(M > 0 ? M : 1) * sizeof(float));
    float* gate = (float*)malloc((size_t)(M > 0 ? M : 1) * sizeof(float));
    vo_matmul_int4_rows_f32(x, up_page, up, H, M, group_size, scale_format);
    vo_matmul_int4_rows_f32(x, gate_page, gate, H, M, group_size, scale_format);
    for (int r = 0; r < M; r++) {
        float g = gate[r];
        float silu = g / (1.0f + expf(-g));
        y_f16[r] = vo_f32_to_f16(silu * up[r]);
    }
    free(up);
    free(gate);
}

VO_API void vo_swiglu_int4(const uint16_t* x_f16, const uint8_t* up_page, const uint8_t* gate_page,
                           uint16_t* y_f16, int H, int M, int group_size, int scale_format) {
    float* x = (float*)malloc((size_t)H * sizeof(float));
    for (int i = 0; i < H; i++) x[i] = vo_f16_to_f32(x_f16[i]);
    vo_swiglu_int4_f32in(x, up_page, gate_page, y_f16, H, M, group_size, scale_format);
    free(x);
}

/* vib3_silu_mul (kernels.cu:772-785): f16 operands, f32 silu(a) * b, f16 result.  The first
 * operand receives the SiLU (the Rust caller passes the gate projection there,
 * kernels.rs:529-537). */
VO_API void vo_silu_mul(const uint16_t* a_f16, const uint16_t* b_f16, uint16_t* y_f16, int dim) {
    for (int i = 0; i < dim; i++) {
        float a = vo_f16_to_f32(a_f16[i]);
        float b = vo_f16_to_f32(b_f16[i]);
        float silu = a / (1.0f + expf(-a));
        y_f16[i] = vo_f32_to_f16(silu * b);
    }
}

/* weighted_accumulate (kernels.rs:1989-1994): f16 += w * f16 through f32, rounded each time. */
VO_API void vo_weighted_accumulate(uint16_t* out_f16, const uint16_t* y_f16, float w, int dim) {
    for (int i = 0; i < dim; i++) {
        float v = vo_f16_to_f32(out_f16[i]) + w * vo_f16_to_f32(y_f16[i]);
        out_f16[i] = vo_f32_to_f16(v);
    }
}

/* weighted_accumulate_f32 (kernels.rs:2028-2035). */
VO_API void vo_weighted_accumulate_f32(float* out, const uint16_t* y_f16, float w, int dim) {
    for (int i = 0; i < dim; i++) out[i] += w * vo_f16_to_f32(y_f16[i]);
}

/* weighted_accumulate_f32_f32 (kernels.rs:2068-2075). */
VO_API void vo_weighted_accumulate_f32_f32(float* out, const float* y, float w, int dim) {
    for (int i = 0; i < dim; i++) out[i] += w * y[i];
}

/* vib3_residual_add_f32_f32_kernel (kernels.cu:817-826). */
VO_API void vo_residual_add_f32_f32(float* acc, const float* layer_out, int dim) {
    for (int i = 0; i < dim; i++) acc[i] += layer_out[i];
}

/* ── Router ────────────────────────────────────────────────────────────────────────────── */

/* Raw router logits.  w_is_f32 = 0: W is f16 [E,H] (the reference's only format,
 * kernels.rs:2337-2340); 1: W is f32 (the benchmark configs ask for fp32 router weights).
 * order 0: one sequential f32 chain per expert, multiply then add (kernels.rs:2344-2362).
 * order 1: the reference CUDA kernel's order (kernels.cu:665-707): 128 interleaved chains
 *          (chain t takes d = t, t+128, ...) accumulated with fused multiply-add (nvcc
 *          contracts `acc += a*b`), a shfl_down tree inside each of the 4 warps, then
 *          (s0 + s2) + (s1 + s3) across warps. */
VO_API void vo_router_logits(const float* x, const void* W, int w_is_f32, int E, int H, int order,
                             float* logits) {
#pragma omp parallel for schedule(static) if (E >= 64)
    for (int e = 0; e < E; e++) {
        const uint16_t* wh = (const uint16_t*)W + (size_t)e * H;
        const float* wf = (const float*)W + (size_t)e * H;
        if (order == 0) {
            float acc = 0.0f;
            for (int d = 0; d < H; d++) {
                float w = w_is_f32 ? wf[d] : vo_f16_to_f32(wh[d]);
                acc += x[d] * w;
            }
            logits[e] = acc;
        } else {
            float p[128];
            for (int t = 0; t < 128; t++) {
                float acc = 0.0f;
                for (int d = t; d < H; d += 128) {
                    float w = w_is_f32 ? wf[d] : vo_f16_to_f32(wh[d]);
                    acc = fmaf(x[d], w, acc);
                }
                p[t] = acc;
            }
            float s[4];
            for (int wp = 0; wp < 4; wp++) {
                float v[32];
                for (int l = 0; l < 32; l++) v[l] = p[wp * 32 + l];
                for (int off = 16; off > 0; off >>= 1)
                    for (int l = 0; l < off; l++) v[l] = v[l] + v[l + off];
                s[wp] = v[0];
            }
            /* warp 0 holds s0..s3 in lanes 0..3 and zeros above (kernels.cu:699-702):
             * offsets 16, 8, 4 add zeros, offset 2 gives s0+s2 and s1+s3, offset 1 their sum. */
            float a = ((s[0] + 0.0f) + 0.0f) + 0.0f;
            float b = ((s[1] + 0.0f) + 0.0f) + 0.0f;
            float c = ((s[2] + 0.0f) + 0.0f) + 0.0f;
            float d2 = ((s[3] + 0.0f) + 0.0f) + 0.0f;
            logits[e] = (a + c) + (b + d2);
        }
    }
}

typedef struct { int idx; float key; } vo_pair;

/* Stable descending order on the key: equal keys keep ascending index, as Rust's stable
 * sort_by with partial_cmp(..).unwrap_or(Equal) does (kernels.rs:2371, :2414). */
static int pair_cmp(const void* pa, const void* pb) {
    const vo_pair* a = (const vo_pair*)pa;
    const vo_pair* b = (const vo_pair*)pb;
    if (a->key > b->key) return -1;
    if (a->key < b->key) return 1;
    return a->idx - b->idx;
}

/* Scoring and top-k of run_router_with_scoring_and_bias (kernels.rs:2364-2437) applied to
 * given logits.  mode 0 = Softmax: top-k on raw logits, softmax over the selected k only.
 * mode 1 = Sigmoid{scaling_factor, normalize}: sigmoid of all, optional bias added for
 * selection only, weights from the unbiased sigmoid, divided by their sum when normalize and
 * sum > 1e-20, then multiplied by scaling_factor.  Returns the number of pairs written. */
VO_API int vo_router_select(const float* logits, int E, int top_k, int mode, float scaling_factor,
                            int normalize, const float* bias, uint16_t* out_ids, float* out_w) {
    if (top_k > E) top_k = E; /* Vec::truncate semantics */
    vo_pair* idx = (vo_pair*)malloc((size_t)E * sizeof(vo_pair));
    float* sig = (float*)malloc((size_t)E * sizeof(float));
    if (mode == 0) {
        for (int e = 0; e < E; e++) { idx[e].idx = e; idx[e].key = logits[e]; }
        qsort(idx, (size_t)E, sizeof(vo_pair), pair_cmp);
        float mx = -INFINITY;
        for (int i = 0; i < top_k; i++) mx = fmaxf(mx, idx[i].key);
        float sum = 0.0f;
        for (int i = 0; i < top_k; i++) sum += expf(idx[i].key - mx);
        for (int i = 0; i < top_k; i++) {
            out_ids[i] = (uint16_t)idx[i].idx;
            out_w[i] = expf(idx[i].key - mx) / sum;
        }
    } else {
        for (int e = 0; e < E; e++) {
            sig[e] = 1.0f / (1.0f + expf(-logits[e]));
            idx[e].idx = e;
            idx[e].key = bias ? sig[e] + bias[e] : sig[e];
        }
        qsort(idx, (size_t)E, sizeof(vo_pair), pair_cmp);
        float total = 0.0f;
        for (int i = 0; i < top_k; i++) {
            out_ids[i] = (uint16_t)idx[i].idx;
            out_w[i] = sig[idx[i].idx];
            total += out_w[i];
        }
        if (normalize && total > 1e-20f)
            for (int i = 0; i < top_k; i++) out_w[i] /= total;
        for (int i = 0; i < top_k; i++) out_w[i] *= scaling_factor;
    }
    free(idx);
    free(sig);
    return top_k;
}

/* run_router_with_scoring_and_bias end to end (kernels.rs:2307-2440). */
VO_API int vo_router(const float* x, const void* W, int w_is_f32, int E, int H, int top_k, int mode,
                     float scaling_factor, int normalize, const float* bias, int order,
                     uint16_t* out_ids, float* out_w, float* logits_out) {
    float* logits = logits_out ? logits_out : (float*)malloc((size_t)E * sizeof(float));
    vo_router_logits(x, W, w_is_f32, E, H, order, logits);
    int n = vo_router_select(logits, E, top_k, mode, scaling_factor, normalize, bias, out_ids, out_w);
    if (!logits_out) free(logits);
    return n;
}

/* ── RMSNorm (the step in front of the path; kernels.rs:2591-2603) ─────────────────────── */

VO_API void vo_rms_norm_f32(const float* x, const float* w_or_null, float* y, int H, float eps) {
    float sum_sq = 0.0f;
    for (int i = 0; i < H; i++) sum_sq += x[i] * x[i];
    float rms = sqrtf(sum_sq / (float)H + eps);
    float inv = 1.0f / rms;
    for (int i = 0; i < H; i++) y[i] = w_or_null ? x[i] * inv * w_or_null[i] : x[i] * inv;
}

/* ── Quantiser (kernels.rs:3778-3831) and its inverse (kernels.rs:3866-3927) ───────────── */

/* Group absmax / 7, q = clamp(round(w / scale) + 8, 0, 15) (Rust f32::round = half away from
 * zero = roundf), low nibble = even column.  The reference writes the scale as BF16
 * (kernels.rs:3803); scale_format 1 writes FP16 instead, as its CUDA kernels expect. */
VO_API void vo_quantize_int4(const float* w, int rows, int cols, int group_size, int scale_format,
                             uint8_t* out) {
    int packed_k = (cols + 1) / 2;
    int num_groups = (cols + group_size - 1) / group_size;
    size_t int4_bytes = (size_t)rows * packed_k;
    memset(out, 0, int4_bytes + (size_t)rows * num_groups * 2);
    uint8_t* scales = out + int4_bytes;
    for (int r = 0; r < rows; r++) {
        const float* row = w + (size_t)r * cols;
        for (int g = 0; g < num_groups; g++) {
            int c0 = g * group_size;
            int c1 = c0 + group_size < cols ? c0 + group_size : cols;
            float max_abs = 0.0f;
            for (int c = c0; c < c1; c++) max_abs = fmaxf(max_abs, fabsf(row[c]));
            float scale = max_abs > 0.0f ? max_abs / 7.0f : 1.0f;
            uint16_t sb = scale_format == 0 ? vo_f32_to_bf16(scale) : vo_f32_to_f16(scale);
            size_t so = ((size_t)r * num_groups + g) * 2;
            scales[so] = (uint8_t)(sb & 0xFF);
            scales[so + 1] = (uint8_t)(sb >> 8);
            for (int c = c0; c < c1; c++) {
                int q = (int)roundf(row[c] / scale) + 8;
                if (q < 0) q = 0;
                if (q > 15) q = 15;
                size_t bo = (size_t)r * packed_k + c / 2;
                if (c % 2 == 0) out[bo] |= (uint8_t)(q & 0x0F);
                else out[bo] |= (uint8_t)((q & 0x0F) << 4);
            }
        }
    }
}

VO_API void vo_dequantize_int4(const uint8_t* data, int rows, int cols, int group_size,
                               int scale_format, float* out) {
    int packed_k = (cols + 1) / 2;
    int num_groups = (cols + group_size - 1) / group_size;
    const uint8_t* scales = data + (size_t)rows * packed_k;
    for (int r = 0; r < rows; r++) {
        for (int b = 0; b < packed_k; b++) {
            uint8_t p = data[(size_t)r * packed_k + b];
            int c0 = 2 * b, c1 = c0 + 1;
            size_t s0 = ((size_t)r * num_groups + c0 / group_size) * 2;
            float sc0 = decode_scale((uint16_t)(scales[s0] | (scales[s0 + 1] << 8)), scale_format);
            out[(size_t)r * cols + c0] = ((float)(p & 0x0F) - 8.0f) * sc0;
            if (c1 < cols) {
                size_t s1 = ((size_t)r * num_groups + c1 / group_size) * 2;
                float sc1 = decode_scale((uint16_t)(scales[s1] | (scales[s1 + 1] << 8)), scale_format);
                out[(size_t)r * cols + c1] = ((float)((p >> 4) & 0x0F) - 8.0f) * sc1;
            }
        }
    }
}

/* ── Page geometry (convert.rs:1807-1812, :1854-1860) and page key (types.rs:259-264) ──── */

VO_API void vo_int4_page_geometry(int rows, int cols, int group_size, int page_size, int* bytes_per_row,
                                  int* rows_per_page, int* num_pages) {
    int packed_k = (cols + 1) / 2;
    int num_groups = (cols + group_size - 1) / group_size;
    int bpr = packed_k + num_groups * 2;
    int rpp = bpr > 0 ? page_size / bpr : rows;
    if (rpp < 1) rpp = 1;
    *bytes_per_row = bpr;
    *rows_per_page = rpp;
    *num_pages = (rows + rpp - 1) / rpp;
}

VO_API uint64_t vo_page_key(uint16_t layer, uint16_t expert, uint16_t segment, uint16_t page_idx) {
    return ((uint64_t)layer << 48) | ((uint64_t)expert << 32) | ((uint64_t)segment << 16) |
           (uint64_t)page_idx;
}

/* Cut one quantised matrix ([rows*packed_k codes][rows*groups scales]) into page images, each
 * [row_count*packed_k codes][row_count*groups scales] (convert.rs:1862-1888).  Writes the
 * images back to back into `out` and the row_start/row_count of each into the two arrays. */
VO_API void vo_split_int4_pages(const uint8_t* matrix, int rows, int cols, int group_size, int page_size,
                                uint8_t* out, int* row_start, int* row_count) {
    int bpr, rpp, np;
    vo_int4_page_geometry(rows, cols, group_size, page_size, &bpr, &rpp, &np);
    int packed_k = (cols + 1) / 2;
    int num_groups = (cols + group_size - 1) / group_size;
    const uint8_t* scales = matrix + (size_t)rows * packed_k;
    size_t o = 0;
    for (int p = 0; p < np; p++) {
        int r0 = p * rpp;
        int rc = rows - r0 < rpp ? rows - r0 : rpp;
        memcpy(out + o, matrix + (size_t)r0 * packed_k, (size_t)rc * packed_k);
        o += (size_t)rc * packed_k;
        memcpy(out + o, scales + (size_t)r0 * num_groups * 2, (size_t)rc * num_groups * 2);
        o += (size_t)rc * num_groups * 2;
        row_start[p] = r0;
        row_count[p] = rc;
    }
}
