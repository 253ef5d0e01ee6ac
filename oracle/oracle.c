/*
 * CPU oracle for the INT4 mixture-of-experts hot path (test infrastructure; see oracle.h).
 *
 * Every function restates, in plain C, the arithmetic of a reference source cited beside it by
 * its path inside the reference project.  fp32 arithmetic is written out operation by operation
 * and the file is compiled with -ffp-contract=off, so a fused multiply-add happens only where
 * fmaf() is written.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define GROUP 64

/* ---- bf16 -------------------------------------------------------------------------------- */

/* Sources/ANEFieldfareHotpath/Infrastructure/ModelIO/Quantization.swift:9-16 — round half to
 * even on the 16 discarded bits, no NaN/Inf special case. */
uint16_t ffo_bf16_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    uint32_t keep_lsb = (u >> 16) & 1u;
    u += 0x7FFFu + keep_lsb;
    return (uint16_t)(u >> 16);
}

/* Quantization.swift:18-20 */
float ffo_bf16_to_float(uint16_t bits) {
    uint32_t u = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void ffo_bf16_bits_n(const float *x, uint16_t *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = ffo_bf16_bits(x[i]);
}

void ffo_bf16_to_float_n(const uint16_t *x, float *out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = ffo_bf16_to_float(x[i]);
}

static inline float bf16_round(float x) { return ffo_bf16_to_float(ffo_bf16_bits(x)); }

/* ---- PRNG -------------------------------------------------------------------------------- */

/* Tests/Support/Validation/PRNG/SplitMix64.swift:9-15 */
uint64_t ffo_splitmix64_next(uint64_t *state) {
    uint64_t z = (*state += 0x9E3779B97F4A7C15ull);
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* SplitMix64.swift:18-21 — 24 mantissa bits, [lo, hi). */
float ffo_splitmix64_uniform(uint64_t *state, float lo, float hi) {
    float u = (float)(ffo_splitmix64_next(state) >> 40) / 16777216.0f;
    float span = hi - lo;
    float scaled = span * u;
    return lo + scaled;
}

/* Tests/Support/Validation/PRNG/SeedTree.swift:12-19 — FNV-1a of the label, XOR the root; the
 * result seeds a SplitMix64 stream. */
uint64_t ffo_seedtree_key(uint64_t root, const char *label) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (const unsigned char *p = (const unsigned char *)label; *p; ++p) {
        h ^= (uint64_t)*p;
        h *= 0x100000001B3ull;
    }
    return root ^ h;
}

void ffo_splitmix64_fill(uint64_t seed, uint64_t *out, int64_t n) {
    uint64_t s = seed;
    for (int64_t i = 0; i < n; ++i) out[i] = ffo_splitmix64_next(&s);
}

/* ---- affine INT4 ------------------------------------------------------------------------- */

static inline uint32_t nibble_at(const uint8_t *packed, int64_t index) {
    uint8_t byte = packed[index >> 1];
    return (index & 1) ? (uint32_t)(byte >> 4) : (uint32_t)(byte & 0x0F);
}

/* Tests/Support/Validation/Reference/Quant/AffineQuantization.swift:24-76 — fixture quantizer:
 * per group of 64, scale=(max-min)/15, bias=min, both through bf16 before the codes are
 * chosen; low nibble holds the even index. */
void ffo_quantize_int4_row(const float *row, int32_t n, uint8_t *packed, uint16_t *scales,
                           uint16_t *biases) {
    memset(packed, 0, (size_t)n / 2);
    for (int32_t g = 0; g < n / GROUP; ++g) {
        const float *v = row + (int64_t)g * GROUP;
        float lo = INFINITY, hi = -INFINITY;
        for (int k = 0; k < GROUP; ++k) {
            if (v[k] < lo) lo = v[k];
            if (v[k] > hi) hi = v[k];
        }
        float scale_f = 1.0f, bias_f = lo;
        if (hi != lo) scale_f = (hi - lo) / 15.0f;
        scales[g] = ffo_bf16_bits(scale_f);
        biases[g] = ffo_bf16_bits(bias_f);
        float scale = ffo_bf16_to_float(scales[g]);
        float bias = ffo_bf16_to_float(biases[g]);
        float inv = scale == 0.0f ? 0.0f : 1.0f / scale;
        for (int k = 0; k < GROUP; ++k) {
            /* Swift's .rounded() is round-half-away-from-zero == roundf */
            float r = roundf((v[k] - bias) * inv);
            int q = (int)r;
            if (q < 0) q = 0;
            if (q > 15) q = 15;
            int64_t idx = (int64_t)g * GROUP + k;
            packed[idx >> 1] |= (uint8_t)(q << ((idx & 1) * 4));
        }
    }
}

/* AffineQuantization.swift:78-93 — w = float(q) * scale + bias (two fp32 operations; the
 * product of a 4-bit code and an 8-bit-mantissa scale is exact, so a fused form gives the same
 * bits). */
void ffo_dequant_int4(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t rows,
                      int32_t cols, float *out) {
    const int32_t groups = cols / GROUP;
#pragma omp parallel for schedule(static) if (!omp_in_parallel() && (int64_t)rows * cols > 1 << 16)
    for (int32_t r = 0; r < rows; ++r) {
        const uint8_t *wr = w + (int64_t)r * (cols / 2);
        for (int32_t g = 0; g < groups; ++g) {
            float scale = ffo_bf16_to_float(s[(int64_t)r * groups + g]);
            float bias = ffo_bf16_to_float(b[(int64_t)r * groups + g]);
            for (int k = 0; k < GROUP; ++k) {
                int64_t c = (int64_t)g * GROUP + k;
                float prod = (float)nibble_at(wr, c) * scale;
                out[(int64_t)r * cols + c] = prod + bias;
            }
        }
    }
}

/* The prefill tensor path multiplies weights rounded to 16 bits
 * (Sources/ANEFieldfareHotpath/Metal/Prefill/prefill.metal:581-590 rounds fma(q,s,b) to half;
 * Metal/TensorCore/tensorops.metal:198 has the bf16 form).  Here: the exact real value
 * q*scale+bias rounded ONCE to bf16 (round-half-even), which is what one bf16 fused
 * multiply-add produces.  q*scale+bias is exact in double for bf16 operands. */
void ffo_dequant_int4_bf16(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t rows,
                           int32_t cols, uint16_t *out) {
    const int32_t groups = cols / GROUP;
    for (int32_t r = 0; r < rows; ++r) {
        const uint8_t *wr = w + (int64_t)r * (cols / 2);
        for (int32_t g = 0; g < groups; ++g) {
            double scale = (double)ffo_bf16_to_float(s[(int64_t)r * groups + g]);
            double bias = (double)ffo_bf16_to_float(b[(int64_t)r * groups + g]);
            for (int k = 0; k < GROUP; ++k) {
                int64_t c = (int64_t)g * GROUP + k;
                double exact = (double)nibble_at(wr, c) * scale + bias;
                /* double -> bf16 with a single rounding: round to odd into fp32 first */
                float f = (float)exact;
                if ((double)f != exact) {
                    uint32_t u;
                    memcpy(&u, &f, 4);
                    /* make the fp32 value the truncation toward zero, then set the sticky bit */
                    int away = fabs((double)f) > fabs(exact);
                    if (away) u -= 1;
                    u |= 1u;
                    memcpy(&f, &u, 4);
                }
                out[(int64_t)r * cols + c] = ffo_bf16_bits(f);
            }
        }
    }
}

/* Tests/ANEFieldfareUpstreamTests/Kernels/Prefill/PrefillGroupedRoutedMoETests.swift:153-178 —
 * one row, scalar, columns ascending: acc += (q*scale + bias) * x[col]. */
float ffo_int4_dot(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t row,
                   int32_t cols, const float *x) {
    const int32_t groups = cols / GROUP;
    const uint8_t *wr = w + (int64_t)row * (cols / 2);
    float acc = 0.0f;
    for (int32_t g = 0; g < groups; ++g) {
        float scale = ffo_bf16_to_float(s[(int64_t)row * groups + g]);
        float bias = ffo_bf16_to_float(b[(int64_t)row * groups + g]);
        for (int k = 0; k < GROUP; ++k) {
            int32_t c = g * GROUP + k;
            float prod = (float)nibble_at(wr, c) * scale;
            float wv = prod + bias;
            float term = wv * x[c];
            acc = acc + term;
        }
    }
    return acc;
}

/* Y[r][o] = ffo_int4_dot(row o, x row r) for every r, bit for bit: the weight row is expanded
 * once and the same column-ascending chain runs for all input rows side by side (the layout the
 * reference's Tests/Support/Validation/Reference/Quant/DequantInt4Gemv.swift:9-38 uses:
 * dequantize the row, then dot).  xt is x transposed to [cols][rpad]. */
/* bf16 nearest to the exact real value q*scale + bias (one rounding, as one bf16 fused multiply-add
 * gives; see ffo_dequant_int4_bf16). */
static inline float weight_bf16(uint32_t q, float scale, float bias) {
    double exact = (double)q * (double)scale + (double)bias;
    float f = (float)exact;
    if ((double)f != exact) {
        uint32_t u;
        memcpy(&u, &f, 4);
        if (fabs((double)f) > fabs(exact)) u -= 1;
        u |= 1u;
        memcpy(&f, &u, 4);
    }
    return bf16_round(f);
}

/* weights_bf16: multiply the weights rounded once to bf16, the operand of the tensor-core prefill
 * path (Sources/ANEFieldfareHotpath/Metal/Prefill/prefill.metal:581-590 rounds to half there). */
static void gemv_rows_t(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t rows,
                        int32_t cols, const float *xt, int32_t n, int32_t rpad, float *y,
                        int32_t y_stride, int32_t weights_bf16) {
    const int32_t groups = cols / GROUP;
#pragma omp parallel if (!omp_in_parallel() && (int64_t)rows * cols * n > 1 << 18)
    {
        float *wrow = (float *)malloc(sizeof(float) * (size_t)cols);
        float *acc = (float *)malloc(sizeof(float) * (size_t)rpad);
#pragma omp for schedule(static)
        for (int32_t o = 0; o < rows; ++o) {
            const uint8_t *wr = w + (int64_t)o * (cols / 2);
            for (int32_t g = 0; g < groups; ++g) {
                float scale = ffo_bf16_to_float(s[(int64_t)o * groups + g]);
                float bias = ffo_bf16_to_float(b[(int64_t)o * groups + g]);
                for (int k = 0; k < GROUP; ++k) {
                    int32_t c = g * GROUP + k;
                    if (weights_bf16) {
                        wrow[c] = weight_bf16(nibble_at(wr, c), scale, bias);
                    } else {
                        float prod = (float)nibble_at(wr, c) * scale;
                        wrow[c] = prod + bias;
                    }
                }
            }
            for (int32_t r = 0; r < rpad; ++r) acc[r] = 0.0f;
            for (int32_t c = 0; c < cols; ++c) {
                const float wv = wrow[c];
                const float *xc = xt + (int64_t)c * rpad;
                for (int32_t r = 0; r < rpad; ++r) {
                    float term = wv * xc[r];
                    acc[r] = acc[r] + term;
                }
            }
            for (int32_t r = 0; r < n; ++r) y[(int64_t)r * y_stride + o] = acc[r];
        }
        free(wrow);
        free(acc);
    }
}

static float *transpose_pad(const float *x, int32_t n, int32_t x_stride, int32_t cols,
                            int32_t *rpad_out) {
    int32_t rpad = (n + 7) & ~7;
    float *xt = (float *)calloc((size_t)cols * rpad, sizeof(float));
    for (int32_t r = 0; r < n; ++r)
        for (int32_t c = 0; c < cols; ++c) xt[(int64_t)c * rpad + r] = x[(int64_t)r * x_stride + c];
    *rpad_out = rpad;
    return xt;
}

void ffo_int4_gemv_rows(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t rows,
                        int32_t cols, const float *x, int32_t x_rows, int32_t x_stride, float *y,
                        int32_t y_stride) {
    int32_t rpad;
    float *xt = transpose_pad(x, x_rows, x_stride, cols, &rpad);
    gemv_rows_t(w, s, b, rows, cols, xt, x_rows, rpad, y, y_stride, 0);
    free(xt);
}

/* Tests/Support/Validation/Reference/MoE/Moe.swift:13-24 — tanh-form GELU, no clamp (the Metal
 * kernels clamp the tanh argument to +-20, which saturates identically in fp32). */
float ffo_gelu_tanh(float x) {
    float cubic = 0.044715f * x;
    cubic = cubic * x;
    cubic = cubic * x;
    float inner = 0.7978845608028654f * (x + cubic);
    float half_x = 0.5f * x;
    return half_x * (1.0f + tanhf(inner));
}

/* One GeGLU expert for T input rows: out = down(act), act = gelu(gate.x) * (up.x).
 * Moe.swift:26-50 gives the composition; the 16-bit rounding of act follows
 * PrefillGroupedRoutedMoETests.swift:139-143 (bf16 here, fp16 there).  round_gate_up rounds the
 * two projections before the activation, as the shared FFN does
 * (Sources/ANEFieldfareHotpath/Metal/MoE/moe.metal:548-570).  out is fp32 [T][out_stride]. */
static void expert_ffn_w(const uint8_t *blob, const ffo_offsets *off, int32_t D, int32_t F,
                         const uint16_t *x, int32_t T, int32_t x_stride, int32_t round_gate_up,
                         int32_t round_act, int32_t weights_bf16, float *out, int32_t out_stride) {
    if (T <= 0) return;
    float *xf = (float *)malloc(sizeof(float) * (size_t)T * D);
    for (int32_t t = 0; t < T; ++t)
        for (int32_t d = 0; d < D; ++d)
            xf[(int64_t)t * D + d] = ffo_bf16_to_float(x[(int64_t)t * x_stride + d]);
    int32_t rpad;
    float *xt = transpose_pad(xf, T, D, D, &rpad);
    float *g = (float *)malloc(sizeof(float) * (size_t)T * F);
    float *u = (float *)malloc(sizeof(float) * (size_t)T * F);
    gemv_rows_t(blob + off->gate_w, (const uint16_t *)(blob + off->gate_s),
                (const uint16_t *)(blob + off->gate_b), F, D, xt, T, rpad, g, F, weights_bf16);
    gemv_rows_t(blob + off->up_w, (const uint16_t *)(blob + off->up_s),
                (const uint16_t *)(blob + off->up_b), F, D, xt, T, rpad, u, F, weights_bf16);
    free(xt);
    for (int64_t i = 0; i < (int64_t)T * F; ++i) {
        float gv = g[i], uv = u[i];
        if (round_gate_up) {
            gv = bf16_round(gv);
            uv = bf16_round(uv);
        }
        float a = ffo_gelu_tanh(gv) * uv;
        g[i] = round_act ? bf16_round(a) : a;
    }
    float *at = transpose_pad(g, T, F, F, &rpad);
    gemv_rows_t(blob + off->down_w, (const uint16_t *)(blob + off->down_s),
                (const uint16_t *)(blob + off->down_b), D, F, at, T, rpad, out, out_stride, weights_bf16);
    free(at);
    free(g);
    free(u);
    free(xf);
}

void ffo_expert_ffn(const uint8_t *blob, const ffo_offsets *off, int32_t D, int32_t F,
                    const uint16_t *x, int32_t T, int32_t x_stride, int32_t round_gate_up,
                    int32_t round_act, float *out, int32_t out_stride) {
    expert_ffn_w(blob, off, D, F, x, T, x_stride, round_gate_up, round_act, 0, out, out_stride);
}

/* ---- router ------------------------------------------------------------------------------ */

/* Router logits with a DEFINED reduction order, so that the top-k indices can be compared for
 * equality with the CUDA kernel.  Structure follows the reference's decode router
 * (Sources/ANEFieldfareHotpath/Metal/MoE/moe.metal:65-103: one 32-lane group per expert row,
 * lane-strided fused multiply-adds, then a lane sum) with bf16 weights in place of INT8:
 *   lane l chains fmaf over elements [256*i + 8*l, 256*i + 8*l + 8) for i = 0,1,.. in
 *   increasing index; the 32 lane sums are added by an xor butterfly with offsets 16,8,4,2,1;
 *   logit_bias[e] is added last.
 * x' = float(x) * float(router_scale) when a scale is given (both bf16, product exact). */
void ffo_router_logits(const ffo_layer *L, const uint16_t *x, float *logits) {
    const int32_t D = L->D;
    float *xs = (float *)malloc(sizeof(float) * (size_t)D);
    for (int32_t d = 0; d < D; ++d) {
        float v = ffo_bf16_to_float(x[d]);
        if (L->router_scale) v = v * ffo_bf16_to_float(L->router_scale[d]);
        xs[d] = v;
    }
    for (int32_t e = 0; e < L->E; ++e) {
        const uint16_t *wr = L->router_w + (int64_t)e * D;
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int32_t base = 8 * l; base < D; base += 256)
                for (int j = 0; j < 8 && base + j < D; ++j)
                    acc = fmaf(ffo_bf16_to_float(wr[base + j]), xs[base + j], acc);
            lane[l] = acc;
        }
        for (int offset = 16; offset >= 1; offset >>= 1) {
            float next[32];
            for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ offset];
            memcpy(lane, next, sizeof(lane));
        }
        float v = lane[0];
        if (L->logit_bias) v = v + L->logit_bias[e];
        logits[e] = v;
    }
    free(xs);
}

/* The INT8 affine router of the shipped checkpoints, in the order of the reference's kernel
 * (Sources/ANEFieldfareHotpath/Metal/MoE/moe.metal:65-103), made definite where the kernel leaves
 * it to the compiler: lane l takes elements 64 g + 2 l and 64 g + 2 l + 1 of every group g in
 * increasing g, x' = float(x) * float(effective_scale) when a scale is given,
 *   acc = fma(s_g, fma(q1, x1', q0 * x0'), acc);  acc = fma(b_g, x0' + x1', acc);
 * the 32 lane sums are added by an xor butterfly (16, 8, 4, 2, 1); logit_bias[e] is added last.
 * codes uint8 [E][D]; scales, biases bf16 [E][D/64]. */
void ffo_router_logits_int8(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases,
                            const uint16_t *effective_scale, const float *logit_bias, int32_t E,
                            int32_t D, const uint16_t *x, float *logits) {
    const int32_t groups = D / 64;
    float *xs = (float *)malloc(sizeof(float) * (size_t)D);
    for (int32_t d = 0; d < D; ++d) {
        float v = ffo_bf16_to_float(x[d]);
        if (effective_scale) v = v * ffo_bf16_to_float(effective_scale[d]);
        xs[d] = v;
    }
    for (int32_t e = 0; e < E; ++e) {
        const uint8_t *wr = codes + (int64_t)e * D;
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int32_t g = 0; g < groups; ++g) {
                const int32_t idx = g * 64 + 2 * l;
                const float s = ffo_bf16_to_float(scales[(int64_t)e * groups + g]);
                const float b = ffo_bf16_to_float(biases[(int64_t)e * groups + g]);
                const float q0 = (float)wr[idx], q1 = (float)wr[idx + 1];
                const float x0 = xs[idx], x1 = xs[idx + 1];
                acc = fmaf(s, fmaf(q1, x1, q0 * x0), acc);
                acc = fmaf(b, x0 + x1, acc);
            }
            lane[l] = acc;
        }
        for (int offset = 16; offset >= 1; offset >>= 1) {
            float next[32];
            for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ offset];
            memcpy(lane, next, sizeof(lane));
        }
        float v = lane[0];
        if (logit_bias) v = v + logit_bias[e];
        logits[e] = v;
    }
    free(xs);
}

void ffo_router_topk_int8(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases,
                          const uint16_t *effective_scale, const float *logit_bias,
                          const uint16_t *gain, int32_t E, int32_t D, int32_t K, const uint16_t *x,
                          int32_t T, int32_t x_stride, uint32_t *ids, uint16_t *weights,
                          float *logits_out) {
#pragma omp parallel for schedule(static) if (!omp_in_parallel() && T > 8)
    for (int32_t t = 0; t < T; ++t) {
        float *logits = (float *)malloc(sizeof(float) * (size_t)E);
        ffo_router_logits_int8(codes, scales, biases, effective_scale, logit_bias, E, D,
                               x + (int64_t)t * x_stride, logits);
        ffo_topk(logits, E, gain, K, ids + (int64_t)t * K, weights + (int64_t)t * K, NULL);
        if (logits_out) memcpy(logits_out + (int64_t)t * E, logits, sizeof(float) * (size_t)E);
        free(logits);
    }
}

/* Selection rule and softmax of Metal/MoE/moe.metal:269-319 (serial top-8) and its CPU statement
 * Tests/ANEFieldfareUpstreamTests/Kernels/MoE/RouterTopKTests.swift:55-71: highest score first,
 * equal scores -> lower expert id; w_i = exp(l_i - l_0) / sum * gain[e_i], stored in 16 bits
 * (bf16 here).  Scores of -inf or NaN are never taken; unfilled slots report expert 0. */
void ffo_topk(const float *logits, int32_t E, const uint16_t *gain, int32_t K, uint32_t *ids,
              uint16_t *weights, float *weights_f32) {
    float score[64];
    uint8_t *taken = (uint8_t *)calloc((size_t)E, 1);
    for (int32_t r = 0; r < K; ++r) {
        int32_t best = -1;
        for (int32_t e = 0; e < E; ++e) {
            if (taken[e] || !(logits[e] > -INFINITY)) continue;
            if (best < 0 || logits[e] > logits[best]) best = e;
        }
        if (best >= 0) {
            taken[best] = 1;
            ids[r] = (uint32_t)best;
            score[r] = logits[best];
        } else {
            ids[r] = 0;
            score[r] = -INFINITY;
        }
    }
    free(taken);
    float ex[64], sum = 0.0f;
    for (int32_t r = 0; r < K; ++r) {
        ex[r] = expf(score[r] - score[0]);
        sum = sum + ex[r];
    }
    for (int32_t r = 0; r < K; ++r) {
        float wv = ex[r] / sum;
        if (gain) wv = wv * ffo_bf16_to_float(gain[ids[r]]);
        if (weights_f32) weights_f32[r] = wv;
        if (weights) weights[r] = ffo_bf16_bits(wv);
    }
}

void ffo_router_topk(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t x_stride,
                     uint32_t *ids, uint16_t *weights, float *logits_out) {
#pragma omp parallel for schedule(static) if (!omp_in_parallel() && T > 8)
    for (int32_t t = 0; t < T; ++t) {
        float *logits = (float *)malloc(sizeof(float) * (size_t)L->E);
        ffo_router_logits(L, x + (int64_t)t * x_stride, logits);
        ffo_topk(logits, L->E, L->gain, L->K, ids + (int64_t)t * L->K, weights + (int64_t)t * L->K,
                 NULL);
        if (logits_out) memcpy(logits_out + (int64_t)t * L->E, logits, sizeof(float) * (size_t)L->E);
        free(logits);
    }
}

/* ---- host permute ------------------------------------------------------------------------ */

/* Sources/ANEFieldfareHotpath/Kernels/Prefill/MoE/PrefillRouter.swift:75-95 — token-major,
 * rank-minor list of (token, expert, rank, 16-bit weight). */
int64_t ffo_make_pairs(const uint32_t *ids, const uint16_t *weights, int32_t T, int32_t K,
                       ffo_pair *pairs) {
    int64_t n = 0;
    for (int32_t t = 0; t < T; ++t)
        for (int32_t r = 0; r < K; ++r) {
            int64_t i = (int64_t)t * K + r;
            pairs[n].token = (uint32_t)t;
            pairs[n].expert = ids[i];
            pairs[n].rank = (uint32_t)r;
            pairs[n].weight_bits = weights ? (uint32_t)weights[i] : 0u;
            ++n;
        }
    return n;
}

static const uint64_t *g_sort_keys;
#pragma omp threadprivate(g_sort_keys)

static int pair_less(const void *pa, const void *pb) {
    const ffo_pair *a = (const ffo_pair *)pa, *b = (const ffo_pair *)pb;
    if (g_sort_keys) {
        uint64_t ka = g_sort_keys[a->expert], kb = g_sort_keys[b->expert];
        if (ka != kb) return ka < kb ? -1 : 1;
    }
    if (a->expert != b->expert) return a->expert < b->expert ? -1 : 1;
    if (a->token != b->token) return a->token < b->token ? -1 : 1;
    if (a->rank != b->rank) return a->rank < b->rank ? -1 : 1;
    return 0;
}

/* Sources/ANEFieldfareHotpath/Kernels/Prefill/MoE/PrefillMoEGrouping.swift:49-110 — sort by
 * (optional per-expert key, expert, token, rank); one group per run of equal experts; tiles of up
 * to tile_experts consecutive groups.  Returns 0, or -1 with *bad_expert set when a pair names an
 * expert >= E (the reference throws expertOutOfRange). */
int32_t ffo_group_pairs(const ffo_pair *pairs, int64_t n_pairs, int32_t T, int32_t K, int32_t E,
                        int32_t tile_experts, const uint64_t *sort_keys, ffo_pair *sorted,
                        ffo_group *groups, int32_t *n_groups, ffo_tile *tiles, int32_t *n_tiles,
                        uint32_t *bad_expert) {
    (void)T;
    (void)K;
    for (int64_t i = 0; i < n_pairs; ++i)
        if (pairs[i].expert >= (uint32_t)E) {
            if (bad_expert) *bad_expert = pairs[i].expert;
            return -1;
        }
    memcpy(sorted, pairs, sizeof(ffo_pair) * (size_t)n_pairs);
    g_sort_keys = sort_keys;
    qsort(sorted, (size_t)n_pairs, sizeof(ffo_pair), pair_less);
    g_sort_keys = NULL;
    int32_t ng = 0;
    for (int64_t i = 0; i < n_pairs;) {
        int64_t j = i;
        while (j < n_pairs && sorted[j].expert == sorted[i].expert) ++j;
        groups[ng].expert = sorted[i].expert;
        groups[ng].pair_start = (uint32_t)i;
        groups[ng].pair_count = (uint32_t)(j - i);
        ++ng;
        i = j;
    }
    int32_t nt = 0;
    for (int32_t g = 0; g < ng; g += tile_experts) {
        int32_t end = g + tile_experts < ng ? g + tile_experts : ng;
        tiles[nt].group_start = (uint32_t)g;
        tiles[nt].group_count = (uint32_t)(end - g);
        tiles[nt].pair_start = groups[g].pair_start;
        tiles[nt].pair_count =
            groups[end - 1].pair_start + groups[end - 1].pair_count - groups[g].pair_start;
        ++nt;
    }
    *n_groups = ng;
    *n_tiles = nt;
    return 0;
}

/* ---- routed experts ---------------------------------------------------------------------- */

/* Expert outputs for a list of (token, expert, rank) pairs.  Pairs are bucketed per expert so
 * each expert's weights are expanded once for all of its tokens; per pair the arithmetic is
 * PrefillGroupedRoutedMoETests.swift:122-151 (act rounded to 16 bits, then the down row dots).
 * Writes fp32 values to v32[(token*K+rank)*D] and/or bf16 to p16 at the same index. */
static void routed_values(const ffo_layer *L, const uint16_t *x, int32_t x_stride,
                          const ffo_pair *pairs, int64_t n_pairs, int32_t round_act,
                          int32_t weights_bf16, float *v32, uint16_t *p16) {
    const int32_t E = L->E, D = L->D, K = L->K;
    int64_t *start = (int64_t *)calloc((size_t)E + 1, sizeof(int64_t));
    for (int64_t i = 0; i < n_pairs; ++i) start[pairs[i].expert + 1]++;
    for (int32_t e = 0; e < E; ++e) start[e + 1] += start[e];
    int64_t *cursor = (int64_t *)malloc(sizeof(int64_t) * (size_t)E);
    memcpy(cursor, start, sizeof(int64_t) * (size_t)E);
    int64_t *order = (int64_t *)malloc(sizeof(int64_t) * (size_t)(n_pairs ? n_pairs : 1));
    for (int64_t i = 0; i < n_pairs; ++i) order[cursor[pairs[i].expert]++] = i;
#pragma omp parallel for schedule(dynamic, 1)
    for (int32_t e = 0; e < E; ++e) {
        int32_t n = (int32_t)(start[e + 1] - start[e]);
        if (n == 0) continue;
        uint16_t *xe = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)n * D);
        float *out = (float *)malloc(sizeof(float) * (size_t)n * D);
        for (int32_t j = 0; j < n; ++j) {
            const ffo_pair *p = &pairs[order[start[e] + j]];
            memcpy(xe + (int64_t)j * D, x + (int64_t)p->token * x_stride, sizeof(uint16_t) * (size_t)D);
        }
        expert_ffn_w(L->experts + (uint64_t)e * L->expert_stride, &L->off, D, L->F, xe, n, D, 0,
                     round_act, weights_bf16, out, D);
        for (int32_t j = 0; j < n; ++j) {
            const ffo_pair *p = &pairs[order[start[e] + j]];
            int64_t base = ((int64_t)p->token * K + p->rank) * D;
            for (int32_t d = 0; d < D; ++d) {
                float v = out[(int64_t)j * D + d];
                if (v32) v32[base + d] = v;
                if (p16) p16[base + d] = ffo_bf16_bits(v);
            }
        }
        free(xe);
        free(out);
    }
    free(order);
    free(cursor);
    free(start);
}

/* Per-route partial rows, bf16, at [(token*K + rank)*D] — the contract of the reference's
 * prefill/verify expert kernels (PrefillGroupedRoutedMoETests.swift:122-151).  Rows not named
 * by a pair are left untouched. */
void ffo_route_partials(const ffo_layer *L, const uint16_t *x, int32_t x_stride,
                        const ffo_pair *pairs, int64_t n_pairs, uint16_t *partials) {
    routed_values(L, x, x_stride, pairs, n_pairs, 1, 0, NULL, partials);
}

/* The same with the weights rounded once to bf16 (the tensor-core prefill path's operand). */
void ffo_route_partials_bf16w(const ffo_layer *L, const uint16_t *x, int32_t x_stride,
                              const ffo_pair *pairs, int64_t n_pairs, uint16_t *partials) {
    routed_values(L, x, x_stride, pairs, n_pairs, 1, 1, NULL, partials);
}

/* Tests/ANEFieldfareUpstreamTests/Kernels/Prefill/PrefillMoETests.swift:46-64 with the kernel's
 * fused accumulate (Metal/Prefill/prefill.metal:558-563): acc = fma(w_r, P_r, acc), r ascending,
 * one 16-bit rounding at the end.  residual (optional, added after the ranks) is this build's
 * extension for the shared-FFN sum. */
void ffo_reduce_token_major(const uint16_t *partials, const uint16_t *weights,
                            const uint16_t *residual, int32_t T, int32_t K, int32_t D,
                            uint16_t *out) {
#pragma omp parallel for schedule(static) if (!omp_in_parallel() && (int64_t)T * D > 1 << 16)
    for (int32_t t = 0; t < T; ++t)
        for (int32_t d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (int32_t r = 0; r < K; ++r)
                acc = fmaf(ffo_bf16_to_float(weights[(int64_t)t * K + r]),
                           ffo_bf16_to_float(partials[((int64_t)t * K + r) * D + d]), acc);
            if (residual) acc = acc + ffo_bf16_to_float(residual[(int64_t)t * D + d]);
            out[(int64_t)t * D + d] = ffo_bf16_bits(acc);
        }
}

/* Tests/Support/Validation/Reference/Primitives/RmsNorm.swift:8-39 —
 * y = x * w * 1/sqrt(mean(x^2) + eps); the sum of squares runs in index order. */
void ffo_rmsnorm(const float *x, const float *w, float eps, int32_t n, float *y) {
    float sum_sq = 0.0f;
    for (int32_t i = 0; i < n; ++i) {
        float sq = x[i] * x[i];
        sum_sq = sum_sq + sq;
    }
    float inv = 1.0f / sqrtf(sum_sq / (float)n + eps);
    for (int32_t i = 0; i < n; ++i) {
        float xw = x[i] * w[i];
        y[i] = xw * inv;
    }
}

void ffo_rmsnorm_bf16(const uint16_t *x, const uint16_t *w, float eps, int32_t T, int32_t n,
                      uint16_t *y) {
#pragma omp parallel for schedule(static) if (!omp_in_parallel() && T > 8)
    for (int32_t t = 0; t < T; ++t) {
        float *xf = (float *)malloc(sizeof(float) * (size_t)n * 3);
        float *wf = xf + n, *yf = xf + 2 * n;
        for (int32_t i = 0; i < n; ++i) {
            xf[i] = ffo_bf16_to_float(x[(int64_t)t * n + i]);
            wf[i] = w ? ffo_bf16_to_float(w[i]) : 1.0f;
        }
        ffo_rmsnorm(xf, wf, eps, n, yf);
        for (int32_t i = 0; i < n; ++i) y[(int64_t)t * n + i] = ffo_bf16_bits(yf[i]);
        free(xf);
    }
}

/* ---- the fused steps either side of the block ----------------------------------------------- */

/* 1/sqrt(mean(x^2) + eps) of a 16-bit row, the squares chained by fmaf in index order
 * (Sources/ANEFieldfareHotpath/Metal/Prefill/prefill.metal:54-85 sums them per thread and then across
 * the threadgroup; here one chain). */
static float rms_inv16(const uint16_t *x, int32_t n, float eps) {
    float acc = 0.0f;
    for (int32_t i = 0; i < n; ++i) {
        const float v = ffo_bf16_to_float(x[i]);
        acc = fmaf(v, v, acc);
    }
    return 1.0f / sqrtf(acc / (float)n + eps);
}

/* prefill_post_attn_setup_block (Metal/Prefill/prefill.metal:244-318): per row
 *   a = r16(attn * rms_inv(attn) * w_post_attn);  hidden = r16(hidden + a);
 *   n = hidden * rms_inv(hidden);  dense_x = r16(n * w_pre_ffn);  routed_x = r16(n * w_pre_ffn2);
 *   router_x = r16(n),  r16 = rounding to the 16-bit activation type (bf16 here, fp16 there). */
void ffo_post_attn_setup(uint16_t *hidden, const uint16_t *attn, const uint16_t *w_post_attn,
                         const uint16_t *w_pre_ffn, const uint16_t *w_pre_ffn2, int32_t T, int32_t D,
                         float eps, uint16_t *dense_x, uint16_t *routed_x, uint16_t *router_x) {
    for (int32_t t = 0; t < T; ++t) {
        uint16_t *h = hidden + (int64_t)t * D;
        const uint16_t *a = attn + (int64_t)t * D;
        const float attn_inv = rms_inv16(a, D, eps);
        for (int32_t i = 0; i < D; ++i) {
            const uint16_t an = ffo_bf16_bits(ffo_bf16_to_float(a[i]) * attn_inv * ffo_bf16_to_float(w_post_attn[i]));
            h[i] = ffo_bf16_bits(ffo_bf16_to_float(h[i]) + ffo_bf16_to_float(an));
        }
        const float hidden_inv = rms_inv16(h, D, eps);
        for (int32_t i = 0; i < D; ++i) {
            const float n = ffo_bf16_to_float(h[i]) * hidden_inv;
            dense_x[(int64_t)t * D + i] = ffo_bf16_bits(n * ffo_bf16_to_float(w_pre_ffn[i]));
            routed_x[(int64_t)t * D + i] = ffo_bf16_bits(n * ffo_bf16_to_float(w_pre_ffn2[i]));
            router_x[(int64_t)t * D + i] = ffo_bf16_bits(n);
        }
    }
}

/* prefill_layer_tail_block (Metal/Prefill/prefill.metal:321-399; the one-row form is
 * Metal/Fusions/fused.metal:470-474): per row
 *   t = r16(h2 * rms_inv(h2) * w_postffn2);  h12 = r16(h1 + t);
 *   u = r16(h12 * rms_inv(h12) * w_postffn);  hidden = r16(hidden + u);
 *   hidden = r16(hidden * r16(layer_scalar)). */
void ffo_layer_tail(const uint16_t *h2, const uint16_t *h1, uint16_t *hidden, const uint16_t *w_postffn2,
                    const uint16_t *w_postffn, int32_t T, int32_t D, float eps, float layer_scalar) {
    uint16_t *h12 = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)D);
    const float scale = ffo_bf16_to_float(ffo_bf16_bits(layer_scalar));
    for (int32_t t = 0; t < T; ++t) {
        const uint16_t *r2 = h2 + (int64_t)t * D, *r1 = h1 + (int64_t)t * D;
        uint16_t *h = hidden + (int64_t)t * D;
        const float inv2 = rms_inv16(r2, D, eps);
        for (int32_t i = 0; i < D; ++i) {
            const uint16_t tmp = ffo_bf16_bits(ffo_bf16_to_float(r2[i]) * inv2 * ffo_bf16_to_float(w_postffn2[i]));
            h12[i] = ffo_bf16_bits(ffo_bf16_to_float(r1[i]) + ffo_bf16_to_float(tmp));
        }
        const float inv12 = rms_inv16(h12, D, eps);
        for (int32_t i = 0; i < D; ++i) {
            const uint16_t u = ffo_bf16_bits(ffo_bf16_to_float(h12[i]) * inv12 * ffo_bf16_to_float(w_postffn[i]));
            const uint16_t sum = ffo_bf16_bits(ffo_bf16_to_float(h[i]) + ffo_bf16_to_float(u));
            h[i] = ffo_bf16_bits(ffo_bf16_to_float(sum) * scale);
        }
    }
    free(h12);
}

/* ---- INT8 affine shared FFN -------------------------------------------------------------------- */

/* One output of an INT8 affine matrix row against a 16-bit input row, in the order of the
 * reference kernels (Sources/ANEFieldfareHotpath/Metal/Quant/dequant_int8.metal:41-83) made
 * definite: lane l takes elements 64 g + 2 l and + 1 of every group g in increasing g,
 *   acc = fma(s_g, fma(q1, x1, q0 * x0), acc);  acc = fma(b_g, x0 + x1, acc);
 * the 32 lane sums are added by an xor butterfly (16, 8, 4, 2, 1). */
static float int8_row_dot(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t cols,
                          const uint16_t *x) {
    const int32_t groups = cols / 64;
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int32_t g = 0; g < groups; ++g) {
            const int32_t idx = g * 64 + 2 * l;
            const float x0 = ffo_bf16_to_float(x[idx]), x1 = ffo_bf16_to_float(x[idx + 1]);
            const float q0 = (float)w[idx], q1 = (float)w[idx + 1];
            acc = fmaf(ffo_bf16_to_float(s[g]), fmaf(q1, x1, q0 * x0), acc);
            acc = fmaf(ffo_bf16_to_float(b[g]), x0 + x1, acc);
        }
        lane[l] = acc;
    }
    for (int offset = 16; offset >= 1; offset >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ offset];
        memcpy(lane, next, sizeof(lane));
    }
    return lane[0];
}

/* SharedExpertInt8 (Kernels/MoE/SharedExpertInt8.swift; shared_int8_gate_up_act_simd,
 * dequant_int8.metal:85-138): act = r16(gelu_tanh(r16(gate x)) * r16(up x)), y = r16(down act).
 * Every projection: codes uint8 [rows][cols], scales and biases bf16 [rows][cols/64]. */
void ffo_shared_ffn_int8(const uint8_t *gate_w, const uint16_t *gate_s, const uint16_t *gate_b,
                         const uint8_t *up_w, const uint16_t *up_s, const uint16_t *up_b,
                         const uint8_t *down_w, const uint16_t *down_s, const uint16_t *down_b,
                         int32_t D, int32_t Fs, const uint16_t *x, int32_t T, uint16_t *y) {
#pragma omp parallel for schedule(static) if (!omp_in_parallel() && T > 2)
    for (int32_t t = 0; t < T; ++t) {
        uint16_t *act = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)Fs);
        const uint16_t *xr = x + (int64_t)t * D;
        const int32_t gd = D / 64, gf = Fs / 64;
        for (int32_t f = 0; f < Fs; ++f) {
            const float g = ffo_bf16_to_float(ffo_bf16_bits(
                int8_row_dot(gate_w + (int64_t)f * D, gate_s + (int64_t)f * gd, gate_b + (int64_t)f * gd, D, xr)));
            const float u = ffo_bf16_to_float(ffo_bf16_bits(
                int8_row_dot(up_w + (int64_t)f * D, up_s + (int64_t)f * gd, up_b + (int64_t)f * gd, D, xr)));
            act[f] = ffo_bf16_bits(ffo_gelu_tanh(g) * u);
        }
        for (int32_t d = 0; d < D; ++d)
            y[(int64_t)t * D + d] = ffo_bf16_bits(
                int8_row_dot(down_w + (int64_t)d * Fs, down_s + (int64_t)d * gf, down_b + (int64_t)d * gf, Fs, act));
        free(act);
    }
}

/* ---- whole layer ------------------------------------------------------------------------- */

/* Shared INT4 FFN: gate and up rounded to 16 bits before the activation, the activation rounded
 * again, the down projection rounded on store (moe.metal:548-570 + the down GEMV;
 * Tests/ANEFieldfareUpstreamTests/Kernels/MoE/SharedExpertInt4Tests.swift:19-28). */
static void shared_ffn_w(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t x_stride,
                         int32_t weights_bf16, uint16_t *y) {
    float *out = (float *)malloc(sizeof(float) * (size_t)T * L->D);
    expert_ffn_w(L->shared, &L->shared_off, L->D, L->Fs, x, T, x_stride, 1, 1, weights_bf16, out, L->D);
    ffo_bf16_bits_n(out, y, (int64_t)T * L->D);
    free(out);
}

void ffo_shared_ffn(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t x_stride,
                    uint16_t *y) {
    shared_ffn_w(L, x, T, x_stride, 0, y);
}

void ffo_shared_ffn_bf16w(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t x_stride,
                          uint16_t *y) {
    shared_ffn_w(L, x, T, x_stride, 1, y);
}

/* Router -> top-K -> routed experts (+ shared FFN as the residual) for T rows of x[T][D].
 * FFO_MODE_DECODE follows the decode kernels (moe.metal:597-638): fp32 expert outputs weighted
 * and added in slot order onto the residual, one rounding.  FFO_MODE_PARTIALS follows
 * verify/prefill: bf16 per-route partials, then ffo_reduce_token_major.  y_f32, when given,
 * receives the value before the last rounding. */
void ffo_moe_layer(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t mode, uint16_t *y,
                   float *y_f32, uint32_t *ids_out, uint16_t *w_out) {
    const int32_t D = L->D, K = L->K;
    uint32_t *ids = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)T * K);
    uint16_t *w = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * K);
    ffo_router_topk(L, x, T, D, ids, w, NULL);
    if (ids_out) memcpy(ids_out, ids, sizeof(uint32_t) * (size_t)T * K);
    if (w_out) memcpy(w_out, w, sizeof(uint16_t) * (size_t)T * K);
    const int32_t wb = (mode & FFO_MODE_BF16_WEIGHTS) ? 1 : 0;
    mode &= ~FFO_MODE_BF16_WEIGHTS;
    uint16_t *h1 = NULL;
    if (L->shared) {
        h1 = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * D);
        shared_ffn_w(L, x, T, D, wb, h1);
    }
    ffo_pair *pairs = (ffo_pair *)malloc(sizeof(ffo_pair) * (size_t)T * K);
    int64_t n_pairs = ffo_make_pairs(ids, w, T, K, pairs);
    if (mode == FFO_MODE_DECODE) {
        float *v = (float *)malloc(sizeof(float) * (size_t)T * K * D);
        routed_values(L, x, D, pairs, n_pairs, 1, wb, v, NULL);
        for (int32_t t = 0; t < T; ++t)
            for (int32_t d = 0; d < D; ++d) {
                float acc = h1 ? ffo_bf16_to_float(h1[(int64_t)t * D + d]) : 0.0f;
                for (int32_t r = 0; r < K; ++r) {
                    float weighted =
                        ffo_bf16_to_float(w[(int64_t)t * K + r]) * v[((int64_t)t * K + r) * D + d];
                    acc = acc + weighted;
                }
                if (y_f32) y_f32[(int64_t)t * D + d] = acc;
                y[(int64_t)t * D + d] = ffo_bf16_bits(acc);
            }
        free(v);
    } else {
        uint16_t *p = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * K * D);
        routed_values(L, x, D, pairs, n_pairs, 1, wb, NULL, p);
        ffo_reduce_token_major(p, w, h1, T, K, D, y);
        if (y_f32) {
#pragma omp parallel for schedule(static)
            for (int32_t t = 0; t < T; ++t)
                for (int32_t d = 0; d < D; ++d) {
                    float acc = 0.0f;
                    for (int32_t r = 0; r < K; ++r)
                        acc = fmaf(ffo_bf16_to_float(w[(int64_t)t * K + r]),
                                   ffo_bf16_to_float(p[((int64_t)t * K + r) * D + d]), acc);
                    if (h1) acc = acc + ffo_bf16_to_float(h1[(int64_t)t * D + d]);
                    y_f32[(int64_t)t * D + d] = acc;
                }
        }
        free(p);
    }
    free(pairs);
    free(h1);
    free(w);
    free(ids);
}

/* Benchmark configuration 4: a stack of MoE blocks with an RMSNorm (no weight) in front of each and
 * no attention:  x <- layer_l(rmsnorm(x)),  l = 0 .. n_layers-1;  y = the last block's output.
 * The norm is Tests/Support/Validation/Reference/Primitives/RmsNorm.swift:8-39 on the bf16 rows
 * (fp32 inside, one rounding on store), standing where the reference has its fused layer tail
 * (Sources/ANEFieldfareHotpath/Metal/Prefill/prefill.metal:321-399).  ids_out (optional) receives
 * every layer's routes [n_layers][T][K]. */
void ffo_moe_stack(const ffo_layer *layers, int32_t n_layers, const uint16_t *x, int32_t T, float eps,
                   int32_t mode, uint16_t *y, uint32_t *ids_out) {
    if (n_layers <= 0 || T <= 0) return;
    const int32_t D = layers[0].D;
    uint16_t *cur = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * D);
    uint16_t *normed = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * D);
    memcpy(cur, x, sizeof(uint16_t) * (size_t)T * D);
    for (int32_t l = 0; l < n_layers; ++l) {
        ffo_rmsnorm_bf16(cur, NULL, eps, T, D, normed);
        ffo_moe_layer(&layers[l], normed, T, mode, cur, NULL,
                      ids_out ? ids_out + (int64_t)l * T * layers[l].K : NULL, NULL);
    }
    memcpy(y, cur, sizeof(uint16_t) * (size_t)T * D);
    free(normed);
    free(cur);
}

void ffo_set_num_threads(int32_t n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int32_t ffo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
