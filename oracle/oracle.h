/*
 * CPU oracle for the INT4 mixture-of-experts hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * CPU test references (Swift, under Tests/Support/Validation and the kernel
 * test files cited per function in oracle.c).  It exists to check the CUDA
 * library and to be timed as the CPU baseline; nothing in the shipped library
 * links, loads or calls it.
 *
 * Pinning status.  Integer/byte results (bf16 encode, PRNG streams, nibble
 * order, pair grouping, blob offsets) are pinned against the known answers the
 * reference's own tests hold.  Floating-point layer outputs are "parity
 * unpinned": the reference stores no golden vectors for this path (every
 * expected value is regenerated from a seed at test time) and its Swift/Metal
 * code cannot be compiled or run on Linux, so no reference output exists to
 * compare with.
 */
#ifndef FIELDFARE_ORACLE_H
#define FIELDFARE_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Byte offsets of the nine sub-tensors inside one expert blob. */
typedef struct {
    uint32_t gate_w, gate_s, gate_b;
    uint32_t up_w, up_s, up_b;
    uint32_t down_w, down_s, down_b;
} ffo_offsets;

typedef struct {
    uint32_t token, expert, rank, weight_bits;
} ffo_pair;

typedef struct {
    uint32_t expert, pair_start, pair_count;
} ffo_group;

typedef struct {
    uint32_t group_start, group_count, pair_start, pair_count;
} ffo_tile;

/* One MoE layer as the oracle sees it (all pointers are host memory). */
typedef struct {
    const uint8_t *experts;      /* E blobs, expert_stride apart            */
    uint64_t expert_stride;
    ffo_offsets off;             /* same for every routed expert            */
    const uint8_t *shared;       /* one blob in the same 9-part order, or 0 */
    ffo_offsets shared_off;
    const uint16_t *router_w;    /* bf16 [E][D]                             */
    const uint16_t *router_scale;/* bf16 [D] multiplied into x, or 0        */
    const uint16_t *gain;        /* bf16 [E] per-expert scale, or 0         */
    const float *logit_bias;     /* fp32 [E] added to the logits, or 0      */
    int32_t E, D, F, Fs, K;
} ffo_layer;

enum {
    FFO_MODE_DECODE = 0,  /* y = bf16(residual + sum_k w_k * v_k), v_k fp32           */
    FFO_MODE_PARTIALS = 1,/* P = bf16(v_k); y = bf16(residual + sum_k fma(w_k, P_k))  */
    /* or-ed onto a mode: every weight is rounded once to bf16 before it is multiplied (the operand
     * of the tensor-core prefill path; ffo_dequant_int4_bf16 gives the same values) */
    FFO_MODE_BF16_WEIGHTS = 2
};

uint16_t ffo_bf16_bits(float x);
float ffo_bf16_to_float(uint16_t bits);
void ffo_bf16_bits_n(const float *x, uint16_t *out, int64_t n);
void ffo_bf16_to_float_n(const uint16_t *x, float *out, int64_t n);

uint64_t ffo_splitmix64_next(uint64_t *state);
float ffo_splitmix64_uniform(uint64_t *state, float lo, float hi);
uint64_t ffo_seedtree_key(uint64_t root, const char *label);
void ffo_splitmix64_fill(uint64_t seed, uint64_t *out, int64_t n);

void ffo_quantize_int4_row(const float *row, int32_t n, uint8_t *packed, uint16_t *scales,
                           uint16_t *biases);
void ffo_dequant_int4(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t rows,
                      int32_t cols, float *out);
void ffo_dequant_int4_bf16(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t rows,
                           int32_t cols, uint16_t *out);
float ffo_int4_dot(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t row,
                   int32_t cols, const float *x);
void ffo_int4_gemv_rows(const uint8_t *w, const uint16_t *s, const uint16_t *b, int32_t rows,
                        int32_t cols, const float *x, int32_t x_rows, int32_t x_stride, float *y,
                        int32_t y_stride);
float ffo_gelu_tanh(float x);
void ffo_expert_ffn(const uint8_t *blob, const ffo_offsets *off, int32_t D, int32_t F,
                    const uint16_t *x, int32_t T, int32_t x_stride, int32_t round_gate_up,
                    int32_t round_act, float *out, int32_t out_stride);

void ffo_post_attn_setup(uint16_t *hidden, const uint16_t *attn, const uint16_t *w_post_attn,
                         const uint16_t *w_pre_ffn, const uint16_t *w_pre_ffn2, int32_t T, int32_t D,
                         float eps, uint16_t *dense_x, uint16_t *routed_x, uint16_t *router_x);
void ffo_layer_tail(const uint16_t *h2, const uint16_t *h1, uint16_t *hidden, const uint16_t *w_postffn2,
                    const uint16_t *w_postffn, int32_t T, int32_t D, float eps, float layer_scalar);
void ffo_shared_ffn_int8(const uint8_t *gate_w, const uint16_t *gate_s, const uint16_t *gate_b,
                         const uint8_t *up_w, const uint16_t *up_s, const uint16_t *up_b,
                         const uint8_t *down_w, const uint16_t *down_s, const uint16_t *down_b,
                         int32_t D, int32_t Fs, const uint16_t *x, int32_t T, uint16_t *y);
void ffo_router_logits(const ffo_layer *L, const uint16_t *x, float *logits);
void ffo_router_logits_int8(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases,
                            const uint16_t *effective_scale, const float *logit_bias, int32_t E,
                            int32_t D, const uint16_t *x, float *logits);
void ffo_router_topk_int8(const uint8_t *codes, const uint16_t *scales, const uint16_t *biases,
                          const uint16_t *effective_scale, const float *logit_bias,
                          const uint16_t *gain, int32_t E, int32_t D, int32_t K, const uint16_t *x,
                          int32_t T, int32_t x_stride, uint32_t *ids, uint16_t *weights,
                          float *logits_out);
void ffo_topk(const float *logits, int32_t E, const uint16_t *gain, int32_t K, uint32_t *ids,
              uint16_t *weights, float *weights_f32);
void ffo_router_topk(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t x_stride,
                     uint32_t *ids, uint16_t *weights, float *logits_out);

int64_t ffo_make_pairs(const uint32_t *ids, const uint16_t *weights, int32_t T, int32_t K,
                       ffo_pair *pairs);
int32_t ffo_group_pairs(const ffo_pair *pairs, int64_t n_pairs, int32_t T, int32_t K, int32_t E,
                        int32_t tile_experts, const uint64_t *sort_keys, ffo_pair *sorted,
                        ffo_group *groups, int32_t *n_groups, ffo_tile *tiles, int32_t *n_tiles,
                        uint32_t *bad_expert);
void ffo_route_partials(const ffo_layer *L, const uint16_t *x, int32_t x_stride,
                        const ffo_pair *pairs, int64_t n_pairs, uint16_t *partials);
void ffo_route_partials_bf16w(const ffo_layer *L, const uint16_t *x, int32_t x_stride,
                              const ffo_pair *pairs, int64_t n_pairs, uint16_t *partials);
void ffo_reduce_token_major(const uint16_t *partials, const uint16_t *weights,
                            const uint16_t *residual, int32_t T, int32_t K, int32_t D,
                            uint16_t *out);
void ffo_rmsnorm(const float *x, const float *w, float eps, int32_t n, float *y);
void ffo_rmsnorm_bf16(const uint16_t *x, const uint16_t *w, float eps, int32_t T, int32_t n,
                      uint16_t *y);

void ffo_shared_ffn(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t x_stride,
                    uint16_t *y);
void ffo_shared_ffn_bf16w(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t x_stride,
                          uint16_t *y);
void ffo_moe_layer(const ffo_layer *L, const uint16_t *x, int32_t T, int32_t mode, uint16_t *y,
                   float *y_f32, uint32_t *ids_out, uint16_t *w_out);
void ffo_moe_stack(const ffo_layer *layers, int32_t n_layers, const uint16_t *x, int32_t T, float eps,
                   int32_t mode, uint16_t *y, uint32_t *ids_out);
int32_t ffo_num_threads(void);
void ffo_set_num_threads(int32_t n);

#ifdef __cplusplus
}
#endif
#endif
