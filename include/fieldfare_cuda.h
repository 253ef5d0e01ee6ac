/*
 * libfieldfare_cuda.so — C ABI of the B200 (sm_100a) INT4 mixture-of-experts hot path.
 *
 * The library stands in for the reference's Metal kernels and their Swift wrappers on one path:
 * router top-8 -> routed INT4 GeGLU experts (+ the shared INT4 FFN) -> weighted combine.  Each
 * entry point names the reference interface it replaces by that file's path inside the reference
 * project.  Conventions follow the reference's own native boundary
 * (Sources/ANEFieldfareANECarrier/include/ANEExpertCarrier.h:14-38): an opaque handle, `bool`
 * results, errors returned as strdup'd C strings the caller frees (ff_string_free or free()),
 * an explicit destroy, a plain info struct.  Calls on one context must be serialized by the
 * caller; different contexts (one per GPU, each driven by its own host thread) and the
 * context-free entry points may be called concurrently.
 *
 * Operators take DEVICE pointers and a CUDA stream (passed as void*, a cudaStream_t; NULL is the
 * legacy default stream).  They enqueue work and return without waiting, the way the
 * reference's `encode...(commandBuffer:)` methods do; only the *_host entry points copy and
 * wait.  All 16-bit activations, scales, biases and route weights are bf16 bit patterns.
 *
 * There is no CPU fallback: every operator launches CUDA kernels on the context's device and
 * fails with a message when that is impossible.
 */
#ifndef FIELDFARE_CUDA_H
#define FIELDFARE_CUDA_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct FFContext FFContext;

/* Byte offsets of the nine sub-tensors of one expert blob.  Layout-identical to the reference's
 * `MoEExpertOffsets` (Sources/ANEFieldfareHotpath/Kernels/MoE/MoE.swift:4-15) and the Metal
 * `ExpertOffsets` (Metal/MoE/moe.metal:49-59). */
typedef struct {
    uint32_t gateWOff, gateSOff, gateBOff;
    uint32_t upWOff, upSOff, upBOff;
    uint32_t downWOff, downSOff, downBOff;
} FFExpertOffsets;

/* Layout-identical to `PrefillTokenExpertPair` (Kernels/Prefill/MoE/PrefillRouter.swift:4-21);
 * the low 16 bits of weightBitsAndReserved hold the route weight (bf16 here, fp16 there). */
typedef struct {
    uint32_t token, expert, rank, weightBitsAndReserved;
} FFTokenExpertPair;

/* `PrefillMoEGroup` / `PrefillMoETile` (Kernels/Prefill/MoE/PrefillMoEGrouping.swift:4-29). */
typedef struct {
    uint32_t expert, pairStart, pairCount;
} FFMoEGroup;
typedef struct {
    uint32_t groupStart, groupCount, pairStart, pairCount;
} FFMoETile;

/* One affine INT4 matrix [rows][cols]: packed codes (cols/2 bytes per row), bf16 scales and
 * biases (cols/64 per row).  Mirrors `SharedExpertProjection`
 * (Kernels/MoE/SharedExpertInt8.swift:7-29) with raw pointers in place of (buffer, offset). */
typedef struct {
    const void *weights;
    const void *scales;
    const void *biases;
    uint32_t rows, cols;
} FFProjection;

/* Shape of the model slice a context serves; fixed at creation so scratch is allocated once. */
typedef struct {
    uint32_t layers;        /* layer slots                                   */
    uint32_t experts;       /* routed experts per layer held by this context */
    uint32_t d;             /* model width (2816)                            */
    uint32_t f;             /* routed intermediate width (704)               */
    uint32_t sharedF;       /* shared FFN intermediate width (2112), 0=none  */
    uint32_t topK;          /* routes per token (8)                          */
    uint32_t maxTokens;     /* largest T any operator call will pass         */
} FFConfig;

/* Counters, in the spirit of `ANEExpertCarrierInfo` (ANEExpertCarrier.h:16-23). */
typedef struct {
    uint64_t kernelLaunches;     /* kernels this context has enqueued          */
    uint64_t weightBytesResident;/* expert + shared + router bytes held in HBM */
    uint64_t scratchBytes;       /* device scratch owned by the context        */
    uint32_t lastActiveExperts;  /* distinct experts of the last verify/prefill (after a sync) */
    uint32_t lastPrefillUnits;   /* GEMM work units of the last prefill call   */
    uint32_t deviceOrdinal;
    uint32_t smCount;
    uint32_t deviceErrorFlag;    /* non-zero: a kernel gave up a bounded wait (after a sync) */
    uint32_t reserved;
} FFInfo;

/* Device time of one kernel name, summed over the launches made while tracing was on. */
typedef struct {
    char name[40];
    uint64_t launches;
    double milliseconds;
} FFTraceEntry;

/* ---- lifetime ---------------------------------------------------------------------------- */

/* Replaces the construction of the reference's kernel wrapper objects from a `MetalContext`
 * (Kernels/MoE/MoE.swift:62-125, Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:210-250).
 * Returns NULL and sets *error on failure (no CUDA device, unsupported shape, out of memory). */
FFContext *ff_create(int32_t deviceOrdinal, const FFConfig *config, const char **error);
void ff_destroy(FFContext *ctx);
void ff_string_free(const char *message);
FFInfo ff_get_info(const FFContext *ctx);

/* Per-kernel device timing: while on, every kernel launch is bracketed by CUDA events on its
 * stream.  ff_get_trace waits for the device, fills up to `capacity` entries (one per kernel
 * name), clears the record and returns the number of names.  The counterpart of the reference's
 * per-encoder GPU timestamps (Infrastructure/Metal/GPUTrace.swift:67-90).  Do not trace while a
 * stream is being captured into a CUDA graph. */
/* Waits for the device and clears the flag ff_get_info reports as deviceErrorFlag (it is sticky:
 * set by a kernel that gave up a bounded wait, 1..11, or that met a route naming an expert that is
 * not resident, 12 — the condition the reference traps with "route expert N is out of range",
 * Runtime/Inference/RealForwardRunner.swift:815). */
bool ff_reset_device_error(FFContext *ctx, const char **error);

void ff_set_tracing(FFContext *ctx, bool enabled);
uint32_t ff_get_trace(FFContext *ctx, FFTraceEntry *entries, uint32_t capacity);

/* Phase times of the last one-token ff_moe_layer / ff_moe_decode launched while tracing was on,
 * in microseconds, from timestamps the first CTA takes inside the kernel: [0] phase A work
 * (router, shared gate/up), [1] wait for the top-k warps, [2] publishing the routes, [3] phase B
 * work (routed gate/up, shared down), [4] requests of phase C's tiles and the CTA-wide wait for phase B's
 * warps, [5] phase C (polling the routed activations, routed down + combine).  A
 * diagnostic with no counterpart in the reference beyond its per-phase GPU nanoseconds
 * (Runtime/Inference/RealForwardRunner.swift:2146-2150). */
bool ff_decode_phase_times(FFContext *ctx, double *microseconds, const char **error);

/* Finer view of the same launch: 288 values [cta][phase][warp][event] for the first and the last
 * CTA (cta 0/1), phases A/B/C, 16 warps, event 0 = the warp's copy requests issued, 1 = its data
 * arrived, 2 = its rows done; microseconds since the first CTA started, -1 where a warp had no
 * work.  Diagnostic, no reference counterpart. */
#define FF_DECODE_WARP_TIME_COUNT 288
bool ff_decode_warp_times(FFContext *ctx, double *microseconds, const char **error);

/* ---- HBM-resident weights ---------------------------------------------------------------- */

/* Copies one layer file's bytes (`packed_experts/layer_%02d.bin`: expertCount blobs,
 * expertStride apart, the nine offsets shared by every expert) verbatim into device memory.
 * Replaces the mmap expert store: `MappedExpertLayer`
 * (Infrastructure/Streaming/MappedExpertLayer.swift:44-209) and `Model.routedExpertOffsets`
 * (Runtime/Inference/ModelExpertIO.swift:11-30).  Checks the schema rules of
 * Runtime/Inference/Model.swift:478-527 (sizes, 4-byte weight / 2-byte scale alignment) plus
 * the 16-byte alignment the 128-bit loads need. */
bool ff_load_layer(FFContext *ctx, uint32_t layer, const void *hostBytes, uint64_t byteCount,
                   uint32_t expertCount, uint64_t expertStride, const FFExpertOffsets *offsets,
                   const char **error);

/* What a validated `packed_experts/layout.json` says. */
typedef struct {
    uint64_t expertStride;
    uint32_t numLayers, expertsPerLayer;
    FFExpertOffsets offsets;      /* the nine sub-tensor offsets of layer 0's experts */
    uint32_t identityPlacement;   /* 1: every expert sits at rank == its id in its layer file */
} FFGTurboLayoutInfo;

/* Reads and checks `<modelDir>/packed_experts/layout.json` without touching a GPU: the decode and
 * structural validation of Sources/ANEFieldfareImportedFormat/GTurboPackedExpertsLayoutV1.swift:65-162
 * (dimensions and stride, duplicate layers and file names, expert ids and physical ranks, per-tensor
 * offset/size/dtype/shape, overlapping ranges) and the runtime's schema check of the routed experts
 * against the model's widths d and f (Runtime/Inference/Model.swift:478-527: U32 4-bit weights
 * [rows][cols/8], BF16 scales and biases [rows][cols/64], alignment, identical across a layer's
 * experts).  Failures carry the reference's messages. */
bool ff_gturbo_validate_layout(const char *modelDir, uint32_t d, uint32_t f, FFGTurboLayoutInfo *info,
                               const char **error);

/* Loads an installed model's routed experts into HBM: validates the layout as above, then copies
 * every `packed_experts/<file>` it names into layer slot `layer` (ff_load_layer), expert e's blob
 * taken from offset physicalRank * expertStride of its file — the expert lookup of
 * Sources/ANEFieldfareHotpath/Infrastructure/ModelIO/PackedExpertsLayout.swift:55-90 and
 * Runtime/Inference/ModelExpertIO.swift:11-35.  A layer file whose size is not expertsPerLayer
 * strides is refused like the reference's manifest cross-check. */
bool ff_load_model_dir(FFContext *ctx, const char *modelDir, const char **error);

/* The shared FFN's three projections from HOST pointers (the reference keeps them as resident
 * tensors: Kernels/MoE/SharedExpertInt4.swift:32-38). */
bool ff_load_shared(FFContext *ctx, uint32_t layer, const FFProjection *gate,
                    const FFProjection *up, const FFProjection *down, const char **error);

/* Router weights bf16 [experts][d] from HOST memory, with the optional per-input scale
 * (`effectiveScale`, bf16 [d]), per-expert gain (`perExpertScale`, bf16 [experts]) — the
 * arguments of `MoE.encodeRouterGemma4` (Kernels/MoE/MoE.swift:168-180) — and an optional fp32
 * per-expert additive logit bias (used by the synthetic benchmark configurations). */
bool ff_load_router(FFContext *ctx, uint32_t layer, const uint16_t *weights,
                    const uint16_t *effectiveScale, const uint16_t *perExpertScale,
                    const float *logitBias, uint32_t experts, uint32_t d, const char **error);

/* The shared FFN in the form the shipped checkpoints carry it: INT8 affine codes (one byte a weight)
 * with one bf16 scale and bias per group of 64 inputs, three projections from HOST memory —
 * `weights` uint8 [rows][cols], `scales`/`biases` bf16 [rows][cols/64]
 * (Kernels/MoE/SharedExpertInt8.swift:7-29; kernels Metal/Quant/dequant_int8.metal:41-138).  Replaces
 * any shared FFN the layer had; every operator that uses the shared FFN takes either form (the
 * INT8 one runs as launches of its own, its rows are the residual of the routed part). */
bool ff_load_shared_int8(FFContext *ctx, uint32_t layer, const FFProjection *gate, const FFProjection *up,
                         const FFProjection *down, const char **error);

/* The router in the form the shipped checkpoints carry it: INT8 affine codes [experts][d] with one
 * bf16 scale and bias per group of 64 inputs (Runtime/Inference/Model.swift:473-475; kernel body
 * Metal/MoE/moe.metal:65-103), from HOST memory; the other arguments as for ff_load_router.
 * Replaces any router the layer had.  Every operator that runs the router takes either form; the
 * one-token kernel then runs the INT8 router as launches of its own in front. */
bool ff_load_router_int8(FFContext *ctx, uint32_t layer, const uint8_t *codes, const uint16_t *scales,
                         const uint16_t *biases, const uint16_t *effectiveScale,
                         const uint16_t *perExpertScale, const float *logitBias, uint32_t experts,
                         uint32_t d, const char **error);

/* Device address of one resident expert blob (the entry the reference's address table holds:
 * Metal/MoE/moe.metal:576-593), 0 when absent. */
uint64_t ff_expert_address(const FFContext *ctx, uint32_t layer, uint32_t expert);

/* ---- operators (device pointers, asynchronous on `stream`) -------------------------------- */

/* Parity hook: expands one resident matrix to fp32 [rows][cols] as w = q*scale + bias.
 * expert = -1 selects the shared FFN; role 0/1/2 = gate/up/down.  Counterpart of the
 * reference's expansion check (Tests/ANEFieldfareHotpathTests/ANEQuantizedCarrierTests.swift:67,
 * Metal/ANE/ane_prefill.metal:17-43). */
bool ff_dequant_probe(FFContext *ctx, uint32_t layer, int32_t expert, uint32_t role, float *out,
                      void *stream, const char **error);
/* Same matrix as the bf16 operand the prefill tensor-core path multiplies. */
bool ff_dequant_probe_bf16(FFContext *ctx, uint32_t layer, int32_t expert, uint32_t role,
                           uint16_t *out, void *stream, const char **error);

/* Router logits, top-K selection (higher score, then lower expert id), softmax over the
 * selected K, times the per-expert gain.  x is bf16 [tokens][xStride]; ids uint32 [tokens][K],
 * weights bf16 [tokens][K]; logits (optional) fp32 [tokens][experts].  Replaces
 * `MoE.encodeRouterGemma4` / `encodeRouterRowsGemma4` (Kernels/MoE/MoE.swift:168-300) and
 * `PrefillRouter.encodeGemma4Block` (Kernels/Prefill/MoE/PrefillRouter.swift:30-73). */
bool ff_router_topk(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                    uint32_t tokens, uint32_t *ids, uint16_t *weights, float *logits,
                    void *stream, const char **error);

/* Decode, one token: y[d] = bf16(residual[d] + sum_k w_k * down_k(gelu(gate_k x) * up_k x)).
 * residual may be NULL (zero).  Replaces `MoE.encodeRoutedPersistentGPUSlots` =
 * gather slots + phase 1 + phase 2 (Kernels/MoE/MoE.swift:312-341,384-417,429-496). */
bool ff_moe_decode(FFContext *ctx, uint32_t layer, const uint16_t *x, const uint32_t *ids,
                   const uint16_t *weights, const uint16_t *residual, uint16_t *y, void *stream,
                   const char **error);

/* Verify block, 1..16 tokens: every (token, rank) route writes its bf16 partial row at
 * partials[(token*K + rank)*d]; each active expert's weights are read once for all of its
 * tokens.  Replaces `PrefillGroupedRoutedMoE.encodeVerifyBound` / `encodeVerifyRows`
 * (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:331-448). */
bool ff_moe_verify(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                   uint32_t tokens, const uint32_t *ids, uint16_t *partials, void *stream,
                   const char **error);

/* Prefill, any token count: device-side permute (the host sort of
 * Kernels/Prefill/MoE/PrefillMoEGrouping.swift:49-110), then the grouped INT4->bf16 tensor-core
 * GEMMs, writing the same partial rows.  Replaces `PrefillGroupedRoutedMoE.encodeStreamedBatched`
 * (PrefillGroupedRoutedMoE.swift:275-326) and the `RoutedPrefillGuest.runLayer` plug-in
 * (Runtime/Supervisor/DeviceSupervisor.swift:18-22). */
bool ff_moe_prefill(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                    uint32_t tokens, const uint32_t *ids, uint16_t *partials, void *stream,
                    const char **error);

/* y[t][c] = bf16(sum_r fma(w[t][r], partials[(t*K+r)*d + c]) (+ residual[t][c])).  Replaces
 * `PrefillMoE.encodeReduceTokenMajor` (Kernels/Prefill/MoE/PrefillMoE.swift:11-32); the optional
 * residual is an addition for the shared-FFN sum. */
bool ff_moe_reduce(FFContext *ctx, const uint16_t *partials, const uint16_t *weights,
                   const uint16_t *residual, uint16_t *y, uint32_t tokens, void *stream,
                   const char **error);

/* The same reduce over partial rows that lie in another order: the row of route (t, r) is row
 * rowIndex[t*K + r] of `partials` (uint32, every entry below the caller's row count).  Used under
 * expert parallelism, where the rows come back from the other GPUs grouped by source, so that no
 * pass over memory is spent on putting them back into (token, rank) order.  The arithmetic per
 * output element is that of ff_moe_reduce.  No counterpart in the reference (one device there). */
bool ff_moe_reduce_indexed(FFContext *ctx, const uint16_t *partials, const uint32_t *rowIndex,
                           const uint16_t *weights, const uint16_t *residual, uint16_t *y,
                           uint32_t tokens, void *stream, const char **error);

/* Shared INT4 FFN for `tokens` rows: y = down(gelu(bf16(gate x)) * bf16(up x)).  GEMV kernels
 * up to 16 rows, tensor-core GEMMs above.  Replaces `SharedExpertInt4.encode`
 * (Kernels/MoE/SharedExpertInt4.swift:32-88) and `PrefillSharedExpert.encodeBlock`
 * (Kernels/Prefill/MoE/PrefillSharedExpert.swift:51-137). */
bool ff_shared_ffn(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                   uint32_t tokens, uint16_t *y, void *stream, const char **error);

/* The shared INT4 FFN for up to 16 rows for callers that must not allocate device memory: a
 * decode loop on a latency budget, where cudaMalloc/cudaFree would synchronize the whole device,
 * or a process whose HBM is already reserved by another runtime (a serving engine that
 * pre-allocates its pool), where cudaMalloc fails or is forbidden by policy.  It has no
 * counterpart in the reference.  It needs no FFContext: the three projections, x and y are
 * DEVICE pointers supplied by the caller, and the only scratch (the GeGLU activations between the
 * two kernels) is a fixed 128 KiB array inside the library image, which every GPU that loads the
 * library holds until the process exits.  Sizes are therefore limited to rows <= 16,
 * intermediate width (gate->rows) <= 4096 and model width (gate->cols) <= 16384; larger requests
 * fail with a message before anything is enqueued.  (Inside those limits every combination runs:
 * when the staged input rows of a kernel do not fit in shared memory together, e.g. 16 rows of
 * width 4096, the kernel is launched in passes of fewer rows.)  x must be 4-byte aligned with an
 * even xStride.  The call performs no cudaMalloc, cudaFree or other allocating routine.  The
 * first call on each device looks up that array's device address (with the device current; the
 * look-up is guarded, so any host thread may make it); make that first call before any stream
 * capture begins.  All calls on a device share the one array and it keeps the last call's
 * contents: nothing in it needs clearing (every element read was written earlier in the same
 * call), but two calls whose kernels overlap on the GPU (issued on different streams without an
 * ordering between them) race on it and must be ordered by the caller.  For 2..16 rows the
 * results are bitwise those of ff_shared_ffn on the same weights and rows (the same kernels); one
 * row differs from ff_shared_ffn, which then runs inside the fused decode kernel with another
 * summation order, by rounding only. */
bool ff_shared_ffn_noalloc(const FFProjection *gate, const FFProjection *up,
                           const FFProjection *down, const uint16_t *x, uint32_t xStride,
                           uint32_t rows, uint16_t *y, uint32_t yStride, void *stream,
                           const char **error);

/* Y[r][o] = sum_k W[o][k] X[r][k] for rows <= 16 input rows, all pointers on the device.
 * Replaces `DequantInt4GEMV.encodeRows` (Kernels/Quant/DequantInt4GEMV.swift:72-117). */
bool ff_int4_gemv_rows(FFContext *ctx, const FFProjection *projection, const uint16_t *x,
                       uint32_t xStride, uint32_t rows, uint16_t *y, uint32_t yStride,
                       void *stream, const char **error);

/* y = x * rsqrt(mean(x^2) + eps) * w per row (w may be NULL).  The inter-layer glue of the
 * layer stack (Metal/Primitives/rmsnorm.metal:65, Metal/Prefill/prefill.metal:88). */
bool ff_rmsnorm(FFContext *ctx, const uint16_t *x, const uint16_t *w, float eps, uint32_t tokens,
                uint16_t *y, void *stream, const char **error);

/* The whole block for `tokens` rows: router -> routed experts + shared FFN -> y, choosing the
 * decode (1), verify (2..16) or prefill path by token count.  This is the unit the throughput
 * metric times.  ids/weights (optional) receive the routes. */
bool ff_moe_layer(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t tokens,
                  uint16_t *y, uint32_t *ids, uint16_t *weights, void *stream,
                  const char **error);

/* The layer stack of benchmark configuration 4 (MoE blocks with an RMSNorm between them, no
 * attention): for l = firstLayer .. firstLayer+layerCount-1:  x <- ff_moe_layer(l, rmsnorm(x)),
 * rmsnorm without a weight, y receives the last block's output.  ids (optional) receives every
 * layer's routes, uint32 [layerCount][tokens][K].  The glue stands where the reference has its
 * fused layer tail (Metal/Prefill/prefill.metal:321-399; CPU statement
 * Tests/Support/Validation/Reference/Primitives/RmsNorm.swift:8-39). */
bool ff_moe_stack(FFContext *ctx, uint32_t firstLayer, uint32_t layerCount, const uint16_t *x,
                  uint32_t tokens, float eps, uint16_t *y, uint32_t *ids, void *stream,
                  const char **error);

/* ff_moe_layer with HOST buffers: copies x in, runs, copies y out, waits.  Host pointers should
 * be page-locked for full copy bandwidth.  One token with a page-locked, 16-byte aligned hostY
 * takes a path without copies around the kernel: the row travels in the kernel's parameters, the
 * kernel writes hostY itself and reports completion through page-locked memory that this call
 * polls; results are the same bits. */
bool ff_moe_layer_host(FFContext *ctx, uint32_t layer, const uint16_t *hostX, uint32_t tokens,
                       uint16_t *hostY, const char **error);

/* ---- host-side permute (exact integer work) ----------------------------------------------- */

/* `PrefillRouter.makeTokenExpertPairs` (Kernels/Prefill/MoE/PrefillRouter.swift:75-95). */
uint64_t ff_make_token_expert_pairs(const uint32_t *ids, const uint16_t *weights,
                                    uint32_t tokens, uint32_t topK, FFTokenExpertPair *pairs);

/* `PrefillMoEGrouping.groupTokenExpertPairs` (PrefillMoEGrouping.swift:49-110): sorted pairs,
 * per-expert groups, tiles of up to tileExpertCount (1..16) groups.  Output arrays must hold
 * pairCount pairs, min(experts, pairCount) groups and as many tiles.  Fails with
 * "route expert N is out of range" like the reference. */
bool ff_group_token_expert_pairs(const FFTokenExpertPair *pairs, uint64_t pairCount,
                                 uint32_t tokens, uint32_t topK, uint32_t experts,
                                 uint32_t tileExpertCount, const uint64_t *expertSortKeys,
                                 FFTokenExpertPair *sortedPairs, FFMoEGroup *groups,
                                 uint32_t *groupCount, FFMoETile *tiles, uint32_t *tileCount,
                                 const char **error);

/* The fused step in front of the block, `prefill_post_attn_setup_block`
 * (Metal/Prefill/prefill.metal:244-318): rows [tokens][d] contiguous, bf16, device pointers; norm
 * weights bf16 [d].  hidden <- r16(hidden + r16(attn * rms_inv(attn) * wPostAttn)); with
 * n = hidden * rms_inv(hidden): denseX = r16(n * wPreFfn) (input of the shared FFN), routedX =
 * r16(n * wPreFfn2) (input of the routed experts), routerX = r16(n) (input of the router). */
bool ff_post_attn_setup(FFContext *ctx, uint16_t *hidden, const uint16_t *attn, const uint16_t *wPostAttn,
                        const uint16_t *wPreFfn, const uint16_t *wPreFfn2, uint32_t tokens, float eps,
                        uint16_t *denseX, uint16_t *routedX, uint16_t *routerX, void *stream,
                        const char **error);

/* The fused step behind the block, `prefill_layer_tail_block` (Metal/Prefill/prefill.metal:321-399;
 * one row: Metal/Fusions/fused.metal:470-474): h2 = the routed experts' combined rows, h1 = the
 * shared FFN's rows; hidden <- r16(r16(hidden + r16(h12 * rms_inv(h12) * wPostFfn)) * r16(layerScalar))
 * with h12 = r16(h1 + r16(h2 * rms_inv(h2) * wPostFfn2)).  In place on `hidden`. */
bool ff_layer_tail(FFContext *ctx, const uint16_t *h2, const uint16_t *h1, uint16_t *hidden,
                   const uint16_t *wPostFfn2, const uint16_t *wPostFfn, uint32_t tokens, float eps,
                   float layerScalar, void *stream, const char **error);

/* The device-side permute on its own (the sort of PrefillMoEGrouping.groupTokenExpertPairs,
 * Kernels/Prefill/MoE/PrefillMoEGrouping.swift:49-110, by any group id): `groupIds` [tokens][topK] on
 * the device, ids >= `groups` are dropped; `sortedPairs` (device) receives (token, group, rank, 0)
 * in (group, token, rank) order, `offsets` (device, [groups + 1]) every group's first row.  The
 * expert-parallel dispatch sorts a rank's routes by destination rank with it.  Asynchronous. */
bool ff_sort_routes(FFContext *ctx, const uint32_t *groupIds, uint32_t tokens, uint32_t groups,
                    FFTokenExpertPair *sortedPairs, uint32_t *offsets, cudaStream_t stream,
                    const char **error);

/* ---- expert parallelism over several GPUs of one process ----------------------------------- */

/* A group of `world` ranks, one GPU each, that splits every layer's experts evenly: rank p holds
 * experts [p*E/world, (p+1)*E/world).  The reference runs on one device and has no counterpart; the
 * operator it stands in for is the whole block of `PrefillMoE` (Kernels/Prefill/MoE/PrefillMoE.swift:
 * 60-140) with the grouped experts spread over devices.  `home[r]` is rank r's context with the
 * router and the shared FFN of every layer (experts = E, topK = K; it needs no expert blobs),
 * `expert[r]` its context holding E/world experts per layer in local order, created with topK = 1
 * (a received row is a one-route token) and maxTokens >= the capacity.  `capacityRows` bounds the
 * rows one rank may receive in a call (0: world * maxTokens * K, the worst case).  Every pair of
 * the group's devices must have peer access.  The contexts stay the caller's. */
typedef struct FFEPGroup FFEPGroup;
FFEPGroup *ff_ep_create(FFContext *const *home, FFContext *const *expert, uint32_t world,
                        uint32_t capacityRows, const char **error);
void ff_ep_destroy(FFEPGroup *group);

/* One MoE block under expert parallelism: x[r] and y[r] are bf16 [tokens][d] on rank r's device,
 * contiguous and 16-byte aligned.  Per rank: router top-K, routes sorted by destination rank on the
 * device, rows and local expert ids stored into the destination's receive buffer over NVLink, the
 * destination's grouped INT4 experts, partial rows copied back, weighted sum in rank order plus the
 * shared FFN's rows.  Rows travel once per route.  The call runs on the group's own streams and is
 * synchronous: inputs must be complete when it is made, outputs are complete when it returns.
 * Results equal ff_moe_layer's on one device holding all experts, bit for bit, for more than 16
 * rows per rank. */
bool ff_ep_moe_layer(FFEPGroup *group, uint32_t layer, const uint16_t *const *x, uint32_t tokens,
                     uint16_t *const *y, const char **error);
/* The stack of benchmark configuration 4 under expert parallelism, ff_moe_stack's statement per
 * rank: for l = firstLayer .. firstLayer+layerCount-1: x <- block(l, rmsnorm(x)).  Between layers
 * the ranks are ordered by events only; the host waits once per layer, for the row counts.
 * Synchronous like ff_ep_moe_layer. */
bool ff_ep_moe_stack(FFEPGroup *group, uint32_t firstLayer, uint32_t layerCount, const uint16_t *const *x,
                     uint32_t tokens, float eps, uint16_t *const *y, const char **error);
/* Where the experts of `layer` live: expert e on rank rankOf[e] in slot localOf[e] of that rank's
 * expert context (host arrays [experts]; every slot of every rank taken once).  Without this call
 * a layer's experts sit in contiguous blocks.  A placement that evens out a skewed routing load
 * keeps the ranks' GEMMs the same length; the blob layout of a layer file is untouched. */
bool ff_ep_set_placement(FFEPGroup *group, uint32_t layer, const uint32_t *rankOf, const uint32_t *localOf,
                         const char **error);
/* Tracing: while enabled, every layer of a call records CUDA events at its phase boundaries on every
 * rank; ff_ep_get_phase_times copies the last traced call's sums over its layers, milliseconds
 * [world][10] in rank order: router (with the stack's RMSNorm), plan (destination, sort, row index),
 * host (the wait for the counts and the queueing of the send), send, wait for the other ranks'
 * rows, experts, copies home (second stream, from the end of the experts), shared FFN (from the
 * end of the experts), wait for the partial rows, reduce.  Returns the number of values written. */
void ff_ep_set_tracing(FFEPGroup *group, bool enabled);
uint32_t ff_ep_get_phase_times(const FFEPGroup *group, double *milliseconds, uint32_t capacity);
/* Rows the last block sent to another GPU (each also came back as a partial row). */
uint64_t ff_ep_last_rows_sent(const FFEPGroup *group);

/* Device-side result of the last ff_moe_prefill permute, copied to the host after a sync:
 * the expert-sorted pairs and per-expert row offsets [experts+1].  For parity tests. */
bool ff_last_prefill_routes(FFContext *ctx, FFTokenExpertPair *sortedPairs, uint32_t *offsets,
                            const char **error);

#ifdef __cplusplus
}
#endif
#endif
