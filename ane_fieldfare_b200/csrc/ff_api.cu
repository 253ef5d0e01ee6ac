// Operator entry points of the C ABI: argument checks, path selection by row count, launches.
#include <string>

#include "ff_internal.cuh"

using namespace ff;

namespace {

struct Call {
    FFContext *ctx;
    LayerStore *L;
    cudaStream_t stream;
};

bool begin(FFContext *ctx, uint32_t layer, void *stream, const char **error, Call *out) {
    if (error) *error = nullptr;
    if (!ctx) return fail(error, "null context");
    if (layer >= ctx->cfg.layers) return fail(error, "layer " + std::to_string(layer) + " out of range");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    out->ctx = ctx;
    out->L = &ctx->layers[layer];
    out->stream = static_cast<cudaStream_t>(stream);
    return true;
}

bool check_rows(const FFContext *ctx, const void *x, uint32_t xStride, uint32_t tokens,
                const char **error) {
    if (!x) return fail(error, "input pointer is null");
    if (tokens > ctx->cfg.maxTokens)
        return fail(error, std::to_string(tokens) + " rows exceed the context's maxTokens " +
                               std::to_string(ctx->cfg.maxTokens));
    if (xStride < ctx->cfg.d) return fail(error, "hidden stride is too small");
    if (xStride % 8 || (reinterpret_cast<uintptr_t>(x) & 15u))
        return fail(error, "input rows must be 16-byte aligned (stride a multiple of 8 elements)");
    return true;
}

bool select_matrix(const Call &c, int32_t expert, uint32_t role, const uint8_t **w,
                   const uint16_t **s, const uint16_t **b, uint32_t *rows, uint32_t *cols,
                   const char **error) {
    if (role > 2) return fail(error, "role must be 0 (gate), 1 (up) or 2 (down)");
    const FFConfig &cfg = c.ctx->cfg;
    const uint8_t *blob;
    const FFExpertOffsets *off;
    uint32_t f;
    if (expert < 0) {
        if (!c.L->shared) return fail(error, "layer has no resident shared FFN");
        blob = c.L->shared;
        off = &c.L->sharedOff;
        f = cfg.sharedF;
    } else {
        if (!c.L->experts || (uint32_t)expert >= c.L->expertCount)
            return fail(error, "expert " + std::to_string(expert) + " is not resident");
        blob = c.L->experts + (uint64_t)expert * c.L->stride;
        off = &c.L->off;
        f = cfg.f;
    }
    const uint32_t *o = &off->gateWOff;
    *w = blob + o[3 * role];
    *s = reinterpret_cast<const uint16_t *>(blob + o[3 * role + 1]);
    *b = reinterpret_cast<const uint16_t *>(blob + o[3 * role + 2]);
    *rows = role == 2 ? cfg.d : f;
    *cols = role == 2 ? f : cfg.d;
    return true;
}

}  // namespace

extern "C" {

bool ff_dequant_probe(FFContext *ctx, uint32_t layer, int32_t expert, uint32_t role, float *out,
                      void *stream, const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    const uint8_t *w;
    const uint16_t *s, *b;
    uint32_t rows, cols;
    if (!select_matrix(c, expert, role, &w, &s, &b, &rows, &cols, error)) return false;
    return launch_dequant_probe(ctx, w, s, b, rows, cols, out, nullptr, c.stream, error);
}

bool ff_dequant_probe_bf16(FFContext *ctx, uint32_t layer, int32_t expert, uint32_t role,
                           uint16_t *out, void *stream, const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    const uint8_t *w;
    const uint16_t *s, *b;
    uint32_t rows, cols;
    if (!select_matrix(c, expert, role, &w, &s, &b, &rows, &cols, error)) return false;
    return launch_dequant_probe(ctx, w, s, b, rows, cols, nullptr, out, c.stream, error);
}

bool ff_router_topk(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                    uint32_t tokens, uint32_t *ids, uint16_t *weights, float *logits,
                    void *stream, const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    if (!check_rows(ctx, x, xStride, tokens, error)) return false;
    if (!ids || !weights) return fail(error, "output pointer is null");
    return launch_router_topk(ctx, *c.L, x, xStride, tokens, ids, weights, logits, c.stream, error);
}

bool ff_moe_decode(FFContext *ctx, uint32_t layer, const uint16_t *x, const uint32_t *ids,
                   const uint16_t *weights, const uint16_t *residual, uint16_t *y, void *stream,
                   const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    if (!check_rows(ctx, x, ctx->cfg.d, 1, error)) return false;
    if (!ids || !weights || !y) return fail(error, "null argument");
    ctx->lastTokens = 1;
    return launch_block_small(ctx, *c.L, x, ctx->cfg.d, 1, ids, weights, false, true, residual,
                              nullptr, nullptr, y, c.stream, error);
}

bool ff_moe_verify(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                   uint32_t tokens, const uint32_t *ids, uint16_t *partials, void *stream,
                   const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    if (!check_rows(ctx, x, xStride, tokens, error)) return false;
    if (!ids || !partials) return fail(error, "null argument");
    if (tokens > (uint32_t)kMaxGemvRows)
        return fail(error, std::to_string(tokens) + " pairs for one expert");
    ctx->lastTokens = tokens;
    return launch_block_small(ctx, *c.L, x, xStride, tokens, ids, nullptr, false, false, nullptr,
                              partials, nullptr, nullptr, c.stream, error);
}

bool ff_moe_prefill(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                    uint32_t tokens, const uint32_t *ids, uint16_t *partials, void *stream,
                    const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    if (!check_rows(ctx, x, xStride, tokens, error)) return false;
    if (!ids || !partials) return fail(error, "null argument");
    ctx->lastTokens = tokens > (uint32_t)kMaxGemvRows ? tokens : kMaxGemvRows + 1;
    return launch_prefill_routed(ctx, *c.L, x, xStride, tokens, ids, partials, c.stream, error);
}

bool ff_moe_reduce(FFContext *ctx, const uint16_t *partials, const uint16_t *weights,
                   const uint16_t *residual, uint16_t *y, uint32_t tokens, void *stream,
                   const char **error) {
    Call c;
    if (!begin(ctx, 0, stream, error, &c)) return false;
    if (!partials || !weights || !y) return fail(error, "null argument");
    if (tokens > ctx->cfg.maxTokens) return fail(error, "rows exceed the context's maxTokens");
    // the kernel reads and writes pairs of 16-bit values as 32-bit words
    if ((reinterpret_cast<uintptr_t>(partials) & 3u) || (reinterpret_cast<uintptr_t>(y) & 3u) ||
        (reinterpret_cast<uintptr_t>(residual) & 3u) || (reinterpret_cast<uintptr_t>(weights) & 1u) || ctx->cfg.d % 2)
        return fail(error, "partials, residual and output rows must be 4-byte aligned");
    return launch_reduce(ctx, partials, weights, residual, y, tokens, c.stream, error);
}

bool ff_moe_reduce_indexed(FFContext *ctx, const uint16_t *partials, const uint32_t *rowIndex,
                           const uint16_t *weights, const uint16_t *residual, uint16_t *y, uint32_t tokens,
                           void *stream, const char **error) {
    Call c;
    if (!begin(ctx, 0, stream, error, &c)) return false;
    if (!partials || !rowIndex || !weights || !y) return fail(error, "null argument");
    if (tokens > ctx->cfg.maxTokens) return fail(error, "rows exceed the context's maxTokens");
    if ((reinterpret_cast<uintptr_t>(partials) & 3u) || (reinterpret_cast<uintptr_t>(y) & 3u) ||
        (reinterpret_cast<uintptr_t>(residual) & 3u) || (reinterpret_cast<uintptr_t>(rowIndex) & 3u) ||
        (reinterpret_cast<uintptr_t>(weights) & 1u) || ctx->cfg.d % 2)
        return fail(error, "partials, residual, output rows and the row index must be 4-byte aligned");
    return launch_reduce(ctx, partials, weights, residual, y, tokens, c.stream, error, rowIndex);
}

bool ff_shared_ffn(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t xStride,
                   uint32_t tokens, uint16_t *y, void *stream, const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    if (!check_rows(ctx, x, xStride, tokens, error)) return false;
    if (!y) return fail(error, "output pointer is null");
    if (c.L->has_shared8()) return launch_shared_int8(ctx, *c.L, x, xStride, tokens, y, c.stream, error);
    // one row goes through the decode kernel (shared part only), so that the layer call and the
    // operators called one by one give the same bits
    if (tokens == 1 && ((uintptr_t)x & 15) == 0)
        return launch_decode_fused(ctx, *c.L, x, nullptr, nullptr, true, false, nullptr, y, c.stream, error);
    if (tokens <= (uint32_t)kMaxGemvRows)
        return launch_shared_small(ctx, *c.L, x, xStride, tokens, y, c.stream, error);
    return launch_prefill_shared(ctx, *c.L, x, xStride, tokens, y, c.stream, error);
}

bool ff_int4_gemv_rows(FFContext *ctx, const FFProjection *projection, const uint16_t *x,
                       uint32_t xStride, uint32_t rows, uint16_t *y, uint32_t yStride,
                       void *stream, const char **error) {
    Call c;
    if (!begin(ctx, 0, stream, error, &c)) return false;
    if (!projection || !x || !y) return fail(error, "null argument");
    if (xStride < projection->cols || yStride < projection->rows)
        return fail(error, "row stride is too small");
    if (xStride % 2 || (reinterpret_cast<uintptr_t>(x) & 3u))
        return fail(error, "input rows must be 4-byte aligned (even stride)");
    if (reinterpret_cast<uintptr_t>(y) & 1u) return fail(error, "output rows must be 2-byte aligned");
    if (!projection->weights || !projection->scales || !projection->biases ||
        (reinterpret_cast<uintptr_t>(projection->scales) & 1u) || (reinterpret_cast<uintptr_t>(projection->biases) & 1u))
        return fail(error, "projection pointers must be non-null, scales and biases 2-byte aligned");
    return launch_gemv_rows(ctx, *projection, x, xStride, rows, y, yStride, c.stream, error);
}

bool ff_rmsnorm(FFContext *ctx, const uint16_t *x, const uint16_t *w, float eps, uint32_t tokens,
                uint16_t *y, void *stream, const char **error) {
    Call c;
    if (!begin(ctx, 0, stream, error, &c)) return false;
    if (!x || !y) return fail(error, "null argument");
    if ((reinterpret_cast<uintptr_t>(x) & 1u) || (reinterpret_cast<uintptr_t>(y) & 1u) ||
        (reinterpret_cast<uintptr_t>(w) & 1u))
        return fail(error, "rows must be 2-byte aligned");
    return launch_rmsnorm(ctx, x, w, eps, tokens, y, c.stream, error);
}

bool ff_moe_layer(FFContext *ctx, uint32_t layer, const uint16_t *x, uint32_t tokens,
                  uint16_t *y, uint32_t *ids, uint16_t *weights, void *stream,
                  const char **error) {
    Call c;
    if (!begin(ctx, layer, stream, error, &c)) return false;
    const FFConfig &cfg = ctx->cfg;
    if (!check_rows(ctx, x, cfg.d, tokens, error)) return false;
    if (!y) return fail(error, "output pointer is null");
    if (tokens == 0) return true;
    LayerStore &L = *c.L;
    // an INT8 shared FFN runs as launches of its own in front; its rows are then the residual that
    // the routed part is added to (the INT4 one is part of the fused kernels)
    const bool shared8 = cfg.sharedF != 0 && L.has_shared8();
    const bool withShared = cfg.sharedF != 0 && L.shared != nullptr && !shared8;
    ctx->lastTokens = tokens;
    const size_t routeCount = (size_t)tokens * cfg.topK;
    bool ok = true;
    if (shared8) ok = launch_shared_int8(ctx, L, x, cfg.d, tokens, ctx->h1, c.stream, error);
    const uint16_t *sharedRows = (withShared || shared8) ? ctx->h1 : nullptr;
    if (!ok) return false;
    if (tokens <= (uint32_t)kMaxGemvRows) {
        const bool decode = tokens == 1;
        ok = launch_block_small(ctx, L, x, cfg.d, tokens, nullptr, nullptr, withShared, decode,
                                shared8 ? ctx->h1 : nullptr, ctx->partials, ctx->h1, y, c.stream, error);
        if (ok && !decode)
            ok = launch_reduce(ctx, ctx->partials, ctx->weights, sharedRows, y, tokens, c.stream, error);
    } else {
        ok = launch_router_topk(ctx, L, x, cfg.d, tokens, ctx->ids, ctx->weights, nullptr, c.stream,
                                error);
        if (ok && withShared)
            ok = launch_prefill_shared(ctx, L, x, cfg.d, tokens, ctx->h1, c.stream, error);
        ok = ok && launch_prefill_routed(ctx, L, x, cfg.d, tokens, ctx->ids, ctx->partials, c.stream,
                                         error);
        ok = ok && launch_reduce(ctx, ctx->partials, ctx->weights, sharedRows, y, tokens, c.stream, error);
    }
    if (!ok) return false;
    if (ids)
        FF_CUDA_OK(cudaMemcpyAsync(ids, ctx->ids, routeCount * sizeof(uint32_t),
                                   cudaMemcpyDeviceToDevice, c.stream),
                   error);
    if (weights)
        FF_CUDA_OK(cudaMemcpyAsync(weights, ctx->weights, routeCount * sizeof(uint16_t),
                                   cudaMemcpyDeviceToDevice, c.stream),
                   error);
    return true;
}

// A stack of MoE blocks with an RMSNorm (no weight) in front of each: x <- block_l(rmsnorm(x)).
bool ff_moe_stack(FFContext *ctx, uint32_t firstLayer, uint32_t layerCount, const uint16_t *x,
                  uint32_t tokens, float eps, uint16_t *y, uint32_t *ids, void *stream,
                  const char **error) {
    Call c;
    if (!begin(ctx, firstLayer, stream, error, &c)) return false;
    const FFConfig &cfg = ctx->cfg;
    if (layerCount == 0 || firstLayer + layerCount > cfg.layers)
        return fail(error, "layers " + std::to_string(firstLayer) + "..+" + std::to_string(layerCount) +
                               " are out of range");
    if (!check_rows(ctx, x, cfg.d, tokens, error)) return false;
    if (!y || (reinterpret_cast<uintptr_t>(y) & 15u)) return fail(error, "output rows must be non-null and 16-byte aligned");
    if (tokens == 0) return true;
    const uint16_t *cur = x;
    const size_t routeCount = (size_t)tokens * cfg.topK;
    for (uint32_t i = 0; i < layerCount; ++i) {
        if (!launch_rmsnorm(ctx, cur, nullptr, eps, tokens, ctx->xDev, c.stream, error)) return false;
        uint16_t *out = i + 1 == layerCount ? y : ctx->yDev;
        if (!ff_moe_layer(ctx, firstLayer + i, ctx->xDev, tokens, out, ids ? ids + i * routeCount : nullptr,
                          nullptr, stream, error))
            return false;
        cur = out;
    }
    return true;
}

bool ff_reset_device_error(FFContext *ctx, const char **error) {
    if (error) *error = nullptr;
    if (!ctx) return fail(error, "null context");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    FF_CUDA_OK(cudaDeviceSynchronize(), error);
    FF_CUDA_OK(cudaMemset(ctx->errorFlag, 0, sizeof(uint32_t)), error);
    return true;
}

// One token with host buffers, without copies around the kernel: the input row travels in the
// kernel parameters, the last CTA writes the output straight into the caller's pinned buffer and
// reports through a mailbox in pinned memory that the host polls.  Returns false (with *handled
// false) when the fast path does not apply.
static bool moe_layer_host_one_token(FFContext *ctx, uint32_t layer, const uint16_t *hostX, uint16_t *hostY,
                                     bool *handled, const char **error) {
    *handled = false;
    const FFConfig &cfg = ctx->cfg;
    if (layer >= cfg.layers || cfg.d > 4096 || !ctx->mailbox) return true;
    LayerStore &L = ctx->layers[layer];
    if (!L.experts || !L.routerW || L.has_shared8()) return true;
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, hostY) != cudaSuccess) {
        cudaGetLastError();
        return true;
    }
    if (attr.type != cudaMemoryTypeHost || !attr.devicePointer || ((uintptr_t)attr.devicePointer & 15)) return true;
    *handled = true;
    const bool withShared = cfg.sharedF != 0 && L.shared != nullptr;
    ctx->lastTokens = 1;
    DecodeHostHandoff handoff{hostX, static_cast<uint16_t *>(attr.devicePointer),
                              const_cast<unsigned long long *>(ctx->mailbox), ++ctx->hostEpoch};
    if (handoff.epoch == 0) handoff.epoch = ++ctx->hostEpoch;  // 0 is the mailbox's initial value
    if (!launch_decode_fused(ctx, L, ctx->xDev, nullptr, nullptr, withShared, true, nullptr, ctx->yDev,
                             ctx->hostStream, error, &handoff))
        return false;
    // poll the mailbox; look at the stream now and then so that a failed launch cannot spin forever
    unsigned long long word = 0;
    for (uint64_t spins = 1;; ++spins) {
        word = *ctx->mailbox;
        if ((uint32_t)word == handoff.epoch) break;
        if ((spins & 0xFFFF) == 0) {
            const cudaError_t state = cudaStreamQuery(ctx->hostStream);
            if (state == cudaSuccess) {
                word = *ctx->mailbox;
                if ((uint32_t)word == handoff.epoch) break;
                return fail(error, "the decode kernel ended without reporting");
            }
            if (state != cudaErrorNotReady) return fail(error, std::string("CUDA: ") + cudaGetErrorString(state));
        }
    }
    const uint32_t flag = (uint32_t)(word >> 32);
    if (flag) return fail(error, "a kernel gave up waiting (error flag " + std::to_string(flag) + ")");
    return true;
}

bool ff_post_attn_setup(FFContext *ctx, uint16_t *hidden, const uint16_t *attn, const uint16_t *wPostAttn,
                        const uint16_t *wPreFfn, const uint16_t *wPreFfn2, uint32_t tokens, float eps,
                        uint16_t *denseX, uint16_t *routedX, uint16_t *routerX, void *stream,
                        const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !hidden || !attn || !wPostAttn || !wPreFfn || !wPreFfn2 || !denseX || !routedX || !routerX)
        return fail(error, "null argument");
    const uintptr_t all = reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(attn) |
                          reinterpret_cast<uintptr_t>(wPostAttn) | reinterpret_cast<uintptr_t>(wPreFfn) |
                          reinterpret_cast<uintptr_t>(wPreFfn2) | reinterpret_cast<uintptr_t>(denseX) |
                          reinterpret_cast<uintptr_t>(routedX) | reinterpret_cast<uintptr_t>(routerX);
    if (all & 1u) return fail(error, "rows must be 2-byte aligned");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    return launch_post_attn_setup(ctx, hidden, attn, wPostAttn, wPreFfn, wPreFfn2, eps, tokens, denseX, routedX,
                                  routerX, static_cast<cudaStream_t>(stream), error);
}

bool ff_layer_tail(FFContext *ctx, const uint16_t *h2, const uint16_t *h1, uint16_t *hidden,
                   const uint16_t *wPostFfn2, const uint16_t *wPostFfn, uint32_t tokens, float eps,
                   float layerScalar, void *stream, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !h2 || !h1 || !hidden || !wPostFfn2 || !wPostFfn) return fail(error, "null argument");
    const uintptr_t all = reinterpret_cast<uintptr_t>(h2) | reinterpret_cast<uintptr_t>(h1) |
                          reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(wPostFfn2) |
                          reinterpret_cast<uintptr_t>(wPostFfn);
    if (all & 1u) return fail(error, "rows must be 2-byte aligned");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    return launch_layer_tail(ctx, h2, h1, hidden, wPostFfn2, wPostFfn, eps, layerScalar, tokens,
                             static_cast<cudaStream_t>(stream), error);
}

bool ff_sort_routes(FFContext *ctx, const uint32_t *groupIds, uint32_t tokens, uint32_t groups,
                    FFTokenExpertPair *sortedPairs, uint32_t *offsets, cudaStream_t stream, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !groupIds || !sortedPairs || !offsets) return fail(error, "null argument");
    if ((reinterpret_cast<uintptr_t>(sortedPairs) & 15u) || (reinterpret_cast<uintptr_t>(groupIds) & 3u) ||
        (reinterpret_cast<uintptr_t>(offsets) & 3u))
        return fail(error, "sorted pairs must be 16-byte aligned, ids and offsets 4-byte aligned");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    return launch_route_sort(ctx, groupIds, tokens, groups, sortedPairs, offsets, stream, error);
}

bool ff_moe_layer_host(FFContext *ctx, uint32_t layer, const uint16_t *hostX, uint32_t tokens,
                       uint16_t *hostY, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !hostX || !hostY) return fail(error, "null argument");
    if (tokens > ctx->cfg.maxTokens) return fail(error, "rows exceed the context's maxTokens");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    if (tokens == 1) {
        bool handled = false;
        const bool ok = moe_layer_host_one_token(ctx, layer, hostX, hostY, &handled, error);
        if (handled || !ok) return ok;
    }
    const size_t bytes = (size_t)tokens * ctx->cfg.d * sizeof(uint16_t);
    FF_CUDA_OK(cudaMemcpyAsync(ctx->xDev, hostX, bytes, cudaMemcpyHostToDevice, ctx->hostStream), error);
    if (!ff_moe_layer(ctx, layer, ctx->xDev, tokens, ctx->yDev, nullptr, nullptr, ctx->hostStream, error))
        return false;
    FF_CUDA_OK(cudaMemcpyAsync(hostY, ctx->yDev, bytes, cudaMemcpyDeviceToHost, ctx->hostStream), error);
    FF_CUDA_OK(cudaStreamSynchronize(ctx->hostStream), error);
    uint32_t flag = 0;
    FF_CUDA_OK(cudaMemcpy(&flag, ctx->errorFlag, sizeof(flag), cudaMemcpyDeviceToHost), error);
    if (flag) return fail(error, "a kernel gave up waiting (error flag " + std::to_string(flag) + ")");
    return true;
}

}  // extern "C"
