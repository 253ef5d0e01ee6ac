// Context lifetime, the HBM-resident weight store, and the host-side pair grouping.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "ff_internal.cuh"

namespace ff {

bool fail(const char **error, const std::string &message) {
    if (error) *error = strdup(message.c_str());
    return false;
}

// Gate, up, down back to back, each as packed codes, scales, biases: the order the reference's
// installer writes (Sources/ANEFieldfareInstallCore/Planning/RepackPlanner.swift:438-490).
FFExpertOffsets packed_offsets(uint32_t d, uint32_t f, uint64_t *payload) {
    const uint32_t w = d * f / 2, s = d * f / kGroup * 2;
    FFExpertOffsets o{};
    uint32_t cursor = 0;
    uint32_t *fields = &o.gateWOff;
    for (int m = 0; m < 3; ++m) {
        fields[3 * m + 0] = cursor;
        fields[3 * m + 1] = cursor + w;
        fields[3 * m + 2] = cursor + w + s;
        cursor += w + 2 * s;
    }
    if (payload) *payload = cursor;
    return o;
}

template <typename T>
static bool dev_alloc(FFContext *ctx, T **ptr, size_t count, const char **error) {
    if (count == 0) count = 1;
    cudaError_t st = cudaMalloc(reinterpret_cast<void **>(ptr), count * sizeof(T));
    if (st != cudaSuccess)
        return fail(error, "cudaMalloc of " + std::to_string(count * sizeof(T)) +
                               " bytes failed: " + cudaGetErrorString(st));
    ctx->scratchBytes += count * sizeof(T);
    return true;
}

static void free_shared8(LayerStore &L) {
    for (int m = 0; m < 3; ++m) {
        cudaFree(L.shared8W[m]);
        cudaFree(L.shared8S[m]);
        cudaFree(L.shared8B[m]);
        L.shared8W[m] = nullptr;
        L.shared8S[m] = L.shared8B[m] = nullptr;
    }
}

static void free_layer(LayerStore &L) {
    cudaFree(L.experts);
    cudaFree(L.shared);
    free_shared8(L);
    cudaFree(L.routerQ);
    cudaFree(L.routerQScale);
    cudaFree(L.routerQBias);
    cudaFree(L.routerW);
    cudaFree(L.routerScale);
    cudaFree(L.gain);
    cudaFree(L.logitBias);
    L = LayerStore{};
}

}  // namespace ff

using namespace ff;

extern "C" {

void ff_string_free(const char *message) { free(const_cast<char *>(message)); }

void ff_destroy(FFContext *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    for (auto &L : ctx->layers) free_layer(L);
    void *ptrs[] = {ctx->logits, ctx->ids, ctx->weights, ctx->plan, ctx->jobs[0], ctx->jobs[1],
                    ctx->acts, ctx->sharedActs, ctx->h1,
                    ctx->partials, ctx->xDev, ctx->yDev, ctx->xSorted, ctx->sortedPairs,
                    ctx->expertOffsets, ctx->blockCounts, ctx->units, ctx->unitCount,
                    ctx->errorFlag, ctx->gridBarrier, ctx->phaseStamps, ctx->mapScratch, ctx->taggedLogits, ctx->taggedActs,
                    ctx->logitsRows, ctx->routeIds, ctx->routeWeights};
    for (void *p : ptrs) cudaFree(p);
    if (ctx->hostStream) cudaStreamDestroy(ctx->hostStream);
    if (ctx->mailbox) cudaFreeHost(const_cast<unsigned long long *>(ctx->mailbox));
    delete ctx;
}

FFContext *ff_create(int32_t deviceOrdinal, const FFConfig *config, const char **error) {
    if (error) *error = nullptr;
    if (!config) {
        fail(error, "config is null");
        return nullptr;
    }
    const FFConfig c = *config;
    if (c.layers == 0 || c.experts == 0 || c.experts > (uint32_t)kMaxExperts || c.topK == 0 ||
        c.topK > 8 || c.topK > c.experts || c.maxTokens == 0) {
        fail(error, "unsupported configuration: need 1..256 experts, topK in 1..8, maxTokens > 0");
        return nullptr;
    }
    if (c.d % kGroup || c.f % kGroup || c.sharedF % kGroup || c.d == 0 || c.f == 0) {
        fail(error, "d, f and sharedF must be multiples of the group size 64");
        return nullptr;
    }
    int count = 0;
    cudaError_t st = cudaGetDeviceCount(&count);
    if (st != cudaSuccess || count == 0) {
        fail(error, std::string("no CUDA device: ") +
                        (st != cudaSuccess ? cudaGetErrorString(st) : "device count is 0"));
        return nullptr;
    }
    if (deviceOrdinal < 0 || deviceOrdinal >= count) {
        fail(error, "device ordinal " + std::to_string(deviceOrdinal) + " out of range");
        return nullptr;
    }
    st = cudaSetDevice(deviceOrdinal);
    if (st != cudaSuccess) {
        fail(error, std::string("cudaSetDevice: ") + cudaGetErrorString(st));
        return nullptr;
    }
    cudaDeviceProp prop{};
    cudaGetDeviceProperties(&prop, deviceOrdinal);
    if (prop.major != 10) {
        fail(error, "this library is built for sm_100a only; device is sm_" +
                        std::to_string(prop.major) + std::to_string(prop.minor));
        return nullptr;
    }
    FFContext *ctx = new FFContext();
    ctx->device = deviceOrdinal;
    ctx->smCount = prop.multiProcessorCount;
    ctx->cfg = c;
    ctx->layers.resize(c.layers);
    const size_t T = c.maxTokens, K = c.topK;
    const size_t smallT = std::min<size_t>(T, kMaxGemvRows);
    const size_t planExperts = std::min<size_t>(c.experts, kMaxGemvRows * K);
    bool ok = cudaStreamCreateWithFlags(&ctx->hostStream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && dev_alloc(ctx, &ctx->logits, smallT * kMaxExperts, error);
    ok = ok && dev_alloc(ctx, &ctx->ids, T * K, error);
    ok = ok && dev_alloc(ctx, &ctx->weights, T * K, error);
    ok = ok && dev_alloc(ctx, &ctx->plan, 1, error);
    ok = ok && dev_alloc(ctx, &ctx->jobs[0], 1 + planExperts, error);
    ok = ok && dev_alloc(ctx, &ctx->jobs[1], 1 + planExperts, error);
    ok = ok && dev_alloc(ctx, &ctx->acts, (T * K + 256) * c.f, error);  // +256: a GEMM row tile may overhang
    ok = ok && dev_alloc(ctx, &ctx->sharedActs, (T + 256) * c.sharedF, error);
    ok = ok && dev_alloc(ctx, &ctx->h1, T * c.d, error);
    ok = ok && dev_alloc(ctx, &ctx->partials, T * K * c.d, error);
    ok = ok && dev_alloc(ctx, &ctx->xDev, T * c.d, error);
    ok = ok && dev_alloc(ctx, &ctx->yDev, T * c.d, error);
    ok = ok && dev_alloc(ctx, &ctx->errorFlag, 4, error);
    if (ok) ok = cudaMemset(ctx->errorFlag, 0, 16) == cudaSuccess;
    ok = ok && dev_alloc(ctx, &ctx->phaseStamps, kPhaseStampSlots, error);
    if (ok) ok = cudaMemset(ctx->phaseStamps, 0, kPhaseStampSlots * 8) == cudaSuccess;
    ok = ok && dev_alloc(ctx, &ctx->taggedLogits, kMaxExperts, error);
    if (ok) ok = cudaMemset(ctx->taggedLogits, 0, kMaxExperts * 8) == cudaSuccess;
    const size_t taggedWords = (size_t)K * c.f / 2 + c.d / 2;
    ok = ok && dev_alloc(ctx, &ctx->taggedActs, taggedWords, error);
    if (ok) ok = cudaMemset(ctx->taggedActs, 0, taggedWords * 8) == cudaSuccess;
    ok = ok && dev_alloc(ctx, &ctx->gridBarrier, 16, error);
    if (ok) ok = cudaMemset(ctx->gridBarrier, 0, 64) == cudaSuccess;
    if (ok) {
        void *box = nullptr;
        ok = cudaHostAlloc(&box, 64, cudaHostAllocMapped) == cudaSuccess;
        if (ok) {
            memset(box, 0, 64);
            ctx->mailbox = static_cast<volatile unsigned long long *>(box);
        } else if (error) {
            fail(error, "cudaHostAlloc of the host mailbox failed");
        }
    }
    if (ok && T > (size_t)kMaxGemvRows) {
        const size_t pairs = T * K;
        const size_t permuteBlocks = (T + 255) / 256;
        // one work unit per (expert, 128-row tile, column tile); tiles <= pairs/128 + experts
        ctx->maxUnits = (uint32_t)(2 * (pairs / 128 + c.experts + 2));  // row tiles: routed half, dense half
        ok = ok && dev_alloc(ctx, &ctx->xSorted, (pairs + 256) * c.d, error);
        if (ok) ok = cudaMemset(ctx->xSorted, 0, (pairs + 256) * c.d * 2) == cudaSuccess;
        ok = ok && dev_alloc(ctx, &ctx->sortedPairs, pairs, error);
        ok = ok && dev_alloc(ctx, &ctx->expertOffsets, c.experts + 1, error);
        ok = ok && dev_alloc(ctx, &ctx->blockCounts, (permuteBlocks + 1) * c.experts, error);
        ok = ok && dev_alloc(ctx, &ctx->units, (size_t)ctx->maxUnits * 4, error);
        ok = ok && dev_alloc(ctx, &ctx->unitCount, 8, error);
        if (ok) ok = cudaMemset(ctx->unitCount, 0, 32) == cudaSuccess;
    }
    if (!ok) {
        if (error && !*error) fail(error, "context allocation failed");
        ff_destroy(ctx);
        return nullptr;
    }
    return ctx;
}

FFInfo ff_get_info(const FFContext *ctx) {
    FFInfo info{};
    if (!ctx) return info;
    info.kernelLaunches = ctx->kernelLaunches;
    info.weightBytesResident = ctx->weightBytes;
    info.scratchBytes = ctx->scratchBytes;
    info.deviceOrdinal = (uint32_t)ctx->device;
    info.smCount = (uint32_t)ctx->smCount;
    cudaSetDevice(ctx->device);
    RoutePlan plan{};
    if (ctx->plan && cudaMemcpy(&plan, ctx->plan, sizeof(plan), cudaMemcpyDeviceToHost) == cudaSuccess)
        info.lastActiveExperts = plan.activeExperts;
    if (ctx->errorFlag)
        cudaMemcpy(&info.deviceErrorFlag, ctx->errorFlag, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    uint32_t counts[4] = {0, 0, 0, 0};
    if (ctx->unitCount &&
        cudaMemcpy(counts, ctx->unitCount, sizeof(counts), cudaMemcpyDeviceToHost) == cudaSuccess) {
        info.lastPrefillUnits = counts[0];
        if (ctx->lastTokens > (uint32_t)kMaxGemvRows) info.lastActiveExperts = counts[2];
    }
    return info;
}

void ff_set_tracing(FFContext *ctx, bool enabled) {
    if (ctx) ctx->tracing = enabled;
}

bool ff_decode_phase_times(FFContext *ctx, double *microseconds, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !microseconds) return fail(error, "null argument");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    FF_CUDA_OK(cudaDeviceSynchronize(), error);
    unsigned long long t[8] = {0};
    FF_CUDA_OK(cudaMemcpy(t, ctx->phaseStamps, sizeof(t), cudaMemcpyDeviceToHost), error);
    for (int i = 0; i < 6; ++i) microseconds[i] = t[i + 1] >= t[i] ? (double)(t[i + 1] - t[i]) * 1e-3 : 0.0;
    return true;
}

bool ff_decode_warp_times(FFContext *ctx, double *microseconds, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !microseconds) return fail(error, "null argument");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    FF_CUDA_OK(cudaDeviceSynchronize(), error);
    std::vector<unsigned long long> t(kPhaseStampSlots, 0);
    FF_CUDA_OK(cudaMemcpy(t.data(), ctx->phaseStamps, t.size() * sizeof(t[0]), cudaMemcpyDeviceToHost), error);
    for (int i = 8; i < kPhaseStampSlots; ++i)
        microseconds[i - 8] = t[i] >= t[0] && t[0] ? (double)(t[i] - t[0]) * 1e-3 : -1.0;
    FF_CUDA_OK(cudaMemset(ctx->phaseStamps + 8, 0, (kPhaseStampSlots - 8) * sizeof(t[0])), error);
    return true;
}

uint32_t ff_get_trace(FFContext *ctx, FFTraceEntry *entries, uint32_t capacity) {
    if (!ctx) return 0;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    uint32_t count = 0;
    for (auto &rec : ctx->trace) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, rec.begin, rec.end);
        cudaEventDestroy(rec.begin);
        cudaEventDestroy(rec.end);
        uint32_t i = 0;
        for (; i < count; ++i)
            if (strncmp(entries[i].name, rec.name, sizeof(entries[i].name) - 1) == 0) break;
        if (i == count) {
            if (count == capacity) continue;
            memset(&entries[i], 0, sizeof(FFTraceEntry));
            strncpy(entries[i].name, rec.name, sizeof(entries[i].name) - 1);
            ++count;
        }
        entries[i].launches++;
        entries[i].milliseconds += ms;
    }
    ctx->trace.clear();
    return count;
}

bool ff_load_layer(FFContext *ctx, uint32_t layer, const void *hostBytes, uint64_t byteCount,
                   uint32_t expertCount, uint64_t expertStride, const FFExpertOffsets *offsets,
                   const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !hostBytes || !offsets) return fail(error, "null argument");
    if (layer >= ctx->cfg.layers) return fail(error, "layer " + std::to_string(layer) + " out of range");
    if (expertCount != ctx->cfg.experts)
        return fail(error, "routed layer " + std::to_string(layer) + " has " +
                               std::to_string(expertCount) + " experts, context expects " +
                               std::to_string(ctx->cfg.experts));
    const uint32_t d = ctx->cfg.d, f = ctx->cfg.f;
    const uint64_t wSize = (uint64_t)d * f / 2, auxSize = (uint64_t)d * f / kGroup * 2;
    const uint32_t *o = &offsets->gateWOff;
    const char *roles[3] = {"gate", "up", "down"};
    uint64_t payload = 0;
    for (int m = 0; m < 3; ++m) {
        const uint64_t w = o[3 * m], s = o[3 * m + 1], b = o[3 * m + 2];
        // Runtime/Inference/Model.swift:494-517: weights 4-byte aligned, scales/biases 2-byte
        // aligned, every sub-tensor inside the blob.  The 128-bit loads need 16 bytes.
        if (w % 4 || s % 2 || b % 2)
            return fail(error, "routed layer " + std::to_string(layer) + " role " + roles[m] +
                                   " does not match the required schema");
        if (w % 16)
            return fail(error, "routed layer " + std::to_string(layer) + " role " + roles[m] +
                                   " weights are not 16-byte aligned (needed by 128-bit loads)");
        payload = std::max({payload, w + wSize, s + auxSize, b + auxSize});
    }
    if (payload > expertStride || expertStride % 16)
        return fail(error, "routed layer " + std::to_string(layer) +
                               " expert stride is smaller than the sub-tensors or not 16-byte aligned");
    if (byteCount < (uint64_t)(expertCount - 1) * expertStride + payload)
        return fail(error, "routed layer " + std::to_string(layer) + " file is truncated");
    if ((d / 2) % 16 || (f / 2) % 16)
        return fail(error, "row bytes must be multiples of 16");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    LayerStore &L = ctx->layers[layer];
    if (L.experts) {
        ctx->weightBytes -= L.stride * L.expertCount;
        cudaFree(L.experts);
        L.experts = nullptr;
    }
    const uint64_t total = (uint64_t)expertCount * expertStride;
    // 256 bytes of slack: the decode kernel fetches 16-byte aligned windows around scale rows
    FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&L.experts), total + 256), error);
    FF_CUDA_OK(cudaMemset(L.experts, 0, total), error);
    FF_CUDA_OK(cudaMemcpy(L.experts, hostBytes, std::min(byteCount, total), cudaMemcpyHostToDevice),
               error);
    L.stride = expertStride;
    L.expertCount = expertCount;
    L.off = *offsets;
    L.mapsReady = false;
    L.decodeMapsReady = false;
    ctx->weightBytes += total;
    return true;
}

static bool check_projection(const FFProjection *p, uint32_t rows, uint32_t cols, const char *name,
                             const char **error) {
    if (!p || !p->weights || !p->scales || !p->biases)
        return fail(error, std::string("SharedExpert ") + name + " projection is null");
    if (p->rows != rows || p->cols != cols)
        return fail(error, std::string("SharedExpert dimension mismatch: ") + name + "=(" +
                               std::to_string(p->rows) + "," + std::to_string(p->cols) + ")");
    return true;
}

bool ff_load_shared(FFContext *ctx, uint32_t layer, const FFProjection *gate,
                    const FFProjection *up, const FFProjection *down, const char **error) {
    if (error) *error = nullptr;
    if (!ctx) return fail(error, "null context");
    if (layer >= ctx->cfg.layers) return fail(error, "layer " + std::to_string(layer) + " out of range");
    const uint32_t d = ctx->cfg.d, fs = ctx->cfg.sharedF;
    if (fs == 0) return fail(error, "context was created without a shared FFN");
    if (!check_projection(gate, fs, d, "gate", error) || !check_projection(up, fs, d, "up", error) ||
        !check_projection(down, d, fs, "down", error))
        return false;
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    LayerStore &L = ctx->layers[layer];
    free_shared8(L);
    uint64_t payload = 0;
    L.sharedOff = packed_offsets(d, fs, &payload);
    if (L.shared) {
        cudaFree(L.shared);
        L.shared = nullptr;
        ctx->weightBytes -= payload;
    }
    FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&L.shared), payload), error);
    const uint64_t wSize = (uint64_t)d * fs / 2, auxSize = (uint64_t)d * fs / kGroup * 2;
    const FFProjection *ps[3] = {gate, up, down};
    const uint32_t *o = &L.sharedOff.gateWOff;
    for (int m = 0; m < 3; ++m) {
        FF_CUDA_OK(cudaMemcpy(L.shared + o[3 * m], ps[m]->weights, wSize, cudaMemcpyHostToDevice), error);
        FF_CUDA_OK(cudaMemcpy(L.shared + o[3 * m + 1], ps[m]->scales, auxSize, cudaMemcpyHostToDevice), error);
        FF_CUDA_OK(cudaMemcpy(L.shared + o[3 * m + 2], ps[m]->biases, auxSize, cudaMemcpyHostToDevice), error);
    }
    L.mapsReady = false;
    L.decodeMapsReady = false;
    ctx->weightBytes += payload;
    return true;
}

static void free_router(ff::LayerStore &L) {
    cudaFree(L.routerW);
    cudaFree(L.routerScale);
    cudaFree(L.gain);
    cudaFree(L.logitBias);
    cudaFree(L.routerQ);
    cudaFree(L.routerQScale);
    cudaFree(L.routerQBias);
    L.routerW = L.routerScale = L.gain = L.routerQScale = L.routerQBias = nullptr;
    L.routerQ = nullptr;
    L.logitBias = nullptr;
}

static bool upload(void **dst, const void *src, size_t bytes, const char **error) {
    FF_CUDA_OK(cudaMalloc(dst, bytes), error);
    FF_CUDA_OK(cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice), error);
    return true;
}

bool ff_load_shared_int8(FFContext *ctx, uint32_t layer, const FFProjection *gate, const FFProjection *up,
                         const FFProjection *down, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !gate || !up || !down) return fail(error, "null argument");
    if (layer >= ctx->cfg.layers) return fail(error, "layer " + std::to_string(layer) + " out of range");
    const uint32_t d = ctx->cfg.d, fs = ctx->cfg.sharedF;
    if (fs == 0) return fail(error, "context was created without a shared FFN");
    if (d % 64 || fs % 64) return fail(error, "widths must be multiples of the group size 64");
    const FFProjection *ps[3] = {gate, up, down};
    const uint32_t wantRows[3] = {fs, fs, d}, wantCols[3] = {d, d, fs};
    for (int m = 0; m < 3; ++m) {
        if (!ps[m]->weights || !ps[m]->scales || !ps[m]->biases) return fail(error, "null projection tensor");
        if (ps[m]->rows != wantRows[m] || ps[m]->cols != wantCols[m])
            return fail(error, "SharedExpert dimension mismatch: gate=(" + std::to_string(gate->rows) + "," +
                                   std::to_string(gate->cols) + ") up=(" + std::to_string(up->rows) + "," +
                                   std::to_string(up->cols) + ") down=(" + std::to_string(down->rows) + "," +
                                   std::to_string(down->cols) + ")");
    }
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    LayerStore &L = ctx->layers[layer];
    if (L.shared) {
        cudaFree(L.shared);
        L.shared = nullptr;
        L.mapsReady = false;
        L.decodeMapsReady = false;
    }
    free_shared8(L);
    for (int m = 0; m < 3; ++m) {
        const size_t codes = (size_t)wantRows[m] * wantCols[m], aux = (size_t)wantRows[m] * (wantCols[m] / 64) * 2;
        if (!upload(reinterpret_cast<void **>(&L.shared8W[m]), ps[m]->weights, codes, error) ||
            !upload(reinterpret_cast<void **>(&L.shared8S[m]), ps[m]->scales, aux, error) ||
            !upload(reinterpret_cast<void **>(&L.shared8B[m]), ps[m]->biases, aux, error))
            return false;
        ctx->weightBytes += codes + 2 * aux;
    }
    return true;
}

bool ff_load_router_int8(FFContext *ctx, uint32_t layer, const uint8_t *codes, const uint16_t *scales,
                         const uint16_t *biases, const uint16_t *effectiveScale,
                         const uint16_t *perExpertScale, const float *logitBias, uint32_t experts,
                         uint32_t d, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !codes || !scales || !biases) return fail(error, "null argument");
    if (layer >= ctx->cfg.layers) return fail(error, "layer " + std::to_string(layer) + " out of range");
    if (d != ctx->cfg.d) return fail(error, "router width does not match the context");
    if (d % 64) return fail(error, "router width must be a multiple of the group size 64");
    if (experts == 0 || experts > (uint32_t)kMaxExperts)
        return fail(error, "numExperts > 256 is not supported");
    if (experts != ctx->cfg.experts)
        return fail(error, "router has " + std::to_string(experts) + " experts, the context expects " +
                               std::to_string(ctx->cfg.experts));
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    LayerStore &L = ctx->layers[layer];
    free_router(L);
    const size_t groups = (size_t)experts * (d / 64);
    if (!upload(reinterpret_cast<void **>(&L.routerQ), codes, (size_t)experts * d, error) ||
        !upload(reinterpret_cast<void **>(&L.routerQScale), scales, groups * 2, error) ||
        !upload(reinterpret_cast<void **>(&L.routerQBias), biases, groups * 2, error))
        return false;
    if (effectiveScale && !upload(reinterpret_cast<void **>(&L.routerScale), effectiveScale, (size_t)d * 2, error))
        return false;
    if (perExpertScale && !upload(reinterpret_cast<void **>(&L.gain), perExpertScale, (size_t)experts * 2, error))
        return false;
    if (logitBias && !upload(reinterpret_cast<void **>(&L.logitBias), logitBias, (size_t)experts * 4, error))
        return false;
    L.routerExperts = experts;
    ctx->weightBytes += (size_t)experts * d + groups * 4;
    // scratch of the INT8 router: logits of every row, and the one-token path's routes
    if (!ctx->logitsRows) {
        FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&ctx->logitsRows),
                              (size_t)ctx->cfg.maxTokens * kMaxExperts * sizeof(float)), error);
        FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&ctx->routeIds), (size_t)ctx->cfg.topK * sizeof(uint32_t)), error);
        FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&ctx->routeWeights), (size_t)ctx->cfg.topK * sizeof(uint16_t)), error);
    }
    return true;
}

bool ff_load_router(FFContext *ctx, uint32_t layer, const uint16_t *weights,
                    const uint16_t *effectiveScale, const uint16_t *perExpertScale,
                    const float *logitBias, uint32_t experts, uint32_t d, const char **error) {
    if (error) *error = nullptr;
    if (!ctx || !weights) return fail(error, "null argument");
    if (layer >= ctx->cfg.layers) return fail(error, "layer " + std::to_string(layer) + " out of range");
    if (d != ctx->cfg.d) return fail(error, "router width does not match the context");
    if (experts == 0 || experts > (uint32_t)kMaxExperts)
        return fail(error, "numExperts > 256 is not supported");
    if (experts != ctx->cfg.experts)
        return fail(error, "router has " + std::to_string(experts) + " experts, the context expects " +
                               std::to_string(ctx->cfg.experts));
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    LayerStore &L = ctx->layers[layer];
    free_router(L);
    const size_t wBytes = (size_t)experts * d * 2;
    FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&L.routerW), wBytes), error);
    FF_CUDA_OK(cudaMemcpy(L.routerW, weights, wBytes, cudaMemcpyHostToDevice), error);
    if (effectiveScale) {
        FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&L.routerScale), (size_t)d * 2), error);
        FF_CUDA_OK(cudaMemcpy(L.routerScale, effectiveScale, (size_t)d * 2, cudaMemcpyHostToDevice), error);
    }
    if (perExpertScale) {
        FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&L.gain), (size_t)experts * 2), error);
        FF_CUDA_OK(cudaMemcpy(L.gain, perExpertScale, (size_t)experts * 2, cudaMemcpyHostToDevice), error);
    }
    if (logitBias) {
        FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&L.logitBias), (size_t)experts * 4), error);
        FF_CUDA_OK(cudaMemcpy(L.logitBias, logitBias, (size_t)experts * 4, cudaMemcpyHostToDevice), error);
    }
    L.routerExperts = experts;
    ctx->weightBytes += wBytes;
    return true;
}

uint64_t ff_expert_address(const FFContext *ctx, uint32_t layer, uint32_t expert) {
    if (!ctx || layer >= ctx->layers.size()) return 0;
    const LayerStore &L = ctx->layers[layer];
    if (!L.experts || expert >= L.expertCount) return 0;
    return reinterpret_cast<uint64_t>(L.experts + (uint64_t)expert * L.stride);
}

// ---- host-side permute ---------------------------------------------------------------------

uint64_t ff_make_token_expert_pairs(const uint32_t *ids, const uint16_t *weights,
                                    uint32_t tokens, uint32_t topK, FFTokenExpertPair *pairs) {
    uint64_t n = 0;
    for (uint32_t t = 0; t < tokens; ++t)
        for (uint32_t r = 0; r < topK; ++r, ++n) {
            const uint64_t i = (uint64_t)t * topK + r;
            pairs[n] = FFTokenExpertPair{t, ids[i], r, weights ? (uint32_t)weights[i] : 0u};
        }
    return n;
}

bool ff_group_token_expert_pairs(const FFTokenExpertPair *pairs, uint64_t pairCount,
                                 uint32_t tokens, uint32_t topK, uint32_t experts,
                                 uint32_t tileExpertCount, const uint64_t *expertSortKeys,
                                 FFTokenExpertPair *sortedPairs, FFMoEGroup *groups,
                                 uint32_t *groupCount, FFMoETile *tiles, uint32_t *tileCount,
                                 const char **error) {
    if (error) *error = nullptr;
    if (topK == 0 || experts == 0 || tileExpertCount < 1 || tileExpertCount > 16)
        return fail(error, "topK and numExperts must be positive and tileExpertCount in 1...16");
    if (pairCount > (uint64_t)tokens * topK) return fail(error, "more pairs than queryCount * topK");
    for (uint64_t i = 0; i < pairCount; ++i)
        if (pairs[i].expert >= experts)
            return fail(error, "route expert " + std::to_string(pairs[i].expert) + " is out of range");
    std::copy(pairs, pairs + pairCount, sortedPairs);
    std::sort(sortedPairs, sortedPairs + pairCount,
              [&](const FFTokenExpertPair &a, const FFTokenExpertPair &b) {
                  if (expertSortKeys) {
                      const uint64_t ka = expertSortKeys[a.expert], kb = expertSortKeys[b.expert];
                      if (ka != kb) return ka < kb;
                  }
                  if (a.expert != b.expert) return a.expert < b.expert;
                  if (a.token != b.token) return a.token < b.token;
                  return a.rank < b.rank;
              });
    uint32_t ng = 0;
    for (uint64_t i = 0; i < pairCount;) {
        uint64_t j = i;
        while (j < pairCount && sortedPairs[j].expert == sortedPairs[i].expert) ++j;
        groups[ng++] = FFMoEGroup{sortedPairs[i].expert, (uint32_t)i, (uint32_t)(j - i)};
        i = j;
    }
    uint32_t nt = 0;
    for (uint32_t g = 0; g < ng; g += tileExpertCount) {
        const uint32_t end = std::min(ng, g + tileExpertCount);
        const FFMoEGroup &first = groups[g], &last = groups[end - 1];
        tiles[nt++] = FFMoETile{g, end - g, first.pairStart,
                                last.pairStart + last.pairCount - first.pairStart};
    }
    *groupCount = ng;
    *tileCount = nt;
    return true;
}

}  // extern "C"
