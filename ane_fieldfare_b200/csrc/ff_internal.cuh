// Internal declarations shared by the translation units of libfieldfare_cuda.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <vector>

#include "fieldfare_cuda.h"

namespace ff {

constexpr int kGroup = 64;        // codes per scale/bias pair
constexpr int kMaxGemvRows = 16;  // input rows one GEMV job can carry (a verify block)
constexpr int kMaxExperts = 256;  // router width limit, as in the reference's prefill router

// ---- error plumbing ------------------------------------------------------------------------

// Stores a strdup'd message in *error (when the caller asked for one) and returns false.
bool fail(const char **error, const std::string &message);

#define FF_CUDA_OK(call, error)                                                              \
    do {                                                                                     \
        cudaError_t ff_status_ = (call);                                                     \
        if (ff_status_ != cudaSuccess)                                                       \
            return ff::fail(error, std::string(#call) + ": " + cudaGetErrorString(ff_status_)); \
    } while (0)

// Per-kernel memo of "dynamic shared-memory limit raised on this device" and of the occupancy at
// the last requested size.  The library's entry points may be called from one host thread per GPU
// (and context-free entry points from any thread), so the memo is guarded by a mutex.
constexpr int kMaxDevices = 64;
class KernelSmemMemo {
public:
    // Makes `kernel` launchable with `smem` bytes of dynamic shared memory on `device` and returns
    // the resident CTAs per SM at (threads, smem) in *perSm (when asked for).
    template <typename Kernel>
    bool prepare(Kernel kernel, int device, size_t smem, int threads, int *perSm, const char **error) {
        if (device < 0 || device >= kMaxDevices) return fail(error, "device ordinal out of range");
        std::lock_guard<std::mutex> guard(lock_);
        Entry &e = entries_[device];
        if (e.limit < smem || !e.touched) {
            FF_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), error);
            e.limit = smem;
            e.touched = true;
        }
        if (perSm) {
            if (e.occSmem != smem || e.occThreads != threads) {
                int n = 0;
                FF_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem), error);
                e.occ = n;
                e.occSmem = smem;
                e.occThreads = threads;
            }
            *perSm = e.occ;
        }
        return true;
    }

private:
    struct Entry {
        size_t limit = 0, occSmem = 0;
        int occ = 0, occThreads = -1;
        bool touched = false;
    };
    std::mutex lock_;
    Entry entries_[kMaxDevices];
};

// ---- work descriptions the kernels read ----------------------------------------------------

// One affine INT4 matrix (or a gate/up pair sharing inputs) applied to up to 16 input rows.
struct GemvJob {
    const uint8_t *w0;   // gate (or the only) matrix: packed codes
    const uint16_t *s0;  // scales
    const uint16_t *b0;  // biases
    const uint8_t *w1;   // up matrix (dual jobs only)
    const uint16_t *s1;
    const uint16_t *b1;
    const uint16_t *in;  // bf16 input rows
    uint16_t *out;       // bf16 output rows
    uint32_t rows;       // weight rows = outputs per input row
    uint32_t cols;       // weight columns = input width
    uint32_t inStride;   // elements between input rows
    uint32_t outStride;  // elements between output rows
    uint32_t n;          // input rows used, 1..16
    uint32_t flags;      // kJobRoundGateUp
    uint32_t inRow[kMaxGemvRows];
    uint32_t outRow[kMaxGemvRows];
};
constexpr uint32_t kJobRoundGateUp = 1u;  // round gate and up to bf16 before the activation

// Output of the device-side route plan for a decode/verify block.
struct RoutePlan {
    uint32_t jobCount[2];    // [0] gate/up jobs, [1] down jobs
    uint32_t itemCount[2];   // (job, row block) work items per phase
    uint32_t activeExperts;  // distinct routed experts in the block
    uint32_t pad[3];
};

struct LayerStore {
    uint8_t *experts = nullptr;  // expertCount blobs, stride apart (a layer file, verbatim)
    uint64_t stride = 0;
    uint32_t expertCount = 0;
    FFExpertOffsets off{};
    uint8_t *shared = nullptr;  // gate, up, down of the shared FFN in the same nine-part order
    FFExpertOffsets sharedOff{};
    uint16_t *routerW = nullptr;
    uint16_t *routerScale = nullptr;
    uint16_t *gain = nullptr;
    float *logitBias = nullptr;
    uint32_t routerExperts = 0;
    // INT8 affine router (the shipped checkpoints' form): codes [experts][d], one bf16 scale and
    // bias per group of 64 inputs; set instead of routerW
    uint8_t *routerQ = nullptr;
    uint16_t *routerQScale = nullptr, *routerQBias = nullptr;
    bool has_router() const { return routerW != nullptr || routerQ != nullptr; }
    // INT8 affine shared FFN (the shipped checkpoints' form): gate, up [sharedF][d] and down
    // [d][sharedF] as codes with one bf16 scale and bias per group of 64; set instead of `shared`
    uint8_t *shared8W[3] = {nullptr, nullptr, nullptr};
    uint16_t *shared8S[3] = {nullptr, nullptr, nullptr}, *shared8B[3] = {nullptr, nullptr, nullptr};
    bool has_shared8() const { return shared8W[0] != nullptr; }
    bool has_shared() const { return shared != nullptr || has_shared8(); }
    // prefill: tensor maps over the packed weights (gate, up, down) of routed and shared blobs
    bool mapsReady = false;
    CUtensorMap routedMap[3];
    CUtensorMap sharedMap[3];
    // one-token kernel: row-box maps of routed gate, routed up, shared gate, shared up, shared down
    bool decodeMapsReady = false;
    CUtensorMap decodeMap[5];
};

}  // namespace ff

constexpr int kPhaseStampSlots = 8 + 2 * 3 * 16 * 3;

struct FFContext {
    int device = 0;
    int smCount = 0;
    FFConfig cfg{};
    std::vector<ff::LayerStore> layers;
    cudaStream_t hostStream = nullptr;  // used by the *_host entry points

    // decode / verify scratch
    float *logits = nullptr;        // [min(maxTokens,16)][experts]
    float *logitsRows = nullptr;    // [maxTokens][experts], allocated with the first INT8 router
    uint32_t *routeIds = nullptr;   // [topK] routes of the one-token path when the router runs as its own launch
    uint16_t *routeWeights = nullptr;
    uint32_t *ids = nullptr;        // [maxTokens][topK]
    uint16_t *weights = nullptr;    // [maxTokens][topK]
    ff::RoutePlan *plan = nullptr;
    ff::GemvJob *jobs[2] = {nullptr, nullptr};
    uint16_t *acts = nullptr;       // [maxTokens*topK][f]
    uint16_t *sharedActs = nullptr; // [maxTokens][sharedF]
    uint16_t *h1 = nullptr;         // [maxTokens][d]
    uint16_t *partials = nullptr;   // [maxTokens*topK][d]
    uint16_t *xDev = nullptr;       // [maxTokens][d] staging for *_host
    uint16_t *yDev = nullptr;

    // prefill scratch (allocated when maxTokens > 16)
    uint16_t *xSorted = nullptr;            // [maxTokens*topK][d] rows in expert order
    FFTokenExpertPair *sortedPairs = nullptr;
    uint32_t *expertOffsets = nullptr;      // [experts+1]
    uint32_t *blockCounts = nullptr;        // permute: [blocks][experts]
    uint32_t *units = nullptr;              // GEMM work units
    uint32_t *unitCount = nullptr;          // [4]
    uint32_t maxUnits = 0;
    uint32_t *errorFlag = nullptr;          // device: set by a kernel that gave up waiting
    unsigned long long *phaseStamps = nullptr;  // device: 8 phase + 288 per-warp timestamps of the fused decode kernel
    unsigned long long *taggedLogits = nullptr;  // device: [kMaxExperts] router logits of the fused decode kernel
    unsigned long long *taggedActs = nullptr;    // device: [topK * f / 2 + d / 2] routed activations, then shared output rows, as polled words
    uint32_t *gridBarrier = nullptr;        // device: eight 64-bit counters of the fused decode kernel
    volatile unsigned long long *mailbox = nullptr;  // pinned host word the decode kernel reports to
    uint32_t hostEpoch = 0;
    CUtensorMap *mapScratch = nullptr;

    // tracing: CUDA events around every kernel launch, aggregated per kernel name
    bool tracing = false;
    struct TraceRecord {
        const char *name;
        cudaEvent_t begin, end;
    };
    std::vector<TraceRecord> trace;

    // counters
    uint64_t kernelLaunches = 0;
    uint64_t weightBytes = 0;
    uint64_t scratchBytes = 0;
    uint32_t lastTokens = 0;
};

namespace ff {

// Counts a kernel launch and, when tracing is on, brackets it with CUDA events on its stream.
struct LaunchScope {
    FFContext *ctx;
    cudaStream_t stream;
    cudaEvent_t begin = nullptr, end = nullptr;
    const char *name;
    LaunchScope(FFContext *c, cudaStream_t s, const char *n) : ctx(c), stream(s), name(n) {
        ctx->kernelLaunches++;
        if (ctx->tracing) {
            cudaEventCreate(&begin);
            cudaEventCreate(&end);
            cudaEventRecord(begin, stream);
        }
    }
    ~LaunchScope() {
        if (begin) {
            cudaEventRecord(end, stream);
            ctx->trace.push_back({name, begin, end});
        }
    }
};

// ff_gemv.cu
bool launch_router_topk(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                        uint32_t tokens, uint32_t *ids, uint16_t *weights, float *logits,
                        cudaStream_t stream, const char **error);
bool launch_block_small(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                        uint32_t tokens, const uint32_t *ids, const uint16_t *weights,
                        bool withShared, bool decodeCombine, const uint16_t *residual,
                        uint16_t *partials, uint16_t *sharedOut, uint16_t *y,
                        cudaStream_t stream, const char **error);
bool launch_reduce(FFContext *ctx, const uint16_t *partials, const uint16_t *weights,
                   const uint16_t *residual, uint16_t *y, uint32_t tokens, cudaStream_t stream,
                   const char **error, const uint32_t *rowIndex = nullptr);
bool launch_gemv_rows(FFContext *ctx, const FFProjection &p, const uint16_t *x, uint32_t xStride,
                      uint32_t rows, uint16_t *y, uint32_t yStride, cudaStream_t stream,
                      const char **error);
bool launch_shared_small(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                         uint32_t tokens, uint16_t *y, cudaStream_t stream, const char **error);
bool launch_rmsnorm(FFContext *ctx, const uint16_t *x, const uint16_t *w, float eps,
                    uint32_t tokens, uint16_t *y, cudaStream_t stream, const char **error);
bool launch_dequant_probe(FFContext *ctx, const uint8_t *w, const uint16_t *s, const uint16_t *b,
                          uint32_t rows, uint32_t cols, float *out32, uint16_t *out16,
                          cudaStream_t stream, const char **error);

// ff_decode.cu
bool make_row_box_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t rowBytes, uint64_t experts,
                      uint64_t expertStride, uint32_t boxBytes, uint32_t boxRows, const char **error);

// Gate/up + GeGLU jobs, then down jobs, of a planned 2..16-row block on the tensor-core block kernels.
bool launch_block_mma(FFContext *ctx, const uint16_t *x, uint32_t xStride, uint32_t tokens, bool withShared,
                      bool haveDownJobs, cudaStream_t stream, const char **error);

// Host hand-off of the one-token kernel: `inlineX` (host memory) travels in the kernel parameters
// instead of `x`; the last CTA copies the output to `hostY` (host memory mapped for the device) and
// stores (error flag << 32 | epoch) to the mailbox word.
struct DecodeHostHandoff {
    const uint16_t *inlineX;
    uint16_t *hostY;
    unsigned long long *mailbox;
    uint32_t epoch;
};
bool launch_decode_fused(FFContext *ctx, const LayerStore &L, const uint16_t *x, const uint32_t *idsIn,
                         const uint16_t *weightsIn, bool withShared, bool routed, const uint16_t *residual,
                         uint16_t *y, cudaStream_t stream, const char **error,
                         const DecodeHostHandoff *host = nullptr);

// ff_prefill.cu
bool prefill_prepare_layer(FFContext *ctx, LayerStore &L, const char **error);
bool launch_prefill_routed(FFContext *ctx, LayerStore &L, const uint16_t *x, uint32_t xStride,
                           uint32_t tokens, const uint32_t *ids, uint16_t *partials,
                           cudaStream_t stream, const char **error);
bool launch_prefill_shared(FFContext *ctx, LayerStore &L, const uint16_t *x, uint32_t xStride,
                           uint32_t tokens, uint16_t *y, cudaStream_t stream, const char **error);
bool launch_post_attn_setup(FFContext *ctx, uint16_t *hidden, const uint16_t *attn, const uint16_t *wPostAttn,
                            const uint16_t *wPreFfn, const uint16_t *wPreFfn2, float eps, uint32_t tokens,
                            uint16_t *denseX, uint16_t *routedX, uint16_t *routerX, cudaStream_t stream,
                            const char **error);
bool launch_layer_tail(FFContext *ctx, const uint16_t *h2, const uint16_t *h1, uint16_t *hidden,
                       const uint16_t *wPostFfn2, const uint16_t *wPostFfn, float eps, float layerScalar,
                       uint32_t tokens, cudaStream_t stream, const char **error);
bool launch_shared_int8(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride, uint32_t tokens,
                        uint16_t *y, cudaStream_t stream, const char **error);
bool launch_route_sort(FFContext *ctx, const uint32_t *groupIds, uint32_t tokens, uint32_t groups,
                       FFTokenExpertPair *sortedPairs, uint32_t *offsets, cudaStream_t stream, const char **error);
bool launch_router_prefill(FFContext *ctx, const LayerStore &L, const uint16_t *x,
                           uint32_t xStride, uint32_t tokens, uint32_t *ids, uint16_t *weights,
                           float *logits, cudaStream_t stream, const char **error);

// nine offsets for a blob holding gate/up [f][d] and down [d][f]
FFExpertOffsets packed_offsets(uint32_t d, uint32_t f, uint64_t *payload);

}  // namespace ff
