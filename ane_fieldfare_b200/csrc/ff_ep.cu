// Expert parallelism behind the C ABI, one process driving every GPU of the group: the experts of a
// layer are split evenly over the ranks (rank p holds experts [p*E/g, (p+1)*E/g)), every rank
// routes its own rows, the rows travel to the ranks that hold their experts as stores into the
// destination's memory, the partial rows come back as peer copies, and the home rank combines
// them.  No collective library: the exchange is this file's own kernel writing over NVLink and
// cudaMemcpyPeerAsync, ordered by events between the ranks' streams.
#include <condition_variable>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "ff_internal.cuh"

using namespace ff;

namespace {

// destination rank of every route: the layer's placement table, or contiguous blocks without one
__global__ void k_ep_destination(const uint32_t *__restrict__ ids, uint32_t n, uint32_t expertsPerRank,
                                 uint32_t experts, const uint32_t *__restrict__ rankOf,
                                 uint32_t *__restrict__ dest) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t e = ids[i];
    dest[i] = e >= experts ? 0xFFFFFFFFu : rankOf ? rankOf[e] : e / expertsPerRank;
}

// where each (token, rank-in-row) route sits in the destination-sorted order
__global__ void k_ep_row_index(const FFTokenExpertPair *__restrict__ pairs, uint32_t n, uint32_t topK,
                               uint32_t *__restrict__ rowIndex) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) rowIndex[pairs[i].token * topK + pairs[i].rank] = i;
}

constexpr uint32_t kMaxRanks = 8;  // the GPUs of one NVSwitch box

// Where a rank's sorted routes go: destination p receives routes [first[p], first[p+1]) as rows
// rows[p][0...] with their local expert ids in ids[p][0...] (pointers into the destinations' memory).
struct SendTable {
    uint16_t *rows[kMaxRanks];
    uint32_t *ids[kMaxRanks];
    uint32_t first[kMaxRanks];
};
// One warp per route: copies the route's input row (16-byte pieces) and its expert id, local to the
// destination, into the destination rank's receive buffers — plain stores, over NVLink when the
// destination is another GPU.  A sorted pair's `expert` field is its destination rank.
__global__ void __launch_bounds__(256)
k_ep_send_rows(const uint16_t *__restrict__ x, uint32_t xStride, uint32_t d,
               const FFTokenExpertPair *__restrict__ pairs, uint32_t n, const uint32_t *__restrict__ ids,
               uint32_t topK, uint32_t expertsPerRank, const uint32_t *__restrict__ localOf,
               const __grid_constant__ SendTable table) {
    const uint32_t warpsPerCta = blockDim.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t i = blockIdx.x * warpsPerCta + (threadIdx.x >> 5); i < n; i += gridDim.x * warpsPerCta) {
        const FFTokenExpertPair p = pairs[i];
        if (p.expert >= kMaxRanks) continue;
        const uint32_t j = i - table.first[p.expert];
        const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)p.token * xStride);
        uint4 *dst = reinterpret_cast<uint4 *>(table.rows[p.expert] + (size_t)j * d);
        for (uint32_t c = lane; c < d / 8; c += 32) dst[c] = src[c];
        if (lane == 0) {
            const uint32_t e = ids[p.token * topK + p.rank];
            table.ids[p.expert][j] = localOf ? localOf[e] : e % expertsPerRank;
        }
    }
}

// Points of a layer at which a traced call records an event on the rank's stream (CopiesHome: on
// its second stream).
enum Mark : uint32_t {
    kLayerStart, kRouterDone, kPlanQueued, kSendStart, kSendDone, kRowsArrived, kExpertsDone, kCopiesHome,
    kSharedDone, kPartialsArrived, kReduceDone, kMarks
};
constexpr uint32_t kPhases = 10;

struct Rank {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t side = nullptr;     // the partial rows' way home (copy engines), beside the shared FFN
    cudaEvent_t sent = nullptr, returned = nullptr, expertsDone = nullptr;
    uint32_t *ids = nullptr;         // [tokens][K] global expert ids
    uint16_t *weights = nullptr;     // [tokens][K]
    uint32_t *dest = nullptr;        // [tokens][K] destination rank of each route
    FFTokenExpertPair *pairs = nullptr;  // routes sorted by destination
    uint32_t *offsets = nullptr;     // [world + 1] first route of each destination
    uint32_t *hostOffsets = nullptr; // pinned copy
    uint32_t *rowIndex = nullptr;    // [tokens][K] row of `back` holding each route's partial
    uint16_t *recvRows = nullptr;    // [capacity][d] rows received for this rank's experts
    uint32_t *recvIds = nullptr;     // [capacity] their local expert ids
    uint16_t *partials = nullptr;    // [capacity][d] this rank's experts' outputs
    uint16_t *back = nullptr;        // [tokens*K][d] partial rows of this rank's own routes, returned
    uint16_t *sharedOut = nullptr;   // [tokens][d]
    uint16_t *normed = nullptr;      // [tokens][d] stack: the layer's input
    uint16_t *between = nullptr;     // [tokens][d] stack: a layer's output that is not the last
    std::vector<cudaEvent_t> marks;     // tracing: kMarks events per layer, in the order of the Mark enum
    std::vector<uint32_t *> placement;  // per layer: [2][experts] rank of every expert, then its local slot; null = contiguous
};

// One host thread per rank, so that a phase is queued on all GPUs at once.  run() hands every
// thread the same job with its rank and returns when all are done; the first failure's message wins.
class Workers {
public:
    using Job = std::function<bool(uint32_t, const char **)>;
    void start(uint32_t n) {
        count = n;
        ok.assign(n, 1);
        errors.assign(n, nullptr);
        for (uint32_t r = 1; r < n; ++r) threads.emplace_back([this, r] { loop(r); });
    }
    ~Workers() {
        {
            std::lock_guard<std::mutex> lock(m);
            stop = true;
            ++generation;
        }
        wake.notify_all();
        for (std::thread &t : threads) t.join();
    }
    bool run(const Job &fn, const char **error) {
        {
            std::lock_guard<std::mutex> lock(m);
            job = &fn;
            pending = count - 1;
            ++generation;
        }
        wake.notify_all();
        errors[0] = nullptr;
        ok[0] = fn(0, &errors[0]);  // rank 0 on the calling thread
        {
            std::unique_lock<std::mutex> lock(m);
            done.wait(lock, [this] { return pending == 0; });
        }
        bool all = true;
        for (uint32_t r = 0; r < count; ++r) {
            if (!ok[r] && all) {
                all = false;
                if (error) *error = errors[r];
                else free(const_cast<char *>(errors[r]));
            } else if (errors[r]) {
                free(const_cast<char *>(errors[r]));
            }
            errors[r] = nullptr;
        }
        return all;
    }

private:
    void loop(uint32_t r) {
        uint64_t seen = 0;
        for (;;) {
            const Job *mine;
            {
                std::unique_lock<std::mutex> lock(m);
                wake.wait(lock, [&] { return generation != seen; });
                seen = generation;
                if (stop) return;
                mine = job;
            }
            errors[r] = nullptr;
            ok[r] = (*mine)(r, &errors[r]);
            {
                std::lock_guard<std::mutex> lock(m);
                --pending;
            }
            done.notify_one();
        }
    }
    uint32_t count = 0, pending = 0;
    uint64_t generation = 0;
    bool stop = false;
    const Job *job = nullptr;
    std::vector<std::thread> threads;
    std::vector<char> ok;
    std::vector<const char *> errors;
    std::mutex m;
    std::condition_variable wake, done;
};

template <typename T>
bool device_alloc(T **p, size_t count, const char **error) {
    FF_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(p), count * sizeof(T)), error);
    return true;
}

}  // namespace

struct FFEPGroup {
    uint32_t world = 0, experts = 0, expertsPerRank = 0, d = 0, topK = 0, maxTokens = 0, capacity = 0;
    std::vector<FFContext *> home, expert;
    std::vector<Rank> ranks;
    uint64_t lastRowsSent = 0;
    bool tracing = false;
    std::vector<double> phaseMs;  // [world][kPhases] of the last traced call
    Workers workers;
};

namespace {

// Records the next mark of a traced layer; a no-op otherwise.
bool mark(const FFEPGroup *g, Rank &R, cudaStream_t stream, const char **error) {
    if (!g->tracing) return true;
    cudaEvent_t e = nullptr;
    FF_CUDA_OK(cudaEventCreate(&e), error);
    R.marks.push_back(e);
    FF_CUDA_OK(cudaEventRecord(e, stream), error);
    return true;
}

void release(FFEPGroup *g) {
    for (Rank &r : g->ranks) {
        cudaSetDevice(r.device);
        if (r.stream) cudaStreamSynchronize(r.stream);
        cudaFree(r.ids); cudaFree(r.weights); cudaFree(r.dest); cudaFree(r.pairs); cudaFree(r.offsets);
        cudaFree(r.rowIndex); cudaFree(r.recvRows); cudaFree(r.recvIds); cudaFree(r.partials);
        cudaFree(r.back); cudaFree(r.sharedOut); cudaFree(r.normed); cudaFree(r.between);
        for (uint32_t *t : r.placement) cudaFree(t);
        for (cudaEvent_t e : r.marks) cudaEventDestroy(e);
        if (r.hostOffsets) cudaFreeHost(r.hostOffsets);
        if (r.side) cudaStreamSynchronize(r.side);
        if (r.sent) cudaEventDestroy(r.sent);
        if (r.returned) cudaEventDestroy(r.returned);
        if (r.expertsDone) cudaEventDestroy(r.expertsDone);
        if (r.stream) cudaStreamDestroy(r.stream);
        if (r.side) cudaStreamDestroy(r.side);
    }
    delete g;
}

bool build_group(FFEPGroup *g, const char **error) {
    const uint32_t world = g->world;
    for (uint32_t r = 0; r < world; ++r) {
        Rank &R = g->ranks[r];
        R.device = g->home[r]->device;
        FF_CUDA_OK(cudaSetDevice(R.device), error);
        for (uint32_t p = 0; p < world; ++p) {
            const int peer = g->home[p]->device;
            if (peer == R.device) continue;
            int can = 0;
            FF_CUDA_OK(cudaDeviceCanAccessPeer(&can, R.device, peer), error);
            if (!can)
                return fail(error, "device " + std::to_string(R.device) + " cannot address device " +
                                       std::to_string(peer) + ": the group needs peer access between all its GPUs");
            const cudaError_t st = cudaDeviceEnablePeerAccess(peer, 0);
            if (st == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else FF_CUDA_OK(st, error);
        }
        FF_CUDA_OK(cudaStreamCreateWithFlags(&R.stream, cudaStreamNonBlocking), error);
        FF_CUDA_OK(cudaEventCreateWithFlags(&R.sent, cudaEventDisableTiming), error);
        FF_CUDA_OK(cudaEventCreateWithFlags(&R.returned, cudaEventDisableTiming), error);
        FF_CUDA_OK(cudaStreamCreateWithFlags(&R.side, cudaStreamNonBlocking), error);
        FF_CUDA_OK(cudaEventCreateWithFlags(&R.expertsDone, cudaEventDisableTiming), error);
        const size_t routes = (size_t)g->maxTokens * g->topK;
        if (!device_alloc(&R.ids, routes, error) || !device_alloc(&R.weights, routes, error) ||
            !device_alloc(&R.dest, routes, error) || !device_alloc(&R.pairs, routes, error) ||
            !device_alloc(&R.offsets, world + 1, error) || !device_alloc(&R.rowIndex, routes, error) ||
            !device_alloc(&R.recvRows, (size_t)g->capacity * g->d, error) ||
            !device_alloc(&R.recvIds, g->capacity, error) ||
            !device_alloc(&R.partials, (size_t)g->capacity * g->d, error) ||
            !device_alloc(&R.back, routes * g->d, error) ||
            !device_alloc(&R.sharedOut, (size_t)g->maxTokens * g->d, error) ||
            !device_alloc(&R.normed, (size_t)g->maxTokens * g->d, error) ||
            !device_alloc(&R.between, (size_t)g->maxTokens * g->d, error))
            return false;
        R.placement.assign(g->home[r]->cfg.layers, nullptr);
        FF_CUDA_OK(cudaMallocHost(reinterpret_cast<void **>(&R.hostOffsets), (world + 1) * sizeof(uint32_t)), error);
    }
    return true;
}

}  // namespace

extern "C" {

FFEPGroup *ff_ep_create(FFContext *const *home, FFContext *const *expert, uint32_t world,
                        uint32_t capacityRows, const char **error) {
    if (error) *error = nullptr;
    if (!home || !expert || world == 0 || world > kMaxRanks) {
        fail(error, "expert-parallel group needs 1...8 ranks with a home and an expert context each");
        return nullptr;
    }
    FFEPGroup *g = new FFEPGroup;
    g->world = world;
    g->home.assign(home, home + world);
    g->expert.assign(expert, expert + world);
    g->ranks.resize(world);
    auto refuse = [&](const std::string &message) -> FFEPGroup * {
        fail(error, message);
        release(g);
        return nullptr;
    };
    for (uint32_t r = 0; r < world; ++r)
        if (!home[r] || !expert[r]) return refuse("null context for rank " + std::to_string(r));
    for (uint32_t r = 0; r < world; ++r) {
        if (home[r]->device != expert[r]->device)
            return refuse("rank " + std::to_string(r) + ": home and expert context sit on different devices");
        for (uint32_t q = 0; q < r; ++q)
            if (home[q]->device == home[r]->device) return refuse("two ranks share device " + std::to_string(home[r]->device));
    }
    const FFConfig &h = home[0]->cfg, &x = expert[0]->cfg;
    g->experts = h.experts;
    g->d = h.d;
    g->topK = h.topK;
    g->maxTokens = h.maxTokens;
    if (h.experts % world) return refuse("the experts do not divide evenly over the ranks");
    g->expertsPerRank = h.experts / world;
    if (h.d % 8) return refuse("the hidden width must be a multiple of 8");
    g->capacity = capacityRows ? capacityRows : world * h.maxTokens * h.topK;
    for (uint32_t r = 0; r < world; ++r) {
        const FFConfig &hr = home[r]->cfg, &xr = expert[r]->cfg;
        if (hr.layers != h.layers || hr.experts != h.experts || hr.d != h.d || hr.topK != h.topK ||
            hr.maxTokens != h.maxTokens)
            return refuse("the home contexts of all ranks must share one configuration");
        if (xr.layers != x.layers || xr.experts != g->expertsPerRank || xr.d != h.d || xr.topK != 1)
            return refuse("an expert context holds experts/world experts of the same width, with topK = 1 "
                          "(a received row is a one-route token)");
        if (xr.maxTokens < g->capacity)
            return refuse("an expert context's maxTokens must cover the group's capacity of " +
                          std::to_string(g->capacity) + " received rows");
    }
    if (!build_group(g, error)) {
        release(g);
        return nullptr;
    }
    g->workers.start(world);
    return g;
}

void ff_ep_destroy(FFEPGroup *group) {
    if (group) release(group);
}

uint64_t ff_ep_last_rows_sent(const FFEPGroup *group) { return group ? group->lastRowsSent : 0; }

// One block, queued on the ranks' streams by one host thread per rank.  The host waits once, for
// the counts of rows per destination; the rest is ordered by events, so consecutive layers need no
// wait between them: a rank sends its next rows only behind its own combine, which waited for
// every rank's experts and copies.  An event must be recorded before another thread queues a wait on it,
// hence the phases: the threads meet between them.  `normFrom` (stack): rows to normalise into the
// rank's `normed` buffer first, which is then the block's input.
static bool run_layer(FFEPGroup *g, uint32_t layer, const uint16_t *const *x, const uint16_t *const *normFrom,
                      float eps, uint32_t tokens, uint16_t *const *y, const char **error) {
    const uint32_t world = g->world, K = g->topK, D = g->d;
    const uint32_t routes = tokens * K;
    const bool withShared = g->home[0]->layers[layer].has_shared();

    // 1. every rank: router, destination of every route, routes sorted by destination, counts to the host
    if (!g->workers.run([&](uint32_t r, const char **err) -> bool {
            Rank &R = g->ranks[r];
            FF_CUDA_OK(cudaSetDevice(R.device), err);
            const uint16_t *in = normFrom ? R.normed : x[r];
            if (!mark(g, R, R.stream, err)) return false;  // kLayerStart
            if (normFrom && !ff_rmsnorm(g->home[r], normFrom[r], nullptr, eps, tokens, R.normed, R.stream, err))
                return false;
            if (!ff_router_topk(g->home[r], layer, in, D, tokens, R.ids, R.weights, nullptr, R.stream, err)) return false;
            if (!mark(g, R, R.stream, err)) return false;  // kRouterDone
            k_ep_destination<<<(routes + 255) / 256, 256, 0, R.stream>>>(R.ids, routes, g->expertsPerRank, g->experts,
                                                                         R.placement[layer], R.dest);
            FF_CUDA_OK(cudaGetLastError(), err);
            if (!ff_sort_routes(g->home[r], R.dest, tokens, world, R.pairs, R.offsets, R.stream, err)) return false;
            FF_CUDA_OK(cudaMemcpyAsync(R.hostOffsets, R.offsets, (world + 1) * sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                       R.stream), err);
            k_ep_row_index<<<(routes + 255) / 256, 256, 0, R.stream>>>(R.pairs, routes, K, R.rowIndex);
            FF_CUDA_OK(cudaGetLastError(), err);
            if (!mark(g, R, R.stream, err)) return false;  // kPlanQueued
            FF_CUDA_OK(cudaStreamSynchronize(R.stream), err);
            if (R.hostOffsets[world] != routes)
                return fail(err, "the router of rank " + std::to_string(r) + " wrote an expert id out of range");
            return true;
        }, error))
        return false;

    // 2. where each source's rows land in each destination's receive buffer
    std::vector<uint32_t> base((size_t)world * (world + 1));  // base[p * (world + 1) + s], the last entry the total
    uint64_t sentAway = 0;
    for (uint32_t p = 0; p < world; ++p) {
        uint32_t total = 0;
        for (uint32_t s = 0; s < world; ++s) {
            base[(size_t)p * (world + 1) + s] = total;
            const uint32_t n = g->ranks[s].hostOffsets[p + 1] - g->ranks[s].hostOffsets[p];
            total += n;
            if (s != p) sentAway += n;
        }
        base[(size_t)p * (world + 1) + world] = total;
        if (total > g->capacity)
            return fail(error, "rank " + std::to_string(p) + " would receive " + std::to_string(total) +
                                   " rows, more than the group's capacity " + std::to_string(g->capacity));
    }
    g->lastRowsSent = sentAway;

    // 3. dispatch: one kernel per rank stores its rows into every destination's buffer
    if (!g->workers.run([&](uint32_t s, const char **err) -> bool {
            Rank &S = g->ranks[s];
            FF_CUDA_OK(cudaSetDevice(S.device), err);
            const uint16_t *in = normFrom ? S.normed : x[s];
            SendTable table{};
            for (uint32_t p = 0; p < world; ++p) {
                const uint32_t at = base[(size_t)p * (world + 1) + s];
                table.rows[p] = g->ranks[p].recvRows + (size_t)at * D;
                table.ids[p] = g->ranks[p].recvIds + at;
                table.first[p] = S.hostOffsets[p];
            }
            const uint32_t ctas = (routes + 7) / 8 < 1184u ? (routes + 7) / 8 : 1184u;
            if (!mark(g, S, S.stream, err)) return false;  // kSendStart
            k_ep_send_rows<<<ctas, 256, 0, S.stream>>>(in, D, D, S.pairs, routes, S.ids, K, g->expertsPerRank,
                                                       S.placement[layer] ? S.placement[layer] + g->experts : nullptr, table);
            FF_CUDA_OK(cudaGetLastError(), err);
            FF_CUDA_OK(cudaEventRecord(S.sent, S.stream), err);
            return mark(g, S, S.stream, err);  // kSendDone
        }, error))
        return false;

    // 4. every rank's experts on what it received; the partial rows copied into their homes, the shared FFN beside that
    if (!g->workers.run([&](uint32_t p, const char **err) -> bool {
            Rank &P = g->ranks[p];
            FF_CUDA_OK(cudaSetDevice(P.device), err);
            for (uint32_t s = 0; s < world; ++s)
                if (s != p) FF_CUDA_OK(cudaStreamWaitEvent(P.stream, g->ranks[s].sent, 0), err);
            const uint32_t total = base[(size_t)p * (world + 1) + world];
            if (!mark(g, P, P.stream, err)) return false;  // kRowsArrived
            if (total &&
                !ff_moe_prefill(g->expert[p], layer, P.recvRows, D, total, P.recvIds, P.partials, P.stream, err))
                return false;
            if (!mark(g, P, P.stream, err)) return false;  // kExpertsDone
            // the partial rows go home by the copy engines on the second stream, while the SMs run the
            // shared FFN
            FF_CUDA_OK(cudaEventRecord(P.expertsDone, P.stream), err);
            FF_CUDA_OK(cudaStreamWaitEvent(P.side, P.expertsDone, 0), err);
            for (uint32_t i = 1; i <= world; ++i) {
                const uint32_t s = (p + i) % world;  // the other GPUs first, this one's own rows last
                const uint32_t first = g->ranks[s].hostOffsets[p], n = g->ranks[s].hostOffsets[p + 1] - first;
                if (!n) continue;
                const uint16_t *src = P.partials + (size_t)base[(size_t)p * (world + 1) + s] * D;
                uint16_t *dst = g->ranks[s].back + (size_t)first * D;
                const size_t bytes = (size_t)n * D * sizeof(uint16_t);
                if (s == p) FF_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, P.side), err);
                else FF_CUDA_OK(cudaMemcpyPeerAsync(dst, g->ranks[s].device, src, P.device, bytes, P.side), err);
            }
            FF_CUDA_OK(cudaEventRecord(P.returned, P.side), err);
            if (!mark(g, P, P.side, err)) return false;  // kCopiesHome
            if (withShared) {
                const uint16_t *in = normFrom ? P.normed : x[p];
                if (!ff_shared_ffn(g->home[p], layer, in, D, tokens, P.sharedOut, P.stream, err)) return false;
            }
            return mark(g, P, P.stream, err);  // kSharedDone
        }, error))
        return false;

    // 5. combine at home: weighted sum of each row's K partials in rank order, plus the shared rows
    return g->workers.run([&](uint32_t r, const char **err) -> bool {
        Rank &R = g->ranks[r];
        FF_CUDA_OK(cudaSetDevice(R.device), err);
        for (uint32_t p = 0; p < world; ++p) FF_CUDA_OK(cudaStreamWaitEvent(R.stream, g->ranks[p].returned, 0), err);
        if (!mark(g, R, R.stream, err)) return false;  // kPartialsArrived
        if (!ff_moe_reduce_indexed(g->home[r], R.back, R.rowIndex, R.weights, withShared ? R.sharedOut : nullptr, y[r],
                                   tokens, R.stream, err))
            return false;
        return mark(g, R, R.stream, err);  // kReduceDone
    }, error);
}

// Sums a traced call's phases per rank over its layers and drops the events.
static bool collect_marks(FFEPGroup *g, const char **error) {
    // phase i runs from mark kFrom[i] to mark kTo[i]
    static const Mark kFrom[kPhases] = {kLayerStart, kRouterDone, kPlanQueued, kSendStart, kSendDone, kRowsArrived,
                                        kExpertsDone, kExpertsDone, kSharedDone, kPartialsArrived};
    static const Mark kTo[kPhases] = {kRouterDone, kPlanQueued, kSendStart, kSendDone, kRowsArrived, kExpertsDone,
                                      kCopiesHome, kSharedDone, kPartialsArrived, kReduceDone};
    g->phaseMs.assign((size_t)g->world * kPhases, 0.0);
    for (uint32_t r = 0; r < g->world; ++r) {
        Rank &R = g->ranks[r];
        FF_CUDA_OK(cudaSetDevice(R.device), error);
        for (size_t at = 0; at + kMarks <= R.marks.size(); at += kMarks)
            for (uint32_t i = 0; i < kPhases; ++i) {
                float ms = 0.0f;
                FF_CUDA_OK(cudaEventElapsedTime(&ms, R.marks[at + kFrom[i]], R.marks[at + kTo[i]]), error);
                g->phaseMs[(size_t)r * kPhases + i] += ms > 0.0f ? ms : 0.0f;
            }
        for (cudaEvent_t e : R.marks) cudaEventDestroy(e);
        R.marks.clear();
    }
    return true;
}

// Waits for every rank's stream and reads every context's error flag.
static bool finish(FFEPGroup *g, const char **error) {
    const uint32_t world = g->world;
    for (uint32_t r = 0; r < world; ++r) {
        FF_CUDA_OK(cudaSetDevice(g->ranks[r].device), error);
        FF_CUDA_OK(cudaStreamSynchronize(g->ranks[r].stream), error);
        FF_CUDA_OK(cudaStreamSynchronize(g->ranks[r].side), error);
    }
    if (g->tracing && !collect_marks(g, error)) return false;
    for (uint32_t r = 0; r < world; ++r) {
        FFContext *both[2] = {g->home[r], g->expert[r]};
        for (FFContext *c : both) {
            uint32_t flag = 0;
            FF_CUDA_OK(cudaSetDevice(c->device), error);
            FF_CUDA_OK(cudaMemcpy(&flag, c->errorFlag, sizeof(flag), cudaMemcpyDeviceToHost), error);
            if (flag) return fail(error, "a kernel of rank " + std::to_string(r) + " gave up waiting (error flag " +
                                             std::to_string(flag) + ")");
        }
    }
    return true;
}

static bool check_call(FFEPGroup *g, uint32_t firstLayer, uint32_t layerCount, const uint16_t *const *x,
                       uint32_t tokens, uint16_t *const *y, const char **error) {
    if (error) *error = nullptr;
    if (!g || !x || !y) return fail(error, "null argument");
    if (tokens > g->maxTokens)
        return fail(error, std::to_string(tokens) + " rows per rank exceed the group's " + std::to_string(g->maxTokens));
    if (layerCount == 0 || firstLayer + layerCount > g->home[0]->cfg.layers ||
        firstLayer + layerCount > g->expert[0]->cfg.layers)
        return fail(error, "layer out of range");
    for (uint32_t r = 0; r < g->world; ++r)
        if (!x[r] || !y[r] || ((reinterpret_cast<uintptr_t>(x[r]) | reinterpret_cast<uintptr_t>(y[r])) & 15u))
            return fail(error, "rank " + std::to_string(r) + ": rows must be non-null and 16-byte aligned");
    // marks a failed traced call left behind
    for (Rank &R : g->ranks) {
        for (cudaEvent_t e : R.marks) cudaEventDestroy(e);
        R.marks.clear();
    }
    return true;
}

bool ff_ep_moe_layer(FFEPGroup *g, uint32_t layer, const uint16_t *const *x, uint32_t tokens,
                     uint16_t *const *y, const char **error) {
    if (!check_call(g, layer, 1, x, tokens, y, error)) return false;
    if (tokens == 0) return true;
    return run_layer(g, layer, x, nullptr, 0.0f, tokens, y, error) && finish(g, error);
}

bool ff_ep_moe_stack(FFEPGroup *g, uint32_t firstLayer, uint32_t layerCount, const uint16_t *const *x,
                     uint32_t tokens, float eps, uint16_t *const *y, const char **error) {
    if (!check_call(g, firstLayer, layerCount, x, tokens, y, error)) return false;
    if (tokens == 0) return true;
    const uint32_t world = g->world;
    std::vector<const uint16_t *> cur(x, x + world);
    std::vector<uint16_t *> out(world);
    for (uint32_t i = 0; i < layerCount; ++i) {
        for (uint32_t r = 0; r < world; ++r) out[r] = i + 1 == layerCount ? y[r] : g->ranks[r].between;
        if (!run_layer(g, firstLayer + i, nullptr, cur.data(), eps, tokens, out.data(), error)) return false;
        for (uint32_t r = 0; r < world; ++r) cur[r] = out[r];
    }
    return finish(g, error);
}

void ff_ep_set_tracing(FFEPGroup *g, bool enabled) {
    if (g) g->tracing = enabled;
}

uint32_t ff_ep_get_phase_times(const FFEPGroup *g, double *milliseconds, uint32_t capacity) {
    if (!g || !milliseconds) return 0;
    uint32_t n = 0;
    for (; n < capacity && n < g->phaseMs.size(); ++n) milliseconds[n] = g->phaseMs[n];
    return n;
}

bool ff_ep_set_placement(FFEPGroup *g, uint32_t layer, const uint32_t *rankOf, const uint32_t *localOf,
                         const char **error) {
    if (error) *error = nullptr;
    if (!g || !rankOf || !localOf) return fail(error, "null argument");
    if (layer >= g->home[0]->cfg.layers) return fail(error, "layer out of range");
    std::vector<uint8_t> taken((size_t)g->world * g->expertsPerRank, 0);
    for (uint32_t e = 0; e < g->experts; ++e) {
        if (rankOf[e] >= g->world || localOf[e] >= g->expertsPerRank)
            return fail(error, "expert " + std::to_string(e) + " is placed outside the group");
        uint8_t &slot = taken[(size_t)rankOf[e] * g->expertsPerRank + localOf[e]];
        if (slot) return fail(error, "two experts share slot " + std::to_string(localOf[e]) + " of rank " + std::to_string(rankOf[e]));
        slot = 1;
    }
    for (Rank &R : g->ranks) {
        FF_CUDA_OK(cudaSetDevice(R.device), error);
        FF_CUDA_OK(cudaStreamSynchronize(R.stream), error);
        if (!R.placement[layer] && !device_alloc(&R.placement[layer], 2 * (size_t)g->experts, error)) return false;
        FF_CUDA_OK(cudaMemcpy(R.placement[layer], rankOf, g->experts * sizeof(uint32_t), cudaMemcpyHostToDevice), error);
        FF_CUDA_OK(cudaMemcpy(R.placement[layer] + g->experts, localOf, g->experts * sizeof(uint32_t),
                              cudaMemcpyHostToDevice), error);
    }
    return true;
}

}  // extern "C"
