// One token through the whole MoE block in ONE cooperative kernel: router, top-8, routed
// gate/up/GeGLU, shared FFN, routed down and the weighted combine.
//
// The step streams 37.5 MB of weights once; at B200's HBM rate that is under 6 us, so separate
// kernels (launch gaps, cold starts) cannot come near the roofline.  Here one CTA per SM runs
// three phases:
//   A  router logits (one warp per expert) and the shared gate/up/GeGLU rows; the shared down
//      rows are already requested;
//   B  every CTA ranks the 128 logits itself (top-8, softmax, gain), then routed gate/up/GeGLU
//      rows and the shared down rows; the routed down rows are requested as the warps finish;
//   C  routed down rows and the fixed-order combine onto the shared output (or the caller's
//      residual).
// Values cross from CTA to CTA as tagged 64-bit words that the readers poll (logits, routed
// activations, shared output rows: value and validity in one L2 round trip), and through one
// arrival counter (the shared activations between A and B).
//
// Weight rows reach the SM as asynchronous copies (completion counted on a per-warp mbarrier)
// into a per-warp shared-memory slot: cp.async.bulk.tensor over row-box maps of the layer where a
// tile's rows lie at one stride (one request brings 8 or 16 row pieces), cp.async.bulk for scale
// runs and for the routed down rows of the eight scattered experts.
//
// Row arithmetic runs on the tensor cores without dequantizing: a warp task is a tile of 16 weight
// rows; per group of 64 codes the packed nibbles are turned into the bf16 values 16+q with two
// integer instructions per pair (the code goes into the mantissa of 16.0) and multiplied with the
// bf16 input by mma.sync m16n8k16 (fp32 accumulate; the product of a 5-bit integer and a bf16 is
// exact).  The group's sum is then scaled:
//     acc += scale * sum((16+q) x) + (bias - 16 scale) * sum(x).
// The eight columns of the MMA are one input row for the gate/up and shared rows, and the eight
// routed experts' activations for the routed down rows (a tile = two output rows of all eight
// experts).  Long rows are split along K between the warps of a pair (or triple) of one CTA and
// added in a fixed order, so results do not depend on scheduling.
//
// Grid-wide waits poll arrival counters in global memory; cooperative launch guarantees that all
// CTAs are resident.  Every spin (grid barrier, copy completion) is bounded: on running
// out it raises the context's error flag and carries on, so the launch always ends.
//
// Reference kernels replaced (paths inside the reference project):
//   Sources/ANEFieldfareHotpath/Metal/MoE/moe.metal:65-120,242-319,500-517,548-570,597-638
//   Sources/ANEFieldfareHotpath/Metal/Quant/dequant_int4.metal:78-169
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>

#include "ff_mma_device.cuh"

namespace ff {

constexpr int kFusedThreads = 512;
constexpr int kFusedWarps = kFusedThreads / 32;
constexpr int kBigWarps = 10;      // warps 0..9: gate/up pairs and the routed down tiles
constexpr int kSharedGuWarps = 8;  // warps 0..7 take the shared gate/up tiles in phase A (K quarters)
constexpr uint32_t kBarrierSpinLimit = 1u << 24;

struct DecodeArgs {
    const uint16_t *routerW, *routerScale, *gain;
    const float *logitBias;
    const uint8_t *experts;
    uint64_t stride;
    FFExpertOffsets off;
    const uint8_t *shared;  // null: no shared FFN, `residual` is added instead
    FFExpertOffsets sharedOff;
    const uint16_t *x;
    const uint16_t *residual;
    const uint32_t *idsIn;  // non-null: routes are given, the router is skipped
    const uint16_t *weightsIn;
    float *logits;
    // Values handed from CTA to CTA travel as 64-bit words (launch tag << 32 | payload) that the
    // readers poll: a word is valid when its tag is the running launch's, so nothing is cleared.
    unsigned long long *taggedLogits;  // [E] payload: the logit's bits
    unsigned long long *taggedActs;    // [K * F / 2] payload: two routed activations (bf16)
    unsigned long long *taggedH1;      // [D / 2] payload: two rows of the shared FFN's output (bf16)
    uint32_t *ids;
    uint16_t *weights;
    uint16_t *acts, *sharedActs, *h1, *y;
    unsigned long long *barrier;  // arrival counter of the grid barrier
    uint32_t *errorFlag;
    unsigned long long *stamps;  // null, or the phase / per-warp timestamp slots (ns)
    int E, D, F, Fs, K;          // K = 0: shared FFN only (y receives its output)
    int expertCount;             // resident experts of the layer: routes at or past it are refused
    int prefetch;                // bit 0: L2 prefetch of the chosen experts' down projections (off by default)
    // host hand-off (null when unused): the last CTA to finish copies y to `hostY` (host memory the
    // device can write), then stores (error flag << 32 | epoch) to `mailbox`, which the host polls
    uint16_t *hostY;
    unsigned long long *mailbox;
    uint32_t epoch;
    // shared-memory carve-up (fused_layout)
    uint32_t regionOffset, partialOffset, slotsOffset, bigBytes, smallBytes;
    uint32_t strideGU, strideGUA, strideSD, strideRD, actStride, winBytes, winPitch;
};

// Row-box tensor maps of the layer (kernel parameters): routed gate, routed up, shared gate, shared
// up, shared down.  A tile's eight (sixteen) row pieces arrive as one tensor copy per matrix.
struct alignas(64) DecodeMaps {
    CUtensorMap m[5];
};
enum : int { kMapRoutedGate = 0, kMapRoutedUp = 1, kMapSharedGate = 2, kMapSharedUp = 3, kMapSharedDown = 4 };

// Fetches a tensor map's descriptor ahead of its first use (the first copy through a map otherwise
// waits for it).
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Bulk L2 prefetch of [p, p + bytes); bytes a multiple of 16, p 16-byte aligned.
__device__ __forceinline__ void prefetch_l2_bulk(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// The grid prefetches [base, base+bytes) in 8 KiB pieces.  Piece i belongs to CTA (i + cursor) mod
// gridDim and to one of its `nthreads` issuing threads (this one is number `tid`), so every SM
// issues the same share: a bulk prefetch is executed by the issuing SM's copy engine, whose
// throughput is a small fraction of HBM's.
// `issue` false: only the cursor moves on (another warp takes this region).
__device__ __forceinline__ void prefetch_region(const uint8_t *base, uint64_t bytes, uint32_t &cursor, uint32_t tid,
                                                uint32_t nthreads, bool issue) {
    constexpr uint32_t kPiece = 8192;
    const uint32_t pieces = (uint32_t)((bytes + kPiece - 1) / kPiece);
    const uint32_t first = (blockIdx.x + gridDim.x - cursor % gridDim.x) % gridDim.x;
    for (uint32_t i = first + tid * gridDim.x; issue && i < pieces; i += gridDim.x * nthreads) {
        const uint64_t offset = (uint64_t)i * kPiece;
        const uint32_t len = (uint32_t)min((uint64_t)kPiece, bytes - offset) & ~15u;
        if (len) prefetch_l2_bulk(base + offset, len);
    }
    cursor += pieces;
}

// Grid-wide synchronisation on 64-bit counters that only grow.  At its start every CTA draws a
// ticket from counter [3]; ticket / gridDim is the launch's generation g (launches on a context
// are serialised, so all CTAs of a launch get the same g).  Every launch adds exactly gridDim to
// counter [0] (shared activations written) — also when a mode does not wait on it — so "everyone
// has arrived" is counter >= (g + 1) * gridDim.  An arrival is a release reduction without a
// return value; a wait polls the counter with acquire loads, bounded.  No reset, no host-side
// state.  [2] counts finished CTAs for the host hand-off.  g also gives the launch's 32-bit tag
// (never 0, different for consecutive launches) for the values that travel as polled words
// (logits, routed activations, shared output rows).
enum : int { kCountShared = 0, kCountDone = 2, kCountTicket = 3 };

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Called by ONE thread after a CTA-level barrier that covers the writes to publish.
__device__ __forceinline__ void counter_arrive(unsigned long long *count) {
    asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(count) : "memory");
}
// Called by ONE thread; a CTA-level barrier afterwards releases the other threads.
__device__ __forceinline__ void counter_wait(const unsigned long long *count, unsigned long long target,
                                             uint32_t *errorFlag) {
    uint32_t spins = 0;
    while (ld_acquire_u64(count) < target) {
        if (++spins > kBarrierSpinLimit) {
            atomicExch(errorFlag, 9u);
            break;
        }
    }
    __threadfence();
}
// The thread that arrives at and waits for the CTA-wide barriers: lane 0 of the last warp (a warp
// with no requests to issue between arriving and waiting).
__device__ __forceinline__ bool is_barrier_thread() { return threadIdx.x == blockDim.x - 32; }

__device__ __forceinline__ void st_tagged(unsigned long long *p, uint32_t tag, uint32_t payload) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(((unsigned long long)tag << 32) | payload) : "memory");
}
__device__ __forceinline__ unsigned long long ld_tagged(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void stamp(const DecodeArgs &a, int slot) {
    if (a.stamps && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.stamps[slot] = t;
    }
}

// Per-warp timestamps of two CTAs (first and last) when tracing: slot 8 + ((cta01 * 3 + phase) * 16 +
// warp) * 3 + which, which = 0 requests issued, 1 data arrived, 2 rows done.
__device__ __forceinline__ void warp_stamp(const DecodeArgs &a, int phase, int which) {
    if (a.stamps && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) && (threadIdx.x & 31) == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        const int c = blockIdx.x == 0 ? 0 : 1;
        a.stamps[8 + ((c * 3 + phase) * 16 + (threadIdx.x >> 5)) * 3 + which] = t;
    }
}

// `n` consecutive groups of a 16-row tile: acc0 / acc1 = this thread's sums for tile rows g and
// g+8.  s0/b0 and s1/b1: the two rows' scales and biases, xs: the input's group sums, all starting
// at the first group.  `odd` picks MMA column 2t+1 instead of 2t.  Groups are taken in ascending
// order whatever the batching, so the result does not depend on it.  Shared by every phase.
__device__ __noinline__ void tile_rows(const uint8_t *lo, const uint8_t *hi, const uint8_t *xg, const uint16_t *s0,
                                       const uint16_t *b0, const uint16_t *s1, const uint16_t *b1, const float *xs,
                                       int n, bool odd, float &acc0, float &acc1) {
    float v0 = 0.0f, v1 = 0.0f;
    int i = 0;
#pragma unroll 1
    for (; i + 4 <= n; i += 4) {
        float d[4][4];
        groups_mma<4>(lo + 32 * i, hi + 32 * i, xg + 128 * i, d);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            v0 = group_scale(v0, s0[i + u], b0[i + u], odd ? d[u][1] : d[u][0], xs[i + u]);
            v1 = group_scale(v1, s1[i + u], b1[i + u], odd ? d[u][3] : d[u][2], xs[i + u]);
        }
    }
    if (i + 2 <= n) {
        float d[2][4];
        groups_mma<2>(lo + 32 * i, hi + 32 * i, xg + 128 * i, d);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            v0 = group_scale(v0, s0[i + u], b0[i + u], odd ? d[u][1] : d[u][0], xs[i + u]);
            v1 = group_scale(v1, s1[i + u], b1[i + u], odd ? d[u][3] : d[u][2], xs[i + u]);
        }
        i += 2;
    }
    if (i < n) {
        float d[1][4];
        groups_mma<1>(lo + 32 * i, hi + 32 * i, xg + 128 * i, d);
        v0 = group_scale(v0, s0[i], b0[i], odd ? d[0][1] : d[0][0], xs[i]);
        v1 = group_scale(v1, s1[i], b1[i], odd ? d[0][3] : d[0][2], xs[i]);
    }
    acc0 = v0;
    acc1 = v1;
}

// Box of a row-box map at (64-bit word x, row y, expert z) into shared memory (128-byte aligned).
// x * 8 bytes must be a multiple of 16.
__device__ __forceinline__ void box_copy(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

// stage_input for rows that other CTAs are still writing as tagged words (two bf16 values each):
// every run of eight values is polled (bounded) until its four words carry `tag`.
__device__ __forceinline__ void stage_tagged(const unsigned long long *src, uint32_t tag, int rows, int n, uint8_t *dst,
                                             uint32_t dstStride, float *sums, uint32_t *errorFlag) {
    const int runsPerRow = n >> 3, runs = rows * runsPerRow;
    auto fetch = [&](int i, uint4 &v) {
        unsigned long long w0, w1, w2, w3;
        asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(w0), "=l"(w1) : "l"(src + 4 * (size_t)i) : "memory");
        asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(w2), "=l"(w3) : "l"(src + 4 * (size_t)i + 2) : "memory");
        v = make_uint4((uint32_t)w0, (uint32_t)w1, (uint32_t)w2, (uint32_t)w3);
        return (uint32_t)(w0 >> 32) == tag && (uint32_t)(w1 >> 32) == tag && (uint32_t)(w2 >> 32) == tag &&
               (uint32_t)(w3 >> 32) == tag;
    };
    for (int base = (threadIdx.x >> 5) << 5; base < runs; base += 2 * blockDim.x) {
        const int i = base + (threadIdx.x & 31), j = i + blockDim.x;
        const bool vi = i < runs, vj = j < runs;
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = make_uint4(0, 0, 0, 0);
        bool ok0 = !vi, ok1 = !vj;
        for (uint32_t spins = 0; spins < kBarrierSpinLimit && !(ok0 && ok1); ++spins) {
            if (!ok0) ok0 = fetch(i, v0);
            if (!ok1) ok1 = fetch(j, v1);
        }
        if (!(ok0 && ok1)) atomicExch(errorFlag, 9u);
        stage_put(i, vi, v0, runsPerRow, dst, dstStride, sums);
        if (base + (int)blockDim.x < runs) stage_put(j, vj, v1, runsPerRow, dst, dstStride, sums);  // warp-uniform
    }
    __syncthreads();
}

// The input row travelling inside the kernel's parameters (no host-to-device copy before the
// launch): up to 4096 bf16 values.
struct InlineRow {
    uint4 v[512];
};

// xInline: null, or the input row in parameter space (read with plain loads).
__device__ __forceinline__ void decode_body(const DecodeArgs &a, const DecodeMaps &maps, const uint16_t *xInline) {
    extern __shared__ __align__(128) uint8_t smemRaw[];
    __shared__ __align__(16) float sLogits[kMaxExperts + 8];  // padded with -inf up to two spans of the ranking
    __shared__ uint32_t sIds[8];
    __shared__ float sWeights[8];
    __shared__ float sScore[8];
    __shared__ __align__(8) uint64_t sCopyBar[kFusedWarps];
    __shared__ unsigned long long sTarget;  // (generation + 1) * gridDim
    __shared__ uint32_t sTag;               // the launch's tag for polled words, from the generation

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = (int)gridDim.x, cta = (int)blockIdx.x;
    const int D = a.D, F = a.F, Fs = a.Fs, K = a.K, E = a.E;
    const int g = lane >> 2, t = lane & 3;
    const int groupsD = D >> 6, groupsF = F >> 6, groupsFs = Fs >> 6;

    // shared memory: x (bf16, run-permuted) | its group sums | region for the shared / routed
    // activations | K-split partial sums | kBigWarps big slots | small slots for the other warps
    uint8_t *xPerm = smemRaw;
    float *xSum = reinterpret_cast<float *>(smemRaw + D * 2);
    uint8_t *region = smemRaw + a.regionOffset;
    float *partial = reinterpret_cast<float *>(smemRaw + a.partialOffset);  // [warp][16]
    uint8_t *slots = smemRaw + a.slotsOffset;
    uint8_t *mySlot = warp < kBigWarps ? slots + (size_t)warp * a.bigBytes
                                        : slots + (size_t)kBigWarps * a.bigBytes + (size_t)(warp - kBigWarps) * a.smallBytes;
    const uint32_t slotAddr = sm_addr(mySlot);
    const uint32_t myBar = sm_addr(&sCopyBar[warp]);
    uint32_t parity = 0;

    if (threadIdx.x == 0) {
        for (int w = 0; w < kFusedWarps; ++w) bar_init(sm_addr(&sCopyBar[w]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp >= 11 && lane == 0) prefetch_tensormap(&maps.m[warp - 11]);  // warps 11..15: the five maps
    // the ticket: drawn now by a thread with nothing to request (warp 9), published to the CTA
    // further down so that nobody waits for the atomic's round trip here
    unsigned long long ticket = 0;
    if (threadIdx.x == 9 * 32) ticket = atomicAdd(a.barrier + kCountTicket, 1ull);
    // this thread's share of the input row is requested before anything else
    const bool xPlain = xInline != nullptr;
    const uint16_t *xSrc = xPlain ? xInline : a.x;
    uint4 xMine = make_uint4(0, 0, 0, 0);
    if ((int)threadIdx.x < (D >> 3))
        xMine = xPlain ? reinterpret_cast<const uint4 *>(xSrc)[threadIdx.x]
                       : __ldcg(reinterpret_cast<const uint4 *>(xSrc) + threadIdx.x);
    __syncthreads();
    uint32_t cursor = 0;
    stamp(a, 0);

    const uint8_t *sh = a.shared;
    const int tilesSGU = sh ? Fs >> 3 : 0;  // 8 gate + 8 up rows per tile, two K halves
    const int tilesSD = sh ? D >> 4 : 0;    // 16 down rows per tile, three K parts

    // Requests of part `part` of `parts` (along K) of a gate/up tile: one box of eight row pieces per
    // matrix (`pitch` bytes per row in the slot: the box is as wide as the pitch, what it reads past
    // the part is not used), then the eight rows' scales and biases of both matrices over the full K
    // (contiguous runs).
    auto issue_gate_up = [&](const CUtensorMap *gateMap, const CUtensorMap *upMap, int expert, const uint8_t *blob,
                             const FFExpertOffsets &off, int tile, int part, int parts, uint32_t pitch) {
        int gb, ge;
        part_range(groupsD, parts, part, gb, ge);
        const uint32_t sb = (uint32_t)groupsD * 16u;
        if (lane == 0) bar_expect(myBar, (ge > gb ? 16u * pitch : 0u) + 4u * sb);
        __syncwarp();
        if (lane < 2) {
            if (ge > gb) box_copy(slotAddr + (uint32_t)lane * 8u * pitch, lane ? upMap : gateMap, gb * 4, tile * 8, expert, myBar);
        } else if (lane >= 16 && lane < 20) {
            const uint32_t which = (uint32_t)lane - 16u;
            const uint32_t src = which == 0 ? off.gateSOff : which == 1 ? off.gateBOff : which == 2 ? off.upSOff : off.upBOff;
            bulk_copy(slotAddr + 16u * pitch + which * sb, blob + src + (size_t)tile * sb, sb, myBar);
        }
    };
    // Gate/up tile part -> this thread's partial sums of gate row tile*8+g and up row tile*8+g.
    auto compute_gate_up = [&](int part, int parts, uint32_t pitch, const uint8_t *xp, const float *xs, float &gate, float &up) {
        int gb, ge;
        part_range(groupsD, parts, part, gb, ge);
        const uint8_t *lo = mySlot + (size_t)g * pitch + 8 * t;
        const uint8_t *hi = mySlot + (size_t)(g + 8) * pitch + 8 * t;
        const uint16_t *sc = reinterpret_cast<const uint16_t *>(mySlot + 16u * pitch);
        const uint16_t *gS = sc + g * groupsD, *gB = gS + 8 * groupsD, *uS = gB + 8 * groupsD, *uB = uS + 8 * groupsD;
        gate = 0.0f;
        up = 0.0f;
        tile_rows(lo, hi, xp + gb * 128 + t * 32, gS + gb, gB + gb, uS + gb, uB + gb, xs + gb, ge - gb, false, gate, up);
    };
    auto issue_shared_down = [&](int tile, int part) {
        int gb, ge;
        part_range(groupsFs, 3, part, gb, ge);
        const uint32_t sb = (uint32_t)groupsFs * 32u;
        if (lane == 0) bar_expect(myBar, (ge > gb ? 16u * a.strideSD : 0u) + 2u * sb);
        __syncwarp();
        if (lane == 0) {
            if (ge > gb) box_copy(slotAddr, &maps.m[kMapSharedDown], gb * 4, tile * 16, 0, myBar);
        } else if (lane >= 16 && lane < 18) {
            const uint32_t which = (uint32_t)lane - 16u;
            bulk_copy(slotAddr + 16u * a.strideSD + which * sb,
                      sh + (which ? a.sharedOff.downBOff : a.sharedOff.downSOff) + (size_t)tile * sb, sb, myBar);
        }
    };

    // ---------------- phase A: router logits, shared gate/up/GeGLU ----------------
    // The router rows are requested first, alone: top-8 heads the critical path, and the copy
    // engine serves an SM's requests in order.
    int eA = (!a.idsIn && K > 0 && warp >= kSharedGuWarps && warp < kBigWarps) ? (warp - kSharedGuWarps) * G + cta
                                                                             : 0x7FFFFFFF;
    if (eA < E) {
        // the router's per-column scales (the same for every expert) come along behind the row
        if (lane == 0) {
            bar_expect(myBar, (uint32_t)D * (a.routerScale ? 4u : 2u));
            bulk_copy(slotAddr, a.routerW + (size_t)eA * D, (uint32_t)D * 2u, myBar);
            if (a.routerScale) bulk_copy(slotAddr + (uint32_t)D * 2u, a.routerScale, (uint32_t)D * 2u, myBar);
        }
        __syncwarp();
    }
    __syncthreads();
    // shared gate/up tiles: four warps per tile (K quarters), two tiles per CTA and round
    const int partA = warp & 3;
    int tA = warp < kSharedGuWarps ? (warp >> 2) * G + cta : 0x7FFFFFFF;
    if (tA < tilesSGU)
        issue_gate_up(&maps.m[kMapSharedGate], &maps.m[kMapSharedUp], 0, sh, a.sharedOff, tA, partA, 4, a.strideGUA);
    const int triple = warp >= kBigWarps ? (warp - kBigWarps) / 3 : 0;
    const int part3 = warp >= kBigWarps ? (warp - kBigWarps) % 3 : 0;
    int tSD = warp >= kBigWarps ? triple * G + cta : 0x7FFFFFFF;
    if (tSD < tilesSD) issue_shared_down(tSD, part3);
    warp_stamp(a, 0, 0);
    if (threadIdx.x == 9 * 32) {
        const unsigned long long gen1 = ticket / gridDim.x + 1ull;
        sTarget = gen1 * gridDim.x;
        sTag = (uint32_t)(gen1 % 0xFFFFFFFFull) + 1u;  // 1 .. 2^32-1: never 0, consecutive launches differ
    }
    stage_input(xSrc, 1, D, xPerm, 0, xSum, xPlain, &xMine);  // ends with a CTA barrier: target and tag are published
    const uint32_t tag = sTag;
    for (; tA < tilesSGU; tA += (kSharedGuWarps / 4) * G) {
        slot_wait(myBar, parity, a.errorFlag);
        warp_stamp(a, 0, 1);
        float gate, up;
        compute_gate_up(partA, 4, a.strideGUA, xPerm, xSum, gate, up);
        slot_release();
        const int next = tA + (kSharedGuWarps / 4) * G;
        if (next < tilesSGU)
            issue_gate_up(&maps.m[kMapSharedGate], &maps.m[kMapSharedUp], 0, sh, a.sharedOff, next, partA, 4, a.strideGUA);
        float *mine = partial + warp * 16;
        if (partA && t == 0) {
            mine[g] = gate;
            mine[8 + g] = up;
        }
        named_barrier(1 + (warp >> 2), 128);
        if (!partA && t == 0) {
            gate = ((gate + mine[16 + g]) + mine[32 + g]) + mine[48 + g];
            up = ((up + mine[16 + 8 + g]) + mine[32 + 8 + g]) + mine[48 + 8 + g];
            a.sharedActs[tA * 8 + g] = f2bf(gelu_tanh(bf16_round(gate)) * bf16_round(up));
        }
        named_barrier(1 + (warp >> 2), 128);
    }
    // eight products of one run: the row's weights and, behind them in the slot, the router's
    // per-column scales (if any); staged input at `base`
    auto router_run = [&](const uint16_t *wr, int base, float acc) {
        const uint4 wv = *reinterpret_cast<const uint4 *>(wr + base);
        // the staged run holds elements 0,4,1,5,2,6,3,7: low halves are 0..3, high halves 4..7
        const uint4 xv = *reinterpret_cast<const uint4 *>(xPerm + base * 2);
        float xe[8] = {__uint_as_float(xv.x << 16),         __uint_as_float(xv.y << 16),
                       __uint_as_float(xv.z << 16),         __uint_as_float(xv.w << 16),
                       __uint_as_float(xv.x & 0xFFFF0000u), __uint_as_float(xv.y & 0xFFFF0000u),
                       __uint_as_float(xv.z & 0xFFFF0000u), __uint_as_float(xv.w & 0xFFFF0000u)};
        if (a.routerScale) {
            const uint4 sv = *reinterpret_cast<const uint4 *>(wr + D + base);
            const uint32_t ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                xe[2 * k] = xe[2 * k] * __uint_as_float(ss[k] << 16);
                xe[2 * k + 1] = xe[2 * k + 1] * __uint_as_float(ss[k] & 0xFFFF0000u);
            }
        }
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            acc = fmaf(__uint_as_float(ww[k] << 16), xe[2 * k], acc);
            acc = fmaf(__uint_as_float(ww[k] & 0xFFFF0000u), xe[2 * k + 1], acc);
        }
        return acc;
    };
    for (; eA < E; eA += (kBigWarps - kSharedGuWarps) * G) {
        slot_wait(myBar, parity, a.errorFlag);
        warp_stamp(a, 0, 1);
        const uint16_t *wr = reinterpret_cast<const uint16_t *>(mySlot);
        float acc = 0.0f;
        for (int base = 8 * lane; base < D; base += 256) acc = router_run(wr, base, acc);
#pragma unroll
        for (int offset = 16; offset >= 1; offset >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, offset);
        if (lane == 0) {
            const float logit = a.logitBias ? acc + a.logitBias[eA] : acc;
            a.logits[eA] = logit;
            // value and validity in one 64-bit store: the readers poll these words
            st_tagged(a.taggedLogits + eA, tag, __float_as_uint(logit));
        }
        slot_release();
        const int next = eA + (kBigWarps - kSharedGuWarps) * G;
        if (next < E && lane == 0) {
            bar_expect(myBar, (uint32_t)D * (a.routerScale ? 4u : 2u));
            bulk_copy(slotAddr, a.routerW + (size_t)next * D, (uint32_t)D * 2u, myBar);
            if (a.routerScale) bulk_copy(slotAddr + (uint32_t)D * 2u, a.routerScale, (uint32_t)D * 2u, myBar);
        }
        __syncwarp();
    }
    warp_stamp(a, 0, 2);
    stamp(a, 1);

    // ---------------- top-8 by warps 8..15 while warps 0..7 finish the shared gate/up rows ----------
    // Each logit travels as one 64-bit word (validity | value) that the readers poll, so ranking
    // waits neither for a counter round trip nor for the other CTAs' shared rows.
    if (K > 0 && !a.idsIn && warp >= kSharedGuWarps) {
        constexpr int kTopkThreads = (kFusedWarps - kSharedGuWarps) * 32;
        const int tid2 = (int)threadIdx.x - kSharedGuWarps * 32;
        // one warp fetches the logits, polling the tagged words (four per lane, coalesced) until
        // every writer's store has shown up
        if (warp == kSharedGuWarps) {
            for (int base = 0; base < E; base += 128) {
                const int e0 = base + 4 * lane;
                const unsigned long long filler = (unsigned long long)tag << 32;
                unsigned long long w[4] = {filler, filler, filler, filler};
                bool ready = false;
                for (uint32_t spins = 0; spins < kBarrierSpinLimit && !ready; ++spins) {
                    if (e0 + 3 < E) {
                        asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(w[0]), "=l"(w[1]) : "l"(a.taggedLogits + e0) : "memory");
                        asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(w[2]), "=l"(w[3]) : "l"(a.taggedLogits + e0 + 2) : "memory");
                    } else {
                        for (int i = 0; i < 4; ++i)
                            if (e0 + i < E)
                                asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w[i]) : "l"(a.taggedLogits + e0 + i) : "memory");
                    }
                    const bool mine = (uint32_t)(w[0] >> 32) == tag && (uint32_t)(w[1] >> 32) == tag &&
                                      (uint32_t)(w[2] >> 32) == tag && (uint32_t)(w[3] >> 32) == tag;
                    ready = __all_sync(0xFFFFFFFFu, mine);
                }
                if (!ready && lane == 0) atomicExch(a.errorFlag, 9u);
                for (int i = 0; i < 4; ++i)
                    if (e0 + i < E) sLogits[e0 + i] = __uint_as_float((uint32_t)w[i]);
            }
        }
        const int rankSpan = (((E + 1) >> 1) + 3) & ~3;
        if (tid2 < 8) {
            sIds[tid2] = 0u;
            sScore[tid2] = -INFINITY;
        } else if (tid2 >= 32 && tid2 < 40 && E + tid2 - 32 < 2 * rankSpan) {
            sLogits[E + tid2 - 32] = -INFINITY;
        }
        named_barrier(8, kTopkThreads);
        // rank of every logit under (higher score, then lower expert id); scores of -inf or NaN
        // are never taken — the order of the serial top-8 (moe.metal:269-303).  Two threads per
        // expert, each counting the competitors of one span (a multiple of four, read as float4).
        {
            for (int idx = tid2; idx < 2 * ((E + 127) & ~127); idx += kTopkThreads) {
                const int e = idx >> 1, half = idx & 1;
                const float v = e < E ? sLogits[e] : -INFINITY;
                const int begin = half * rankSpan;
                int rank = 0;
#pragma unroll 4
                for (int o = begin; o < begin + rankSpan; o += 4) {
                    const float4 c = *reinterpret_cast<const float4 *>(sLogits + o);
                    // a competitor wins with a higher score, or the same score and a lower id
                    rank += (c.x > v || (c.x == v && o < e)) ? 1 : 0;
                    rank += (c.y > v || (c.y == v && o + 1 < e)) ? 1 : 0;
                    rank += (c.z > v || (c.z == v && o + 2 < e)) ? 1 : 0;
                    rank += (c.w > v || (c.w == v && o + 3 < e)) ? 1 : 0;
                }
                rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 1);
                if (half == 0 && v > -INFINITY && rank < K) {
                    sIds[rank] = (uint32_t)e;
                    sScore[rank] = v;
                }
            }
        }
        named_barrier(8, kTopkThreads);
        if (warp == kSharedGuWarps) {
            // softmax over the chosen scores: exponentials in parallel, the sum in rank order
            const float score = lane < K ? sScore[lane] : -INFINITY;
            const float top = __shfl_sync(0xFFFFFFFFu, score, 0);
            const float ex = lane < K ? expf(score - top) : 0.0f;
            float sum = 0.0f;
            for (int r = 0; r < K; ++r) sum += __shfl_sync(0xFFFFFFFFu, ex, r);
            if (lane < K) {
                float w = ex / sum;
                if (a.gain) w = w * bf2f(a.gain[sIds[lane]]);
                const uint16_t wb = f2bf(w);
                sWeights[lane] = bf2f(wb);
                if (blockIdx.x == 0) {
                    a.ids[lane] = sIds[lane];
                    a.weights[lane] = wb;
                }
            }
        }
    } else {
        // Given routes.  A route past the resident experts would address memory outside the layer:
        // it is replaced by expert 0 with weight 0 and reported through the error flag (the
        // reference refuses such a route with "route expert N is out of range").
        if (K > 0 && a.idsIn && threadIdx.x < K) {
            uint32_t id = a.idsIn[threadIdx.x];
            float w = bf2f(a.weightsIn[threadIdx.x]);
            if (id >= (uint32_t)a.expertCount) {
                atomicExch(a.errorFlag, 12u);
                id = 0u;
                w = 0.0f;
            }
            sIds[threadIdx.x] = id;
            sWeights[threadIdx.x] = w;
        }
    }
    // barrier 1 covers the shared activations; the routed rows are requested between arriving
    // and waiting (the CTA barrier also publishes the routes to all warps)
    __syncthreads();
    if (is_barrier_thread()) counter_arrive(a.barrier + kCountShared);
    stamp(a, 2);
    stamp(a, 3);
    const int tilesF = F >> 3;
    const int tilesRouted = K * tilesF;
    int tB = warp < kBigWarps ? (warp >> 1) * G + cta : 0x7FFFFFFF;
    if (tB < tilesRouted) {
        const int slot = tB / tilesF;
        issue_gate_up(&maps.m[kMapRoutedGate], &maps.m[kMapRoutedUp], (int)sIds[slot],
                      a.experts + (size_t)sIds[slot] * a.stride, a.off, tB - slot * tilesF, warp & 1, 2, a.strideGU);
    }
    warp_stamp(a, 1, 0);
    // Routed down tile: output rows 2*tile, 2*tile+1 of all eight experts.  Tile row rho*8 + e is
    // row 2*tile+rho of expert e; lane l copies row piece l (l < 16), or the 16-byte aligned window
    // around the two rows' scales (l even) or biases (l odd) of expert (l-16)/2.
    // Tiles go to the warps in the order 10..15, 0..9: the warps of the shared down rows are done
    // early in phase B and request their routed down tile then, into their own slot, so that it is
    // in shared memory when the second grid barrier opens; warps 0..9 request theirs at the barrier.
    const int tilesRD = D >> 1;
    const int orderC = warp >= kBigWarps ? warp - kBigWarps : warp + (kFusedWarps - kBigWarps);
    auto issue_routed_down = [&](int tile) {
        const uint32_t piece = (uint32_t)groupsF * 32u;
        if (lane == 0) bar_expect(myBar, 16u * piece + 16u * a.winBytes);
        __syncwarp();
        const int e = lane < 16 ? (lane & 7) : ((lane - 16) >> 1);
        const uint8_t *blob = a.experts + (size_t)sIds[e < K ? e : 0] * a.stride;
        if (lane < 16) {
            const int row = tile * 2 + (lane >> 3);
            bulk_copy(slotAddr + (uint32_t)lane * a.strideRD, blob + a.off.downWOff + (size_t)row * (F >> 1), piece, myBar);
        } else {
            const uint32_t srcOff = ((lane & 1) ? a.off.downBOff : a.off.downSOff) + (uint32_t)tile * 4u * (uint32_t)groupsF;
            // windows: scales of expert e at e * winPitch, biases at (8 + e) * winPitch
            bulk_copy(slotAddr + 16u * a.strideRD + (uint32_t)(((lane & 1) << 3) + e) * a.winPitch, blob + (srcOff & ~15u),
                      a.winBytes, myBar);
        }
    };
    uint8_t *saPerm = region;
    float *saSum = reinterpret_cast<float *>(region + Fs * 2);
    if (sh) {
        if (is_barrier_thread()) counter_wait(a.barrier + kCountShared, sTarget, a.errorFlag);
        __syncthreads();
        stage_input(a.sharedActs, 1, Fs, saPerm, 0, saSum);
    }
    bool downAsked = !(a.prefetch & 1) || warp >= K;
    for (; tB < tilesRouted; tB += (kBigWarps / 2) * G) {
        slot_wait(myBar, parity, a.errorFlag);
        warp_stamp(a, 1, 1);
        if (!downAsked) {
            // The down projections of the chosen experts go to L2 for phase C: warp k asks for
            // expert k's once its own rows are there.  Earlier, the prefetch shares HBM with the
            // gate/up rows that the arithmetic is waiting for; from here on it runs under the
            // arithmetic.
            for (int k = 0; k < K; ++k) {
                const uint8_t *blob = a.experts + (size_t)sIds[k] * a.stride;
                prefetch_region(blob + a.off.downWOff,
                                (uint64_t)a.off.downBOff - a.off.downWOff + (uint64_t)D * F / kGroup * 2, cursor, lane, 32,
                                k == warp);
            }
            downAsked = true;
        }
        float gate, up;
        compute_gate_up(warp & 1, 2, a.strideGU, xPerm, xSum, gate, up);
        slot_release();
        const int next = tB + (kBigWarps / 2) * G;
        if (next < tilesRouted) {
            const int slot = next / tilesF;
            issue_gate_up(&maps.m[kMapRoutedGate], &maps.m[kMapRoutedUp], (int)sIds[slot],
                          a.experts + (size_t)sIds[slot] * a.stride, a.off, next - slot * tilesF, warp & 1, 2, a.strideGU);
        }
        float *mine = partial + warp * 16;
        if ((warp & 1) && t == 0) {
            mine[g] = gate;
            mine[8 + g] = up;
        }
        named_barrier(1 + (warp >> 1), 64);
        if (!(warp & 1)) {
            // the tile's eight activations are one run of the staged row: four tagged words,
            // written by the lanes t == 0 of even g (the odd neighbour's value comes by shuffle)
            gate += mine[16 + g];
            up += mine[16 + 8 + g];
            const uint32_t act = f2bf(gelu_tanh(gate) * up);
            const uint32_t two = act | (__shfl_down_sync(0xFFFFFFFFu, act, 4) << 16);
            if (t == 0 && !(g & 1)) st_tagged(a.taggedActs + ((tB * 8 + g) >> 1), tag, two);
        }
        named_barrier(1 + (warp >> 1), 64);
    }
    for (; tSD < tilesSD; tSD += 2 * G) {
        slot_wait(myBar, parity, a.errorFlag);
        warp_stamp(a, 1, 1);
        int gb, ge;
        part_range(groupsFs, 3, part3, gb, ge);
        const uint8_t *lo = mySlot + (size_t)g * a.strideSD + 8 * t;
        const uint8_t *hi = mySlot + (size_t)(g + 8) * a.strideSD + 8 * t;
        const uint16_t *sS = reinterpret_cast<const uint16_t *>(mySlot + 16u * a.strideSD);
        const uint16_t *sB = sS + 16 * groupsFs;
        float v0, v1;
        tile_rows(lo, hi, saPerm + gb * 128 + t * 32, sS + g * groupsFs + gb, sB + g * groupsFs + gb,
                  sS + (g + 8) * groupsFs + gb, sB + (g + 8) * groupsFs + gb, saSum + gb, ge - gb, false, v0, v1);
        slot_release();
        const int next = tSD + 2 * G;
        if (next < tilesSD) issue_shared_down(next, part3);
        float *mine = partial + warp * 16;
        if (part3 && t == 0) {
            mine[g] = v0;
            mine[8 + g] = v1;
        }
        named_barrier(6 + triple, 96);
        if (!part3) {
            v0 = (v0 + mine[16 + g]) + mine[32 + g];
            v1 = (v1 + mine[16 + 8 + g]) + mine[32 + 8 + g];
            const uint32_t r0 = f2bf(v0), r1 = f2bf(v1);
            if (K > 0) {
                // read as the residual of the routed rows in phase C: tagged words of two rows
                const uint32_t two0 = r0 | (__shfl_down_sync(0xFFFFFFFFu, r0, 4) << 16);
                const uint32_t two1 = r1 | (__shfl_down_sync(0xFFFFFFFFu, r1, 4) << 16);
                if (t == 0 && !(g & 1)) {
                    st_tagged(a.taggedH1 + ((tSD * 16 + g) >> 1), tag, two0);
                    st_tagged(a.taggedH1 + ((tSD * 16 + 8 + g) >> 1), tag, two1);
                }
            } else if (t == 0) {
                a.y[tSD * 16 + g] = (uint16_t)r0;
                a.y[tSD * 16 + 8 + g] = (uint16_t)r1;
            }
        }
        named_barrier(6 + triple, 96);
    }
    int tC = orderC * G + cta;
    if (K > 0 && warp >= kBigWarps && tC < tilesRD) issue_routed_down(tC);
    warp_stamp(a, 1, 2);
    stamp(a, 4);
    if (K == 0) {
        stamp(a, 5);
        stamp(a, 6);
        return;
    }

    // No grid barrier before phase C: the routed activations and the shared output rows are polled
    // as tagged words while they are staged.
    if (warp < kBigWarps && tC < tilesRD) issue_routed_down(tC);
    warp_stamp(a, 2, 0);
    __syncthreads();  // the region still holds the shared activations that phase B's warps read
    stamp(a, 5);

    // ---------------- phase C: routed down rows and the combine ----------------
    {
        // activations of slot e: run-permuted bf16 at region + e * actStride, group sums behind them
        float *actSum = reinterpret_cast<float *>(region + 8 * a.actStride);
        if (K < 8) {
            for (int e = K; e < 8; ++e) {
                for (int i = threadIdx.x; i < (F >> 3); i += blockDim.x)
                    reinterpret_cast<uint4 *>(region + (size_t)e * a.actStride)[i] = make_uint4(0, 0, 0, 0);
                for (int i = threadIdx.x; i < groupsF; i += blockDim.x) actSum[e * groupsF + i] = 0.0f;
            }
        }
        stage_tagged(a.taggedActs, tag, K, F, region, a.actStride, actSum, a.errorFlag);
        for (; tC < tilesRD; tC += kFusedWarps * G) {
            slot_wait(myBar, parity, a.errorFlag);
            warp_stamp(a, 2, 1);
            // this thread: expert g, tile rows g (rho 0) and g+8 (rho 1); column g of the MMA is
            // held by the lane with t == g/2 as d[g&1] (rho 0) and d[2 + (g&1)] (rho 1)
            const uint8_t *lo = mySlot + (size_t)g * a.strideRD + 8 * t;
            const uint8_t *hi = mySlot + (size_t)(g + 8) * a.strideRD + 8 * t;
            const uint8_t *xe = region + (size_t)g * a.actStride + t * 32;
            const uint32_t rowOff = (uint32_t)tC * 4u * (uint32_t)groupsF;
            const uint8_t *win = mySlot + 16u * a.strideRD + (uint32_t)g * a.winPitch;
            const uint16_t *sS = reinterpret_cast<const uint16_t *>(win + ((a.off.downSOff + rowOff) & 15u));
            const uint16_t *sB = reinterpret_cast<const uint16_t *>(win + 8u * a.winPitch + ((a.off.downBOff + rowOff) & 15u));
            const float *xs = actSum + g * groupsF;
            const bool odd = g & 1;
            const int row = tC * 2 + (lane & 1);
            // the residual: rows 2*tile and 2*tile+1 of the shared output are one tagged word, asked
            // for now and checked after the arithmetic; or the caller's residual row
            unsigned long long resWord = 0;
            if (a.shared && lane == 0) resWord = ld_tagged(a.taggedH1 + tC);
            float acc = (!a.shared && a.residual && lane < 2) ? bf2f(__ldcg(a.residual + row)) : 0.0f;
            float v0, v1;
            tile_rows(lo, hi, xe, sS, sB, sS + groupsF, sB + groupsF, xs, groupsF, odd, v0, v1);
            slot_release();
            if (a.shared) {
                if (lane == 0) {
                    uint32_t spins = 0;
                    while ((uint32_t)(resWord >> 32) != tag) {
                        if (++spins > kBarrierSpinLimit) {
                            atomicExch(a.errorFlag, 9u);
                            break;
                        }
                        resWord = ld_tagged(a.taggedH1 + tC);
                    }
                }
                const uint32_t two = __shfl_sync(0xFFFFFFFFu, (uint32_t)resWord, 0);
                acc = bf2f((uint16_t)((lane & 1) ? two >> 16 : two & 0xFFFFu));
            }
            const int next = tC + kFusedWarps * G;
            if (next < tilesRD) issue_routed_down(next);
            // lane 0 combines row 2*tile, lane 1 row 2*tile+1, experts in rank order
            for (int k = 0; k < K; ++k) {
                const int src = 4 * k + (k >> 1);
                const float e0 = __shfl_sync(0xFFFFFFFFu, v0, src);
                const float e1 = __shfl_sync(0xFFFFFFFFu, v1, src);
                acc = __fadd_rn(acc, __fmul_rn(sWeights[k], (lane & 1) ? e1 : e0));
            }
            if (lane < 2) a.y[row] = f2bf(acc);
        }
    }
    warp_stamp(a, 2, 2);
    stamp(a, 6);

    // ---------------- host hand-off by the last CTA to finish ----------------
    if (a.mailbox) {
        __shared__ uint32_t sLast;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            const unsigned long long old = atomicAdd(a.barrier + kCountDone, 1ull);
            sLast = (old % gridDim.x == gridDim.x - 1) ? 1u : 0u;
        }
        __syncthreads();
        if (sLast) {
            __threadfence();
            for (int i = threadIdx.x; i < (D >> 3); i += blockDim.x)
                reinterpret_cast<uint4 *>(a.hostY)[i] = __ldcg(reinterpret_cast<const uint4 *>(a.y) + i);
            // one system-scope release by one thread publishes the row (ordered before it by the CTA
            // barrier) together with the error flag and the epoch, as one 64-bit word
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned long long word =
                    ((unsigned long long)__ldcg(a.errorFlag) << 32) | (unsigned long long)a.epoch;
                asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.mailbox), "l"(word) : "memory");
            }
        }
    }
}

__global__ void __launch_bounds__(kFusedThreads, 1)
k_decode_fused(const DecodeArgs a, const __grid_constant__ DecodeMaps maps) {
    decode_body(a, maps, nullptr);
}

__global__ void __launch_bounds__(kFusedThreads, 1)
k_decode_fused_inline_x(const DecodeArgs a, const __grid_constant__ DecodeMaps maps,
                        const __grid_constant__ InlineRow row) {
    decode_body(a, maps, reinterpret_cast<const uint16_t *>(&row));
}

struct FusedLayout {
    uint32_t regionOffset, partialOffset, slotsOffset, bigBytes, smallBytes;
    uint32_t strideGU, strideGUA, strideSD, strideRD, actStride, winBytes, winPitch;
    size_t total;
};

static FusedLayout fused_layout(const FFConfig &c) {
    const uint32_t D = c.d, F = c.f, Fs = c.sharedF;
    const uint32_t groupsD = D / 64, groupsF = F / 64, groupsFs = Fs / 64;
    FusedLayout l{};
    l.strideGU = piece_stride(((groupsD + 1) / 2) * 32);   // routed tiles: K halves
    l.strideGUA = piece_stride(((groupsD + 3) / 4) * 32);  // shared tiles: K quarters
    l.strideSD = Fs ? piece_stride(((groupsFs + 2) / 3) * 32) : 32;
    l.strideRD = piece_stride(groupsF * 32);
    l.winBytes = pad16u(4 * groupsF) + 16;
    // window pitch: 80 modulo 128 puts the eight experts' windows on different banks
    l.winPitch = l.winBytes;
    while ((l.winPitch & 127u) != 80u) l.winPitch += 16u;
    // per-expert activation stride: 16 modulo 128.  A quarter-warp's 128-bit load covers two
    // experts, four lanes each reading 16 bytes at 32-byte steps; the second expert's chunks then
    // fall into the gaps of the first.
    l.actStride = F * 2;
    while ((l.actStride & 127u) != 16u) l.actStride += 16u;
    const uint32_t xPart = (D * 2 + groupsD * 4 + 127u) & ~127u;
    const uint32_t sharedPart = Fs ? Fs * 2 + groupsFs * 4 : 0;
    const uint32_t actsPart = 8 * l.actStride + 8 * groupsF * 4;
    l.regionOffset = xPart;
    l.partialOffset = (l.regionOffset + std::max(sharedPart, actsPart) + 127u) & ~127u;
    l.slotsOffset = l.partialOffset + kFusedWarps * 16 * 4;
    const uint32_t gateUp = 16 * l.strideGU + 4 * groupsD * 16;
    const uint32_t down8 = 16 * l.strideRD + 16 * l.winPitch;
    const uint32_t sharedDown = Fs ? 16 * l.strideSD + 2 * groupsFs * 32 : 0;
    l.bigBytes = (std::max({gateUp, down8, D * 4}) + 127u) & ~127u;
    l.smallBytes = (std::max({sharedDown, down8, 128u}) + 127u) & ~127u;
    l.total = (size_t)l.slotsOffset + (size_t)kBigWarps * l.bigBytes + (size_t)(kFusedWarps - kBigWarps) * l.smallBytes;
    return l;
}

// One decode row through router (unless ids are given), routed experts and the shared FFN (or
// the caller's residual), as one cooperative launch.  routed = false: the shared FFN alone, y
// receives its output.
bool launch_decode_fused(FFContext *ctx, const LayerStore &L, const uint16_t *x, const uint32_t *idsIn,
                         const uint16_t *weightsIn, bool withShared, bool routed, const uint16_t *residual,
                         uint16_t *y, cudaStream_t stream, const char **error, const DecodeHostHandoff *host) {
    const FFConfig &c = ctx->cfg;
    if (routed && !L.experts) return fail(error, "layer has no resident experts");
    if (routed && !idsIn && !L.has_router()) return fail(error, "layer has no resident router");
    if (routed && !idsIn && L.routerQ) {
        // The kernel's own router reads bf16 rows.  An INT8 router runs as its own launches in
        // front (logits, top-K), and the kernel takes the routes as given.
        if (host) return fail(error, "the host hand-off needs a bf16 router");
        if (L.routerExperts != L.expertCount) return fail(error, "router and layer disagree on the expert count");
        if (!launch_router_topk(ctx, L, x, ctx->cfg.d, 1, ctx->routeIds, ctx->routeWeights, nullptr, stream, error))
            return false;
        idsIn = ctx->routeIds;
        weightsIn = ctx->routeWeights;
    }
    if (withShared && !L.shared) return fail(error, "layer has no resident shared FFN");
    if (!routed && !withShared) return fail(error, "nothing to compute");
    if (c.topK > 8) return fail(error, "decode supports at most 8 routes");
    if (c.d % 64 || c.f % 64 || c.sharedF % 64) return fail(error, "widths must be multiples of 64");
    DecodeArgs a{};
    a.routerW = L.routerW;
    a.routerScale = L.routerScale;
    a.gain = L.gain;
    a.logitBias = L.logitBias;
    a.experts = L.experts;
    a.stride = L.stride;
    a.off = L.off;
    a.shared = withShared ? L.shared : nullptr;
    a.sharedOff = L.sharedOff;
    a.x = x;
    a.residual = residual;
    a.idsIn = idsIn;
    a.weightsIn = weightsIn;
    a.logits = ctx->logits;
    a.taggedLogits = ctx->taggedLogits;
    a.taggedActs = ctx->taggedActs;
    a.taggedH1 = ctx->taggedActs + (size_t)c.topK * c.f / 2;
    a.ids = ctx->ids;
    a.weights = ctx->weights;
    a.acts = ctx->acts;
    a.sharedActs = ctx->sharedActs;
    a.h1 = ctx->h1;
    a.y = y;
    a.barrier = reinterpret_cast<unsigned long long *>(ctx->gridBarrier);
    a.errorFlag = ctx->errorFlag;
    a.stamps = ctx->tracing ? ctx->phaseStamps : nullptr;
    static const int prefetchMode = [] {
        const char *env = getenv("FF_DECODE_PREFETCH");
        return env ? atoi(env) : 0;  // off: measured slower than the early requests of phase C's tiles
    }();
    a.prefetch = prefetchMode;
    a.E = idsIn ? (int)L.expertCount : (int)L.routerExperts;
    a.expertCount = (int)L.expertCount;
    if (routed && !idsIn && L.routerExperts != L.expertCount)
        return fail(error, "router has " + std::to_string(L.routerExperts) + " experts, the layer " +
                               std::to_string(L.expertCount));
    a.D = (int)c.d;
    a.F = (int)c.f;
    a.Fs = withShared ? (int)c.sharedF : 0;
    a.K = routed ? (int)c.topK : 0;
    if (a.E > kMaxExperts) return fail(error, "too many experts for the decode kernel");
    const FusedLayout lay = fused_layout(c);
    const size_t smem = lay.total;
    if (smem > 227 * 1024)
        return fail(error, "model shape too large for the fused decode kernel's shared memory");
    // bulk copies need 16-byte aligned sources: every sub-tensor offset and the blob stride
    const uint32_t *ro = &L.off.gateWOff, *so = &L.sharedOff.gateWOff;
    for (int i = 0; i < 9; ++i)
        if ((routed && (ro[i] % 16 || L.stride % 16)) || (withShared && so[i] % 16))
            return fail(error, "sub-tensor offsets must be multiples of 16 bytes for the decode kernel");
    if (!(host && host->inlineX) && ((uintptr_t)x & 15) != 0) return fail(error, "input row must be 16-byte aligned");
    // row-box tensor maps of the layer, built once per loaded layer
    LayerStore &Lm = const_cast<LayerStore &>(L);
    if (!Lm.decodeMapsReady) {
        memset(Lm.decodeMap, 0, sizeof(Lm.decodeMap));
        if (L.experts) {
            const uint32_t *o = &L.off.gateWOff;
            for (int m = 0; m < 2; ++m)
                if (!make_row_box_map(&Lm.decodeMap[kMapRoutedGate + m], L.experts + o[3 * m], c.f, c.d / 2,
                                      L.expertCount, L.stride, lay.strideGU, 8, error))
                    return false;
        }
        if (L.shared && c.sharedF) {
            const uint32_t *o = &L.sharedOff.gateWOff;
            for (int m = 0; m < 2; ++m)
                if (!make_row_box_map(&Lm.decodeMap[kMapSharedGate + m], L.shared + o[3 * m], c.sharedF, c.d / 2, 1,
                                      0, lay.strideGUA, 8, error))
                    return false;
            if (!make_row_box_map(&Lm.decodeMap[kMapSharedDown], L.shared + o[6], c.d, c.sharedF / 2, 1, 0,
                                  lay.strideSD, 16, error))
                return false;
        }
        Lm.decodeMapsReady = true;
    }
    static thread_local DecodeMaps maps;
    memcpy(maps.m, L.decodeMap, sizeof(maps.m));
    a.regionOffset = lay.regionOffset;
    a.partialOffset = lay.partialOffset;
    a.slotsOffset = lay.slotsOffset;
    a.bigBytes = lay.bigBytes;
    a.smallBytes = lay.smallBytes;
    a.strideGU = lay.strideGU;
    a.strideGUA = lay.strideGUA;
    a.strideSD = lay.strideSD;
    a.strideRD = lay.strideRD;
    a.actStride = lay.actStride;
    a.winBytes = lay.winBytes;
    a.winPitch = lay.winPitch;
    static KernelSmemMemo memo, memoInline;
    int perSm = 0;
    if (!memo.prepare(k_decode_fused, ctx->device, smem, kFusedThreads, &perSm, error)) return false;
    if (perSm < 1) return fail(error, "fused decode kernel does not fit on an SM");
    if (!memoInline.prepare(k_decode_fused_inline_x, ctx->device, smem, kFusedThreads, &perSm, error)) return false;
    if (perSm < 1) return fail(error, "fused decode kernel does not fit on an SM");
    const int grid = ctx->smCount;
    if (host) {
        a.hostY = host->hostY;
        a.mailbox = host->mailbox;
        a.epoch = host->epoch;
    }
    LaunchScope scope(ctx, stream, "decode_fused");
    if (host && host->inlineX) {
        if (c.d > 4096) return fail(error, "input row too long to travel in the kernel parameters");
        static thread_local InlineRow row;
        memcpy(&row, host->inlineX, (size_t)c.d * 2);
        void *params[] = {&a, &maps, &row};
        FF_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(k_decode_fused_inline_x),
                                               dim3(grid), dim3(kFusedThreads), params, smem, stream),
                   error);
    } else {
        void *params[] = {&a, &maps};
        FF_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(k_decode_fused), dim3(grid),
                                               dim3(kFusedThreads), params, smem, stream),
                   error);
    }
    return true;
}

}  // namespace ff
