// Prefill path of the INT4 MoE block: router for many rows, device-side permute (counting sort by
// expert), and the grouped INT4 -> bf16 GEMMs on the 5th-generation tensor cores.
//
// GEMM scheme.  A work unit is (row tile of up to 128 expert-sorted rows, column tile of 256
// outputs: 128 gate + 128 up rows, or 256 down rows).  The wide column tile halves the re-reads of
// the activation tile from L2, which bound the narrower tilings.  Per 64-wide step along the contraction (= one quantization group):
//   * one thread issues TMA loads: the activations' [128 x 64] bf16 tile (128-byte swizzle) and
//     four [64 rows x 32 bytes] tiles of packed 4-bit codes, completing on an mbarrier;
//   * sixteen warps turn the packed tile into the bf16 operand tile in shared memory, half a
//     weight row per thread: codes -> bf16 pairs by a mask trick, then one bf16x2 fused multiply-add
//     with the group's scale and bias (a single rounding of q*scale+bias), stored in the
//     128-byte-swizzled K-major layout the MMA descriptor expects;
//   * one thread issues four tcgen05.mma (M=128, N=256, K=16) accumulating in TMEM, then
//     tcgen05.commit to free the stage;
//   * four warps drain the finished accumulator from TMEM (tcgen05.ld), apply the epilogue
//     (GeGLU to bf16 activations, or bf16 partial rows scattered to (token, rank)), while the
//     next unit's MMAs fill the other accumulator buffer.
// Within every aligned run of eight contraction elements the order is 0,4,1,5,2,6,3,7 in BOTH
// operands (the mask trick yields codes j and j+4 side by side), which leaves every dot product
// unchanged; the activation buffers this file writes use that order.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the context's error flag and
// the whole CTA leaves its loops, frees its TMEM and returns.
//
// Reference kernels this file stands in for (paths inside the reference project):
//   Sources/ANEFieldfareHotpath/Metal/Prefill/prefill.metal:447-542 (router block),
//   :609-779 (routed experts as tiled matrix multiplies),
//   Sources/ANEFieldfareHotpath/Metal/TensorCore/tensorops.metal:14-298 (dense INT4 GEMM),
//   Sources/ANEFieldfareHotpath/Kernels/Prefill/MoE/PrefillMoEGrouping.swift:49-110 (the sort).
#include <algorithm>
#include <cstring>

#include "ff_gemv_device.cuh"
#include "ff_internal.cuh"

namespace ff {

// ---- small device helpers --------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- router for many rows ------------------------------------------------------------------

// For every expert the logit is formed in the order the decode router uses (lane l chains fmaf
// over [256 i + 8 l, +8) for i ascending, butterfly 16..1, then the logit bias), so logits and
// indices are bitwise those of the single-row kernel.  Then the warp-wide top-K.
//
// A warp owns kTok tokens and walks the experts eight at a time with a register tile of
// kTok x 8 running sums.  The tokens' inputs sit in shared memory as bf16 for the whole kernel;
// the router rows stream through a small ring, one [8 experts x 256 inputs] block per copy (a
// tiled bulk tensor copy issued by a producer warp, completion on an mbarrier), in exactly the
// order the chains consume them: block i of a slice holds, for lane l, its eight elements of
// step i.  Per block a lane turns the 8 x 8 router values and its kTok x 8 inputs into fp32 once
// and issues 8 x kTok x 8 fmaf, element by element over all chains, so consecutive fmaf are
// independent.  A CTA takes 32 tokens (4096 tokens = 128 CTAs, one wave); shared memory holds
// their inputs whatever the split into warps, and the split that measured best is sixteen warps of
// two tokens (four warps per scheduler hide the shared-memory and conversion latencies): 164 us
// for 4096 tokens, against 182 us with eight warps of four, 214 us with four warps of eight, and
// 197 us for the previous kernel (whole eight-expert slices in shared memory, four tokens per
// warp, four warps per SM in two waves, packed FMAs fed by three integer-pipe cycles of conversions
// each).  In-kernel cycle counts: the chains 135 us of which 10 % waiting for blocks, top-K 15 us.
constexpr int kRouterTokensPerCta = 32;  // computing warps x tokens per warp (one more warp issues the copies)
constexpr int kRouterExperts = 8;   // experts per slice = rows of a streamed block
constexpr int kRouterBlockK = 256;  // inputs per streamed block: one step of every lane's chain
constexpr int kRouterRing = 8;      // blocks in flight
constexpr uint32_t kRouterBlockBytes = kRouterExperts * kRouterBlockK * 2;

__device__ __forceinline__ bool rt_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
static __device__ __noinline__ bool rt_wait_slow(uint32_t bar, uint32_t parity) {
    bool done = false;
    for (uint32_t spin = 0; spin < (1u << 22) && !done; ++spin) done = rt_try_wait(bar, parity);
    return done;
}
// bounded; the first poll stands alone (inside the bounded loop it costs about 200 cycles even
// when the barrier is complete)
__device__ __forceinline__ bool rt_wait(uint32_t bar, uint32_t parity) {
    return rt_try_wait(bar, parity) || rt_wait_slow(bar, parity);
}

template <int kTok>
__global__ void __launch_bounds__((kRouterTokensPerCta / kTok + 1) * 32)
k_router_rows(const __grid_constant__ CUtensorMap mapW, const uint16_t *scale, const float *bias,
              const uint16_t *gain, const uint16_t *x, uint32_t xStride, int T, int E, int D, int K,
              uint32_t *ids, uint16_t *weights, float *logitsOut, uint32_t *errorFlag) {
    constexpr int kRouterWarps = kRouterTokensPerCta / kTok;
    extern __shared__ __align__(128) uint8_t rsmRaw[];
    __shared__ __align__(8) uint64_t ringBar[2 * kRouterRing];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // ring of router blocks, then per computing warp: kTok input rows as bf16 and kTok x E logits
    const size_t perWarp = (size_t)kTok * D * 2 + (size_t)kTok * E * 4;
    const uint32_t ringAddr = (uint32_t)__cvta_generic_to_shared(rsmRaw);
    const uint32_t barBase = (uint32_t)__cvta_generic_to_shared(&ringBar[0]);
    auto barFull = [&](int s) { return barBase + 8u * (uint32_t)s; };
    auto barEmpty = [&](int s) { return barBase + 8u * (uint32_t)(kRouterRing + s); };
    const int nSlices = (E + kRouterExperts - 1) / kRouterExperts;
    const int nBlocks = (D + kRouterBlockK - 1) / kRouterBlockK;
    if (threadIdx.x == 0) {
        for (int st = 0; st < kRouterRing; ++st) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barFull(st)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(barEmpty(st)), "r"(kRouterWarps) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kRouterWarps) {
        // ---- producer: every block of every slice, in consumption order ----
        if (lane == 0) {
            uint32_t st = 0, phase = 0;
            bool ok = true;
            for (int sl = 0; sl < nSlices && ok; ++sl)
                for (int i = 0; i < nBlocks; ++i) {
                    if (!rt_wait(barEmpty(st), phase ^ 1u)) {
                        atomicExch(errorFlag, 11u);
                        ok = false;
                        break;
                    }
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barFull(st)),
                                 "r"(kRouterBlockBytes)
                                 : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                        " [%0], [%1, {%2, %3}], [%4];" ::"r"(ringAddr + st * kRouterBlockBytes),
                        "l"(reinterpret_cast<uint64_t>(&mapW)), "r"(i * kRouterBlockK), "r"(sl * kRouterExperts),
                        "r"(barFull(st))
                        : "memory");
                    if (++st == kRouterRing) {
                        st = 0;
                        phase ^= 1u;
                    }
                }
        }
        return;
    }

    uint8_t *warpBase = rsmRaw + (size_t)kRouterRing * kRouterBlockBytes + warp * perWarp;
    uint16_t *xs = reinterpret_cast<uint16_t *>(warpBase);
    float *lg = reinterpret_cast<float *>(warpBase + (size_t)kTok * D * 2);
    const int t0 = (blockIdx.x * kRouterWarps + warp) * kTok;
    const int nTok = max(0, min(kTok, T - t0));
    for (int tt = 0; tt < kTok; ++tt) {
        const uint16_t *xr = x + (size_t)min(t0 + min(tt, max(nTok, 1) - 1), T - 1) * xStride;
        for (int i = lane * 8; i < D; i += 256)
            *reinterpret_cast<uint4 *>(xs + (size_t)tt * D + i) = *reinterpret_cast<const uint4 *>(xr + i);
    }
    __syncwarp();

    uint32_t st = 0, phase = 0;
    bool ok = true;
    for (int sl = 0; sl < nSlices && ok; ++sl) {
        float acc[kTok][kRouterExperts];
#pragma unroll
        for (int t = 0; t < kTok; ++t)
#pragma unroll
            for (int e = 0; e < kRouterExperts; ++e) acc[t][e] = 0.0f;
        for (int i = 0; i < nBlocks; ++i) {
            if (!rt_wait(barFull(st), phase)) {
                if (lane == 0) atomicExch(errorFlag, 11u);
                ok = false;
                break;
            }
            const int base = i * kRouterBlockK + 8 * lane;
            if (base < D) {
                float xv[kTok][8];
                uint4 sv = make_uint4(0, 0, 0, 0);
                if (scale) sv = *reinterpret_cast<const uint4 *>(scale + base);
                const uint32_t ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                for (int t = 0; t < kTok; ++t) {
                    const uint4 raw = *reinterpret_cast<const uint4 *>(xs + (size_t)t * D + base);
                    const uint32_t xr[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float a0 = __uint_as_float(xr[k] << 16), a1 = __uint_as_float(xr[k] & 0xFFFF0000u);
                        if (scale) {
                            a0 = a0 * __uint_as_float(ss[k] << 16);
                            a1 = a1 * __uint_as_float(ss[k] & 0xFFFF0000u);
                        }
                        xv[t][2 * k] = a0;
                        xv[t][2 * k + 1] = a1;
                    }
                }
                const uint8_t *blockPtr = rsmRaw + (size_t)st * kRouterBlockBytes;
                float wv[kRouterExperts][8];
#pragma unroll
                for (int e = 0; e < kRouterExperts; ++e) {
                    const uint4 raw = *reinterpret_cast<const uint4 *>(blockPtr + (size_t)e * (kRouterBlockK * 2) + lane * 16);
                    const uint32_t ww[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        wv[e][2 * k] = __uint_as_float(ww[k] << 16);
                        wv[e][2 * k + 1] = __uint_as_float(ww[k] & 0xFFFF0000u);
                    }
                }
                // element by element, all (token, expert) chains side by side: consecutive fmaf are
                // independent, every chain still takes its eight elements in ascending order
#pragma unroll
                for (int k = 0; k < 8; ++k)
#pragma unroll
                    for (int e = 0; e < kRouterExperts; ++e)
#pragma unroll
                        for (int t = 0; t < kTok; ++t) acc[t][e] = fmaf(wv[e][k], xv[t][k], acc[t][e]);
            }
            // this warp is done with the block
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(barEmpty(st)) : "memory");
            if (++st == kRouterRing) {
                st = 0;
                phase ^= 1u;
            }
        }
        if (!ok) break;
#pragma unroll
        for (int t = 0; t < kTok; ++t)
#pragma unroll
            for (int e = 0; e < kRouterExperts; ++e) {
                float v = acc[t][e];
#pragma unroll
                for (int offset = 16; offset >= 1; offset >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, offset);
                const int ex = sl * kRouterExperts + e;
                if (lane == 0 && ex < E) lg[t * E + ex] = bias ? v + bias[ex] : v;
            }
    }
    __syncwarp();
    for (int tt = 0; tt < nTok; ++tt) {
        const int t = t0 + tt;
        if (logitsOut)
            for (int e = lane; e < E; e += 32) logitsOut[(size_t)t * E + e] = lg[tt * E + e];
        warp_topk(lg + tt * E, E, K, gain, ids + (size_t)t * K, weights + (size_t)t * K);
    }
}

static bool make_router_map(CUtensorMap *map, const void *base, uint64_t experts, uint64_t d, const char **error);

template <int kTok>
static bool launch_router_rows(FFContext *ctx, const LayerStore &L, const CUtensorMap &mapW, size_t smem,
                               const uint16_t *x, uint32_t xStride, uint32_t tokens, uint32_t *ids,
                               uint16_t *weights, float *logits, cudaStream_t stream, const char **error) {
    const int E = (int)L.routerExperts, D = (int)ctx->cfg.d;
    constexpr int kThreads = (kRouterTokensPerCta / kTok + 1) * 32;
    static KernelSmemMemo memo;
    if (!memo.prepare(k_router_rows<kTok>, ctx->device, smem, kThreads, nullptr, error)) return false;
    const uint32_t perCta = kRouterTokensPerCta;
    {
        LaunchScope scope(ctx, stream, "router_rows");
        k_router_rows<kTok><<<(tokens + perCta - 1) / perCta, kThreads, smem, stream>>>(
            mapW, L.routerScale, L.logitBias, L.gain, x, xStride, (int)tokens, E, D, (int)ctx->cfg.topK, ids,
            weights, logits, ctx->errorFlag);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

bool launch_router_prefill(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                           uint32_t tokens, uint32_t *ids, uint16_t *weights, float *logits,
                           cudaStream_t stream, const char **error) {
    const int E = (int)L.routerExperts, D = (int)ctx->cfg.d;
    if (D % 8) return fail(error, "hidden size must be a multiple of 8");
    // a tiled copy descriptor over the router matrix, [8 experts x 256 inputs] boxes (built per call:
    // encoding is host arithmetic only)
    CUtensorMap mapW;
    if (!make_router_map(&mapW, L.routerW, (uint64_t)E, (uint64_t)D, error)) return false;
    // shared memory: the ring, and per CTA 32 tokens' inputs and logits whatever the split into warps
    const size_t smem = (size_t)kRouterRing * kRouterBlockBytes +
                        (size_t)kRouterTokensPerCta * ((size_t)D * 2 + (size_t)E * 4);
    if (smem > 226 * 1024) return fail(error, "model width too large for the router's shared memory");
    return launch_router_rows<2>(ctx, L, mapW, smem, x, xStride, tokens, ids, weights, logits, stream, error);
}

// ---- device-side permute -------------------------------------------------------------------

constexpr int kSortTokens = 256;  // tokens per permute block

constexpr uint32_t kRowTile = 192;  // rows of one expert per GEMM unit (accumulator columns)

struct RowTile {
    uint32_t rowStart;  // first row in expert-sorted order
    uint32_t rows;      // 1..kRowTile
    uint32_t expert;
    uint32_t pad;
};

// Per-warp segment histogram of a block's routes: warp w owns routes [w*seg, (w+1)*seg) of the
// block; lanes holding the same expert are grouped with match.any and the group's lowest lane adds
// the group size.  segCount is [8 warps][E] in shared memory, zeroed by the caller.
__device__ __forceinline__ void segment_histogram(const uint32_t *routes, int n, int seg, int E,
                                                  uint32_t *segCount) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int begin = warp * seg, end = min(n, begin + seg);
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        const bool valid = i < end;
        const uint32_t e = valid ? routes[i] : 0xFFFFFFFFu;
        const uint32_t mask = __match_any_sync(0xFFFFFFFFu, e);
        if (valid && e < (uint32_t)E && (mask & ((1u << lane) - 1u)) == 0u)
            segCount[warp * E + e] += (uint32_t)__popc(mask);
        __syncwarp();
    }
}

// Pass 1: per block of 256 tokens, how many routes name each expert.
__global__ void __launch_bounds__(256)
k_route_count(const uint32_t *ids, int T, int K, int E, uint32_t *blockCounts) {
    extern __shared__ uint32_t sRoutes[];
    __shared__ uint32_t segCount[8 * kMaxExperts];
    const int t0 = blockIdx.x * kSortTokens;
    const int n = min(kSortTokens, T - t0) * K;
    for (int i = threadIdx.x; i < n; i += blockDim.x) sRoutes[i] = ids[(size_t)t0 * K + i];
    for (int i = threadIdx.x; i < 8 * E; i += blockDim.x) segCount[i] = 0;
    __syncthreads();
    segment_histogram(sRoutes, n, (n + 7) / 8, E, segCount);
    __syncthreads();
    const int e = threadIdx.x;
    if (e < E) {
        uint32_t c = 0;
        for (int w = 0; w < 8; ++w) c += segCount[w * E + e];
        blockCounts[(size_t)blockIdx.x * E + e] = c;
    }
}

// Pass 2 (one block): exclusive prefix of every expert's counts over the blocks, expert offsets,
// and the list of row tiles (up to kRowTile rows of one expert each), experts ascending.
// counts[0] = row tiles, counts[1] = pairs, counts[2] = experts with at least one pair.
__global__ void __launch_bounds__(256)
k_route_scan(uint32_t *blockCounts, int blocks, int E, uint32_t *expertOffsets, RowTile *tiles,
             uint32_t maxTiles, uint32_t *counts) {
    __shared__ uint32_t total[kMaxExperts];
    __shared__ uint32_t offset[kMaxExperts + 1];
    __shared__ uint32_t tileBase[kMaxExperts + 1];
    const int e = threadIdx.x;
    if (e < E) {
        // eight blocks' counts are fetched together (independent loads), then turned into prefixes
        uint32_t run = 0;
        for (int b0 = 0; b0 < blocks; b0 += 8) {
            uint32_t c[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) c[i] = b0 + i < blocks ? blockCounts[(size_t)(b0 + i) * E + e] : 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (b0 + i < blocks) {
                    blockCounts[(size_t)(b0 + i) * E + e] = run;
                    run += c[i];
                }
        }
        total[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0, tilesRun = 0, active = 0;
        for (int i = 0; i < E; ++i) {
            offset[i] = run;
            tileBase[i] = tilesRun;
            run += total[i];
            tilesRun += (total[i] + kRowTile - 1u) / kRowTile;
            active += total[i] ? 1u : 0u;
        }
        offset[E] = run;
        tileBase[E] = tilesRun;
        counts[0] = min(tilesRun, maxTiles);
        counts[1] = run;
        counts[2] = active;
        counts[3] = 0;
    }
    __syncthreads();
    if (e < E) expertOffsets[e] = offset[e];
    if (e == 0) expertOffsets[E] = offset[E];
    if (e < E) {
        const uint32_t n = total[e];
        for (uint32_t i = 0, tix = tileBase[e]; i < n; i += kRowTile, ++tix)
            if (tix < maxTiles) tiles[tix] = RowTile{offset[e] + i, min(kRowTile, n - i), (uint32_t)e, 0u};
    }
}

// Pass 3: every route's position in (expert, token, rank) order; writes the sorted pair list.
// Position = expert offset + routes to the expert in earlier blocks + in earlier warp segments of
// this block + earlier in this warp's segment (earlier 32-route batches, then lower lanes).
__global__ void __launch_bounds__(256)
k_route_scatter(const uint32_t *ids, const uint16_t *weights, int T, int K, int E,
                const uint32_t *blockCounts, const uint32_t *expertOffsets,
                FFTokenExpertPair *sorted) {
    extern __shared__ uint32_t sRoutes[];
    __shared__ uint32_t segCount[8 * kMaxExperts];
    const int t0 = blockIdx.x * kSortTokens;
    const int n = min(kSortTokens, T - t0) * K;
    for (int i = threadIdx.x; i < n; i += blockDim.x) sRoutes[i] = ids[(size_t)t0 * K + i];
    for (int i = threadIdx.x; i < 8 * E; i += blockDim.x) segCount[i] = 0;
    __syncthreads();
    const int seg = (n + 7) / 8;
    segment_histogram(sRoutes, n, seg, E, segCount);
    __syncthreads();
    const int e = threadIdx.x;
    if (e < E) {
        // turn the segment counts into each segment's first position for this expert
        uint32_t run = expertOffsets[e] + blockCounts[(size_t)blockIdx.x * E + e];
        for (int w = 0; w < 8; ++w) {
            const uint32_t c = segCount[w * E + e];
            segCount[w * E + e] = run;
            run += c;
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int begin = warp * seg, end = min(n, begin + seg);
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        const bool valid = i < end;
        const uint32_t ex = valid ? sRoutes[i] : 0xFFFFFFFFu;
        const uint32_t mask = __match_any_sync(0xFFFFFFFFu, ex);
        const bool live = valid && ex < (uint32_t)E;
        uint32_t pos = 0;
        if (live) pos = segCount[warp * E + ex] + (uint32_t)__popc(mask & ((1u << lane) - 1u));
        __syncwarp();
        if (live && (mask & ((1u << lane) - 1u)) == 0u) segCount[warp * E + ex] += (uint32_t)__popc(mask);
        __syncwarp();
        if (live) {
            const uint32_t token = (uint32_t)(t0 + i / K), rank = (uint32_t)(i % K);
            const uint32_t wbits = weights ? (uint32_t)weights[(size_t)token * K + rank] : 0u;
            sorted[pos] = FFTokenExpertPair{token, ex, rank, wbits};
        }
    }
}

// Row tiles of a dense problem: T rows of one "expert" (the shared FFN).
__global__ void k_dense_tiles(int T, RowTile *tiles, uint32_t *counts) {
    const int n = (T + (int)kRowTile - 1) / (int)kRowTile;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        tiles[i] = RowTile{(uint32_t)i * kRowTile, (uint32_t)min((int)kRowTile, T - i * (int)kRowTile), 0u, 0u};
    if (threadIdx.x == 0) {
        counts[0] = (uint32_t)n;
        counts[1] = (uint32_t)T;
        counts[2] = 1;
        counts[3] = 0;
    }
}

// Copies rows of x into the GEMM's activation buffer, reordering every aligned run of eight
// elements to 0,4,1,5,2,6,3,7.  pairs == null: row r of the output is row r of x; otherwise row r
// is the token of sorted pair r.  One thread per 16 bytes.
__global__ void __launch_bounds__(256)
k_gather_rows(const uint16_t *x, uint32_t xStride, const FFTokenExpertPair *pairs,
              const uint32_t *rowCountPtr, uint32_t rowCount, int D, uint16_t *out) {
    const uint32_t rows = rowCountPtr ? rowCountPtr[1] : rowCount;
    const int chunksPerRow = D / 8;
    const size_t total = (size_t)rows * chunksPerRow;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / chunksPerRow);
        const int c = (int)(i - (size_t)r * chunksPerRow);
        const uint32_t src = pairs ? pairs[r].token : r;
        const uint4 v = *reinterpret_cast<const uint4 *>(x + (size_t)src * xStride + c * 8);
        // halves h0..h7 -> h0,h4,h1,h5,h2,h6,h3,h7
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410);
        o.y = __byte_perm(v.x, v.z, 0x7632);
        o.z = __byte_perm(v.y, v.w, 0x5410);
        o.w = __byte_perm(v.y, v.w, 0x7632);
        *reinterpret_cast<uint4 *>(out + (size_t)r * D + c * 8) = o;
    }
}

// ---- tcgen05 / TMA / mbarrier wrappers ------------------------------------------------------

constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out or another thread of the CTA gave up; the
// caller leaves its loop.  `abortFlag` lives in shared memory.  kSleep: pause between polls, for
// the warps whose polling would otherwise take issue slots from the dequantizing warps.
// The first poll stands alone in front of the loop: measured on the device, a wait that finds its
// barrier already complete costs 7 cycles this way and about 200 when the poll sits inside the
// bounded loop.
template <bool kSleep>
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t *abortFlag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (kSleep) __nanosleep(40);
        if ((i & 255u) == 255u && *abortFlag) return false;
    }
    *abortFlag = 1u;
    return false;
}
template <bool kSleep>
__device__ __forceinline__ bool mbar_wait_impl(uint32_t bar, uint32_t parity, volatile uint32_t *abortFlag) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow<kSleep>(bar, parity, abortFlag);
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abortFlag) {
    return mbar_wait_impl<false>(bar, parity, abortFlag);
}
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar, uint32_t parity, volatile uint32_t *abortFlag) {
    return mbar_wait_impl<true>(bar, parity, abortFlag);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_generic_to_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tc_load_32cols(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 tile stored with the 128-byte swizzle:
// rows are 128 bytes apart, groups of eight rows 1024 bytes apart (stride byte offset), the
// leading byte offset is unused for swizzled K-major tiles (set to 1), descriptor version 1,
// layout type 2 (128-byte swizzle).  The tile base must be 1024-byte aligned; `byteOffset`
// advances along K inside the swizzle atom (32 bytes per K=16 slice).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smemAddr) {
    uint64_t desc = (uint64_t)((smemAddr & 0x3FFFFu) >> 4);
    desc |= (uint64_t)1 << 16;
    desc |= (uint64_t)(1024 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}
// Instruction descriptor: fp32 accumulate, bf16 A and B, both K-major, M = 256 (128 rows in
// either CTA of the pair), N = `n` (a multiple of 32 up to 256, half of it in either CTA).
__device__ __forceinline__ uint32_t umma_idesc_bf16_m256(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem] over the CTA pair: in either CTA, A is 128 lanes x 16 bf16
// (eight 32-bit columns per lane), B half of the N rows, D 128 lanes x N columns.
__device__ __forceinline__ void tc_mma_bf16_a_tmem(uint32_t tmemD, uint32_t tmemA, uint64_t descB,
                                                   uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmemD),
        "r"(tmemA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tc_store_32cols(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// ---- two CTAs of a cluster working as one tensor-core unit (cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the shared::cluster address of `addr` (a shared-memory address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
// arrive on a barrier that may live in the other CTA of the pair (`clusterAddr` from map_to_cta)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t clusterAddr) {
    // (default semantics, release at CTA scope: a cluster-scope release holds the warp until everything it
    // has in flight is acknowledged, over a thousand cycles here; what the other CTA's MMA reads
    // from this CTA is ordered by the tcgen05 fences and the TMA's own barrier, not by this arrive)
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait on a barrier that the other CTA of the pair arrives on
template <bool kSleep>
__device__ __noinline__ bool mbar_wait_cluster_slow(uint32_t bar, uint32_t parity, volatile uint32_t *abortFlag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (kSleep) __nanosleep(40);
        if ((i & 255u) == 255u && *abortFlag) return false;
    }
    *abortFlag = 1u;
    return false;
}
template <bool kSleep>
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t *abortFlag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    return mbar_wait_cluster_slow<kSleep>(bar, parity, abortFlag);
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// This CTA's part of a tile that the pair's MMA reads from both CTAs; completes on the leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y,
                                                 uint32_t leaderBar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leaderBar)
        : "memory");
}
// arrives once on the barrier at this shared-memory offset in both CTAs when the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"((uint16_t)3)
        : "memory");
}

// ---- grouped INT4 GEMM ---------------------------------------------------------------------

constexpr int kWeightRows = 128;  // weight rows of a unit = TMEM lanes of its accumulator
constexpr int kTileK = 64;        // one quantization group per step
constexpr int kTokStages = 8;     // token half tiles (TMA destinations)
constexpr int kPackStages = 8;    // packed-code tiles (TMA destinations)
constexpr int kGroups = 4;        // dequantizing groups
constexpr int kWStages = kGroups; // dequantized weight tiles in TMEM, one per dequantizing group
constexpr int kDequantWarps = 16; // four groups of four warps; a group covers the 128 TMEM lanes
// warp 0 TMA, warp 1 MMA, warps 2-17 dequantize, warps 18-21 epilogue (TMEM lane quarter = warp & 3)
constexpr int kGemmThreads = (2 + kDequantWarps + 4) * 32;
constexpr uint32_t kTokHalfRows = kRowTile / 2;                   // rows of a token tile held by either CTA of a pair
constexpr uint32_t kTokTileBytes = kTokHalfRows * kTileK * 2;     // 12288 (a multiple of the 1024-byte swizzle atom)
constexpr uint32_t kPackTileBytes = kWeightRows * kTileK / 2;     // 4096: two [64 rows x 32 bytes] boxes
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccCols = kRowTile;                           // accumulators at columns 0 and 192
constexpr uint32_t kWCol0 = 2 * kAccCols;                         // weight stages: 32 columns each from 384
constexpr int kXchgPitch = 17;                                    // floats per exchanged row (16 + 1 pad)
constexpr uint32_t kXchgBytes = 2u * 128u * kXchgPitch * 4u;      // two buffers x 128 rows
constexpr uint32_t kStagePitchGateUp = 64 * 2 + 16;               // bytes per token row of the output tile
constexpr uint32_t kStagePitchDown = 128 * 2 + 16;
constexpr uint32_t kStageBytesGateUp = 32u * kStagePitchGateUp;   // one 32-token output tile
constexpr uint32_t kStageBytesDown = 32u * kStagePitchDown;
// gate/up: exchange buffers + two output tiles; down: two output tiles + two row tables
constexpr uint32_t kEpilogueBytesGateUp = kXchgBytes + 2u * kStageBytesGateUp;
constexpr uint32_t kEpilogueBytesDown = 2u * kStageBytesDown + 2u * kRowTile * 4u;
static_assert(kWCol0 + kWStages * 32 <= kTmemCols, "tensor memory layout");
static_assert(kRowTile % 32 == 0 && kRowTile <= 256, "row tile");

enum GemmMode : int { kModeGateUp = 0, kModeDown = 1 };

struct GemmArgs {
    const uint8_t *blobBase;   // expert 0's blob
    uint64_t expertStride;
    uint32_t scaleOff[2];      // byte offsets of the scales of matrix 0 / 1 inside a blob
    uint32_t biasOff[2];
    uint32_t K;                // contraction length (multiple of 64)
    uint32_t N;                // outputs per row: F (gate/up) or D (down)
    uint32_t nTiles;           // weight-row tiles: ceil(N/64) for gate/up, ceil(N/128) for down
    const RowTile *tiles;
    const uint32_t *counts;    // counts[0] = row tiles
    uint16_t *out;             // gate/up: activations [row][N]; down: output rows [*][N]
    const FFTokenExpertPair *pairs;  // down: row -> (token, rank); null: row -> row
    uint32_t topK;
    uint32_t roundGateUp;      // gate/up: round both to bf16 before the activation
    uint32_t *errorFlag;
};

// position of element i of an aligned run of eight in the order 0,4,1,5,2,6,3,7
__device__ __forceinline__ uint32_t interleaved_position(uint32_t i) {
    return (i & ~7u) | (((i & 3u) << 1) | ((i >> 2) & 1u));
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
k_grouped_int4_gemm(const __grid_constant__ CUtensorMap mapTok, const __grid_constant__ CUtensorMap mapW0,
                    const __grid_constant__ CUtensorMap mapW1, const GemmArgs args) {
    extern __shared__ uint8_t gemmSmemRaw[];
    __shared__ uint64_t barriers[2 * kTokStages + 2 * kPackStages + 2 * kWStages + 4 + 5];
    __shared__ uint32_t tmemBaseSlot;
    __shared__ volatile uint32_t abortFlag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rawBase = smem_u32(gemmSmemRaw);
    const uint32_t base = (rawBase + 1023u) & ~1023u;
    const uint32_t groupsK = args.K / kTileK;

    // carve-up: token stages (1024-aligned), packed stages, the epilogue's exchange buffers
    // (stage addresses are computed, not tabulated: an array indexed by the running stage would
    // live in local memory)
    const uint32_t tokBase = base, packBase = tokBase + kTokStages * kTokTileBytes;
    auto tokAddrOf = [&](uint32_t s) { return tokBase + s * kTokTileBytes; };
    auto packAddrOf = [&](uint32_t s) { return packBase + s * kPackTileBytes; };
    uint8_t *epilogueSmem = gemmSmemRaw + (packBase + kPackStages * kPackTileBytes - rawBase);
    constexpr uint32_t kStageBytes = MODE == kModeGateUp ? kStageBytesGateUp : kStageBytesDown;
    float *xchg = reinterpret_cast<float *>(epilogueSmem);                                 // gate/up only
    uint8_t *stageBuf = epilogueSmem + (MODE == kModeGateUp ? kXchgBytes : 0u);
    uint32_t *rowTable = reinterpret_cast<uint32_t *>(stageBuf + 2u * kStageBytes);        // down only
    uint32_t *scaleSlots = reinterpret_cast<uint32_t *>(
        epilogueSmem + (MODE == kModeGateUp ? kEpilogueBytesGateUp : kEpilogueBytesDown));  // [ceil(groupsK/4)][512]

    const uint32_t barBase = smem_u32(barriers);
    auto barAt = [&](int i) { return barBase + 8u * (uint32_t)i; };
    auto barTokFull = [&](int s) { return barAt(s); };
    auto barTokEmpty = [&](int s) { return barAt(kTokStages + s); };
    auto barPackFull = [&](int s) { return barAt(2 * kTokStages + s); };
    auto barPackEmpty = [&](int s) { return barAt(2 * kTokStages + kPackStages + s); };
    auto barWFull = [&](int s) { return barAt(2 * kTokStages + 2 * kPackStages + s); };
    auto barWEmpty = [&](int s) { return barAt(2 * kTokStages + 2 * kPackStages + kWStages + s); };
    auto barAccFull = [&](int s) { return barAt(2 * kTokStages + 2 * kPackStages + 2 * kWStages + s); };
    auto barAccEmpty = [&](int s) { return barAt(2 * kTokStages + 2 * kPackStages + 2 * kWStages + 2 + s); };
    auto barXchg = [&](int s) { return barAt(2 * kTokStages + 2 * kPackStages + 2 * kWStages + 4 + s); };
    auto barStage = [&](int s) { return barAt(2 * kTokStages + 2 * kPackStages + 2 * kWStages + 6 + s); };
    const uint32_t barRows = barAt(2 * kTokStages + 2 * kPackStages + 2 * kWStages + 8);

    // The two CTAs of a cluster work as one unit of the tensor core: the leader (rank 0) issues
    // the MMAs for both.  Barriers that say "full" to the MMA issuer live in the leader and count
    // both CTAs' arrivals; barriers that the MMAs' completion frees exist in either CTA and are
    // signalled in both by one multicast commit.
    const uint32_t ctaRank = cluster_cta_rank();
    const bool leader = ctaRank == 0u;
    if (threadIdx.x == 0) {
        abortFlag = 0;
        for (int s = 0; s < kTokStages; ++s) {
            mbar_init(barTokFull(s), 1);
            mbar_init(barTokEmpty(s), 1);  // one tcgen05.commit
        }
        for (int s = 0; s < kPackStages; ++s) {
            mbar_init(barPackFull(s), 1);
            mbar_init(barPackEmpty(s), 4);  // the four warps of the group that read it
        }
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(barWFull(s), 8);   // (leader's is used) the four warps of the group in either CTA
            mbar_init(barWEmpty(s), 1);  // (unused: the weight stages are released through the token ring)
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(barAccFull(s), 1);   // one tcgen05.commit
            mbar_init(barAccEmpty(s), 8);  // (leader's is used) four epilogue warps in either CTA
            mbar_init(barXchg(s), 128);    // every epilogue thread
            mbar_init(barStage(s), 128);
        }
        mbar_init(barRows, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&tmemBaseSlot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the other CTA's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmemBase = tmemBaseSlot;

    // A pair's unit: one row tile, two neighbouring weight-row tiles (this CTA takes 2 np + rank).
    const uint32_t rowTiles = args.counts[0];
    const uint32_t nPairs = (args.nTiles + 1u) >> 1;
    const uint32_t units = rowTiles * nPairs;
    const uint32_t firstUnit = blockIdx.x >> 1, unitStride = gridDim.x >> 1;
    auto tileOf = [&](uint32_t u) { return args.tiles[u / nPairs]; };
    auto ntOf = [&](uint32_t u) { return 2u * (u % nPairs) + ctaRank; };
    // accumulator columns of a tile: its rows to the next multiple of 32, half of them in either CTA
    auto columnsOf = [&](const RowTile &tile) { return max(32u, (tile.rows + 31u) & ~31u); };
    // weight rows 0..127 of a unit: gate rows [64 nt, +64) | up rows [64 nt, +64) for the gate/up
    // GEMM, matrix rows [128 nt, +128) for the down GEMM; loaded as two boxes of 64 rows

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t ts = 0, tPhase = 0, ps = 0, pPhase = 0;
            bool ok = true;
            for (uint32_t u = firstUnit; u < units && ok; u += unitStride) {
                const RowTile tile = tileOf(u);
                const uint32_t nt = ntOf(u);
                // this CTA's half of the tile's rows
                const int row0 = (int)(tile.rowStart + ctaRank * (columnsOf(tile) >> 1));
                for (uint32_t g = 0; g < groupsK; ++g) {
                    if (!mbar_wait_idle(barPackEmpty(ps), pPhase ^ 1u, &abortFlag)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(barPackFull(ps), kPackTileBytes);
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const CUtensorMap *map = (MODE == kModeGateUp && q == 1) ? &mapW1 : &mapW0;
                        const int wRow = MODE == kModeGateUp ? (int)nt * 64 : (int)nt * 128 + q * 64;
                        tma_load_3d(packAddrOf(ps) + (uint32_t)q * (kPackTileBytes / 2), map,
                                    (int)(g * (kTileK / 2)), wRow, (int)tile.expert, barPackFull(ps));
                    }
                    if (++ps == kPackStages) {
                        ps = 0;
                        pPhase ^= 1u;
                    }
                    if (!mbar_wait_idle(barTokEmpty(ts), tPhase ^ 1u, &abortFlag)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(barTokFull(ts), kTokTileBytes);
                    tma_load_2d(tokAddrOf(ts), &mapTok, (int)(g * kTileK), row0, barTokFull(ts));
                    if (++ts == kTokStages) {
                        ts = 0;
                        tPhase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && leader) {
            uint32_t ts = 0, ws = 0, wPhase = 0, acc = 0, accPhase = 0;
            bool ok = true;
            for (uint32_t u = firstUnit; u < units && ok; u += unitStride) {
                const RowTile tile = tileOf(u);
                const uint32_t idesc = umma_idesc_bf16_m256(columnsOf(tile));
                if (!mbar_wait_cluster<true>(barAccEmpty(acc), accPhase ^ 1u, &abortFlag)) break;
                tc_fence_after();
                const uint32_t tmemD = tmemBase + acc * kAccCols;
                for (uint32_t g = 0; g < groupsK; ++g) {
                    // (the group that arrives here has also seen both token halves land)
                    if (!mbar_wait_cluster<false>(barWFull(ws), wPhase, &abortFlag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t descTok = umma_desc_sw128(tokAddrOf(ts));
                    const uint32_t tmemW = tmemBase + kWCol0 + ws * 32u;
#pragma unroll
                    for (uint32_t kk = 0; kk < kTileK / 16; ++kk) {
                        // per 16-element slice: eight columns further in TMEM, 32 bytes (>> 4 = 2)
                        // further in the token tile
                        tc_mma_bf16_a_tmem(tmemD, tmemW + 8u * kk, descTok + 2u * kk, idesc,
                                           (g | kk) != 0u ? 1u : 0u);
                    }
                    // one signal per step: the token stage is free, and so is the weight stage that
                    // the same step used (the dequantizers wait on the token ring's barrier, too)
                    tc_commit_pair(barTokEmpty(ts));
                    if (++ts == kTokStages) ts = 0;
                    if (++ws == kWStages) {
                        ws = 0;
                        wPhase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit_pair(barAccFull(acc));
                if (++acc == 2) {
                    acc = 0;
                    accPhase ^= 1u;
                }
            }
        }
    } else if (warp < 2 + kDequantWarps) {
        // ---------------- dequantizers ----------------
        // Group `grp` (four warps, one per TMEM lane quarter) takes every fourth step of the CTA's
        // sequence of steps and owns weight stage `grp`; a thread turns one weight row's 64 codes
        // of the step into 32 bf16 pairs and stores them to its TMEM lane.  Four steps are in
        // work at once, which hides a step's latencies behind the other groups' arithmetic.
        const uint32_t grp = (uint32_t)(warp - 2) >> 2;
        const uint32_t m = (uint32_t)(warp & 3) * 32u + (uint32_t)lane;  // weight row of the unit = TMEM lane
        const uint32_t tmemW = tmemBase + kWCol0 + grp * 32u + (((uint32_t)(warp & 3) * 32u) << 16);
        const uint32_t matrix = MODE == kModeGateUp ? (m >> 6) : 0u;

        // The thread's scale/bias pairs of a unit (one per step it takes there) are fetched in one
        // batch when it enters the unit and kept in a private column of shared memory, so that no
        // global load is in flight in the steady loop (a load in flight would hold up the
        // releasing arrive below for the load's whole latency).
        uint32_t *myScales = scaleSlots + (uint32_t)(threadIdx.x - 64);  // [slot][512 threads]
        uint32_t u = firstUnit, g = grp;   // the thread's current step: unit and step inside it
        uint32_t gFirst = 0;               // its first step inside the current unit
        auto enter_unit = [&]() {          // after u or g changed so that g < groupsK again, or at the start
            while (g >= groupsK && u < units) {
                g -= groupsK;
                u += unitStride;
            }
            gFirst = g;
            if (u >= units) return;
            const RowTile tile = tileOf(u);
            const uint32_t nt = ntOf(u);
            const uint32_t wRow = MODE == kModeGateUp ? nt * 64u + (m & 63u) : nt * 128u + m;
            const bool liveRow = wRow < args.N;
            const uint8_t *blob = args.blobBase + (size_t)tile.expert * args.expertStride;
            // (selected, not indexed: a run-time index into the parameters would copy them to local memory)
            const uint32_t scaleOff = matrix ? args.scaleOff[1] : args.scaleOff[0];
            const uint32_t biasOff = matrix ? args.biasOff[1] : args.biasOff[0];
            const uint16_t *sg = reinterpret_cast<const uint16_t *>(blob + scaleOff) + (size_t)wRow * groupsK;
            const uint16_t *bg = reinterpret_cast<const uint16_t *>(blob + biasOff) + (size_t)wRow * groupsK;
            for (uint32_t i0 = 0; g + 4u * i0 < groupsK; i0 += 4) {
                uint32_t v[4];
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const uint32_t gi = min(g + 4u * (i0 + i), groupsK - 1u);
                    v[i] = liveRow ? ((uint32_t)__ldg(sg + gi) | ((uint32_t)__ldg(bg + gi) << 16)) : 0u;
                }
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i)
                    if (g + 4u * (i0 + i) < groupsK) myScales[(i0 + i) * (uint32_t)(kDequantWarps * 32)] = v[i];
            }
        };
        enter_unit();
        const uint32_t leaderWFull = map_to_cta(barWFull(grp), 0u);
        static_assert(kTokStages == kPackStages, "the dequantizers use one ring index for both");
        uint32_t ps = grp % kPackStages, pPhase = 0, ownSteps = 0;
        while (u < units) {
            const uint32_t sb = myScales[((g - gFirst) >> 2) * (uint32_t)(kDequantWarps * 32)];
            // The weight stage `grp` was last read by the MMAs of this group's previous step, four
            // steps back: its completion is that step's signal on the token ring (stage ps - 4,
            // which in a ring of eight is ps + 4; the group's n-th step, n >= 1, meets that
            // barrier's completion number (n - 1) / 2).
            static_assert(kTokStages == 2 * kWStages, "the weight stages are released through the token ring");
            if (!mbar_wait(barPackFull(ps), pPhase, &abortFlag) ||
                (ownSteps && !mbar_wait(barTokEmpty((ps + kWStages) % kTokStages), ((ownSteps - 1u) >> 1) & 1u, &abortFlag)))
                break;
            tc_fence_after();

            uint32_t s2, b2;
            asm("prmt.b32 %0, %1, %1, 0x1010;" : "=r"(s2) : "r"(sb));
            asm("prmt.b32 %0, %1, %1, 0x3232;" : "=r"(b2) : "r"(sb));
            uint32_t w[8];
            const uint32_t src = packAddrOf(ps) + m * 32u;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                         : "r"(src));
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                         : "r"(src + 16u));
            uint32_t o[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // codes i and i+4 of the word as the bf16 pair (128+q_i, 128+q_{i+4})
                    uint32_t pair = ((w[j] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
                    uint32_t q2, v2;
                    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(q2) : "r"(pair), "r"(0x43004300u));
                    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(v2) : "r"(q2), "r"(s2), "r"(b2));
                    o[j * 4 + i] = v2;
                }
            }
            tc_store_32cols(tmemW, o);
            // this CTA's half of the step's token tile must have landed before the MMA is told to go
            const bool landed = mbar_wait(barTokFull(ps), pPhase, &abortFlag);
            tc_wait_st();
            if (!landed) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(leaderWFull);
                mbar_arrive(barPackEmpty(ps));
            }
            ps += kWStages;
            if (ps >= kPackStages) {
                ps -= kPackStages;
                pPhase ^= 1u;
            }
            ++ownSteps;
            g += kWStages;
            if (g >= groupsK) enter_unit();
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> shared -> global ----------------
        // A thread holds one weight row's results for the unit's tokens (one token per accumulator
        // column).  Per 32 tokens the four warps put their bf16 results into a [token][output]
        // tile in shared memory and then write it out a token row at a time, 16 bytes per thread.
        // All buffers alternate between two copies: a copy is rewritten two chunks (or units)
        // later, after every thread has passed a barrier in between, hence after it was read.
        const uint32_t quarter = (uint32_t)(warp & 3);
        const uint32_t m = quarter * 32u + (uint32_t)lane;
        const uint32_t t = (uint32_t)threadIdx.x - (2u + kDequantWarps) * 32u;  // 0..127
        uint32_t acc = 0, accPhase = 0, chunk = 0, unitNo = 0;
        bool ok = true;
        for (uint32_t u = firstUnit; u < units && ok; u += unitStride, ++unitNo) {
            const RowTile tile = tileOf(u);
            const uint32_t nt = ntOf(u);
            uint32_t *rowOf = rowTable + (unitNo & 1u) * kRowTile;
            if (MODE == kModeDown) {
                // where each of the unit's rows goes
                for (uint32_t r = t; r < tile.rows; r += 128u) {
                    uint32_t outRow = tile.rowStart + r;
                    if (args.pairs) {
                        const FFTokenExpertPair p = args.pairs[outRow];
                        outRow = p.token * args.topK + p.rank;
                    }
                    rowOf[r] = outRow;
                }
                mbar_arrive(barRows);
            }
            if (!mbar_wait_idle(barAccFull(acc), accPhase, &abortFlag)) break;
            if (MODE == kModeDown && !mbar_wait(barRows, unitNo & 1u, &abortFlag)) break;
            tc_fence_after();
            const uint32_t taddr = tmemBase + acc * kAccCols + ((quarter * 32u) << 16);
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < tile.rows; c0 += 32, ++chunk) {
                uint32_t v[32];
                tc_load_32cols(taddr + c0, v);
                tc_wait_ld();
                const uint32_t which = chunk & 1u, parity = (chunk >> 1) & 1u;
                uint8_t *stage = stageBuf + which * kStageBytes;
                if (MODE == kModeGateUp) {
                    // lanes 0..63 hold gate, lanes 64..127 up of features [64 nt, +64).  The gate
                    // warps hand the second 16 tokens' gates to the up warps and take the first 16
                    // tokens' ups from them; either side then finishes 16 tokens of its feature.
                    const bool isUp = m >= 64u;
                    float *buf = xchg + which * (128u * kXchgPitch);
                    float *mine = buf + m * kXchgPitch;
#pragma unroll
                    for (int j = 0; j < 16; ++j) mine[j] = __uint_as_float(isUp ? v[j] : v[16 + j]);
                    mbar_arrive(barXchg(which));
                    if (!mbar_wait(barXchg(which), parity, &abortFlag)) {
                        ok = false;
                        break;
                    }
                    const float *theirs = buf + (m ^ 64u) * kXchgPitch;
                    // tile [32 tokens][64 features in the interleaved order], 144-byte pitch
                    uint16_t *col = reinterpret_cast<uint16_t *>(stage) + (isUp ? 16u : 0u) * (kStagePitchGateUp / 2) +
                                    interleaved_position(m & 63u);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float own = __uint_as_float(isUp ? v[16 + j] : v[j]);
                        const float other = theirs[j];
                        float g = isUp ? other : own, uu = isUp ? own : other;
                        if (args.roundGateUp) {
                            g = bf2f(f2bf(g));
                            uu = bf2f(f2bf(uu));
                        }
                        col[(uint32_t)j * (kStagePitchGateUp / 2)] = f2bf(gelu_tanh_fast(g) * uu);
                    }
                    mbar_arrive(barStage(which));
                    if (!mbar_wait(barStage(which), parity, &abortFlag)) {
                        ok = false;
                        break;
                    }
                    // a token row of the tile is 128 bytes: eight threads, 16 tokens per pass
                    const uint32_t piece = t & 7u;
                    const uint32_t col0 = nt * 64u + piece * 8u;
#pragma unroll
                    for (uint32_t pass = 0; pass < 2; ++pass) {
                        const uint32_t tok = pass * 16u + (t >> 3);
                        if (c0 + tok < tile.rows && col0 < args.N) {
                            const uint4 val = *reinterpret_cast<const uint4 *>(stage + tok * kStagePitchGateUp + piece * 16u);
                            *reinterpret_cast<uint4 *>(args.out + (size_t)(tile.rowStart + c0 + tok) * args.N + col0) = val;
                        }
                    }
                } else {
                    // tile [32 tokens][128 outputs], 272-byte pitch
                    uint16_t *col = reinterpret_cast<uint16_t *>(stage) + m;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        col[(uint32_t)j * (kStagePitchDown / 2)] = f2bf(__uint_as_float(v[j]));
                    mbar_arrive(barStage(which));
                    if (!mbar_wait(barStage(which), parity, &abortFlag)) {
                        ok = false;
                        break;
                    }
                    // a token row of the tile is 256 bytes: sixteen threads, 8 tokens per pass
                    const uint32_t piece = t & 15u;
                    const uint32_t col0 = nt * 128u + piece * 8u;
#pragma unroll
                    for (uint32_t pass = 0; pass < 4; ++pass) {
                        const uint32_t tok = pass * 8u + (t >> 4);
                        if (c0 + tok < tile.rows && col0 < args.N) {
                            const uint4 val = *reinterpret_cast<const uint4 *>(stage + tok * kStagePitchDown + piece * 16u);
                            *reinterpret_cast<uint4 *>(args.out + (size_t)rowOf[c0 + tok] * args.N + col0) = val;
                        }
                    }
                }
            }
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(barAccEmpty(acc), 0u));
            if (++acc == 2) {
                acc = 0;
                accPhase ^= 1u;
            }
        }
    }

    // teardown: every thread arrives here, also after a wait that ran out
    __syncwarp();
    if (abortFlag) {
        // give copies still in flight time to land before shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        if (threadIdx.x == 0) atomicExch(args.errorFlag, 1u + (uint32_t)MODE);
    }
    tc_fence_before();
    __syncthreads();
    // neither CTA leaves (or frees its tensor memory) while the other may still arrive on its
    // barriers or have MMAs reading its shared memory
    cluster_sync_all();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase),
                     "r"(kTmemCols)
                     : "memory");
    }
}

// ---- host side -----------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled(const char **error) {
    // looked up once (thread-safe initialisation of a function-local static)
    static const EncodeTiledFn fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t st = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
        if (st != cudaSuccess || q != cudaDriverEntryPointSuccess) sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    if (!fn) fail(error, "cuTensorMapEncodeTiled is not available from the driver");
    return fn;
}

// bf16 activations [rows][k] (row pitch `strideElems`), box 64 x kTokHalfRows (the half of a row
// tile that one CTA of a pair holds), 128-byte swizzle.
static bool make_activation_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t k,
                                uint64_t strideElems, const char **error) {
    EncodeTiledFn fn = encode_tiled(error);
    if (!fn) return false;
    cuuint64_t dims[2] = {k, rows};
    cuuint64_t strides[1] = {strideElems * 2};
    cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)kTokHalfRows};
    cuuint32_t elem[2] = {1, 1};
    CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(error, "cuTensorMapEncodeTiled(activations) failed: " + std::to_string((int)rc));
    return true;
}

// router matrix bf16 [experts][d]: boxes of 256 inputs x 8 experts, no swizzle; parts of a box past
// the matrix read as zero.
static bool make_router_map(CUtensorMap *map, const void *base, uint64_t experts, uint64_t d, const char **error) {
    EncodeTiledFn fn = encode_tiled(error);
    if (!fn) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (d * 2) % 16) return fail(error, "router rows must be 16-byte aligned");
    cuuint64_t dims[2] = {d, experts};
    cuuint64_t strides[1] = {d * 2};
    cuuint32_t box[2] = {(cuuint32_t)kRouterBlockK, (cuuint32_t)kRouterExperts};
    cuuint32_t elem[2] = {1, 1};
    CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(error, "cuTensorMapEncodeTiled(router) failed: " + std::to_string((int)rc));
    return true;
}

// packed codes of one matrix across all experts: bytes [experts][rows][cols/2], box 32 x 64 x 1.
// Packed codes of one matrix across all experts seen as 64-bit words [experts][rows][rowBytes/8],
// box `boxBytes` x `boxRows` x 1 without swizzle: a tile of whole row pieces in one copy, rows
// `boxBytes` apart in shared memory.  Out-of-range parts of a box read as zero.
bool make_row_box_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t rowBytes, uint64_t experts,
                      uint64_t expertStride, uint32_t boxBytes, uint32_t boxRows, const char **error) {
    EncodeTiledFn fn = encode_tiled(error);
    if (!fn) return false;
    if (rowBytes % 16 || boxBytes % 16 || boxBytes / 8 > 256 || boxRows > 256 || expertStride % 16)
        return fail(error, "row box does not fit a tensor map");
    cuuint64_t dims[3] = {rowBytes / 8, rows, experts};
    cuuint64_t strides[2] = {rowBytes, expertStride ? expertStride : rows * rowBytes};
    cuuint32_t box[3] = {boxBytes / 8, boxRows, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(error, "cuTensorMapEncodeTiled(row boxes) failed: " + std::to_string((int)rc));
    return true;
}

static bool make_weight_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols,
                            uint64_t experts, uint64_t expertStride, const char **error) {
    EncodeTiledFn fn = encode_tiled(error);
    if (!fn) return false;
    cuuint64_t dims[3] = {cols / 2, rows, experts};
    cuuint64_t strides[2] = {cols / 2, expertStride};
    cuuint32_t box[3] = {(cuuint32_t)(kTileK / 2), 64, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(error, "cuTensorMapEncodeTiled(weights) failed: " + std::to_string((int)rc));
    return true;
}

bool prefill_prepare_layer(FFContext *ctx, LayerStore &L, const char **error) {
    if (L.mapsReady) return true;
    const FFConfig &c = ctx->cfg;
    if (L.experts) {
        const uint32_t *o = &L.off.gateWOff;
        for (int m = 0; m < 3; ++m) {
            const uint64_t rows = m == 2 ? c.d : c.f, cols = m == 2 ? c.f : c.d;
            if (!make_weight_map(&L.routedMap[m], L.experts + o[3 * m], rows, cols, L.expertCount,
                                 L.stride, error))
                return false;
        }
    }
    if (L.shared) {
        const uint32_t *o = &L.sharedOff.gateWOff;
        uint64_t payload = 0;
        packed_offsets(c.d, c.sharedF, &payload);
        for (int m = 0; m < 3; ++m) {
            const uint64_t rows = m == 2 ? c.d : c.sharedF, cols = m == 2 ? c.sharedF : c.d;
            if (!make_weight_map(&L.sharedMap[m], L.shared + o[3 * m], rows, cols, 1,
                                 (payload + 15) & ~15ull, error))
                return false;
        }
    }
    L.mapsReady = true;
    return true;
}

static size_t gemm_smem_bytes(int mode, uint32_t K) {
    const size_t scaleSlots = (size_t)((K / kTileK + kGroups - 1) / kGroups) * kDequantWarps * 32 * sizeof(uint32_t);
    return 1024 + (size_t)kTokStages * kTokTileBytes + (size_t)kPackStages * kPackTileBytes +
           (mode == kModeGateUp ? kEpilogueBytesGateUp : kEpilogueBytesDown) + scaleSlots;
}

template <int MODE>
static bool launch_gemm(FFContext *ctx, const CUtensorMap &mapA, const CUtensorMap &mapW0,
                        const CUtensorMap &mapW1, const GemmArgs &args, uint32_t maxUnits,
                        cudaStream_t stream, const char **error) {
    auto kernel = k_grouped_int4_gemm<MODE>;
    const size_t smem = gemm_smem_bytes(MODE, args.K);
    if (smem > 226 * 1024) return fail(error, "contraction length too large for the GEMM's shared memory");
    static KernelSmemMemo memo;
    if (!memo.prepare(kernel, ctx->device, smem, kGemmThreads, nullptr, error)) return false;
    // clusters of two CTAs; a cluster takes (row tile, pair of weight-row tiles) units
    const uint32_t pairUnits = (maxUnits + 1) / 2 + 1;
    const uint32_t grid = 2u * std::max(1u, std::min<uint32_t>((uint32_t)ctx->smCount / 2u, pairUnits));
    {
        LaunchScope scope(ctx, stream, MODE == kModeGateUp ? "int4_gemm_gate_up_act" : "int4_gemm_down");
        kernel<<<grid, kGemmThreads, smem, stream>>>(mapA, mapW0, mapW1, args);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

static bool check_gemm_shapes(const FFConfig &c, uint32_t f, const char **error) {
    if (c.d % 64 || f % 64) return fail(error, "GEMM path needs widths that are multiples of 64");
    return true;
}

bool launch_prefill_routed(FFContext *ctx, LayerStore &L, const uint16_t *x, uint32_t xStride,
                           uint32_t tokens, const uint32_t *ids, uint16_t *partials,
                           cudaStream_t stream, const char **error) {
    const FFConfig &c = ctx->cfg;
    if (tokens == 0) return true;
    if (!ctx->xSorted) return fail(error, "context was created with maxTokens <= 16: no prefill scratch");
    if (!L.experts) return fail(error, "layer has no resident experts");
    if (!check_gemm_shapes(c, c.f, error) || !prefill_prepare_layer(ctx, L, error)) return false;
    const int T = (int)tokens, K = (int)c.topK, E = (int)L.expertCount;
    const uint32_t blocks = (tokens + kSortTokens - 1) / kSortTokens;
    const size_t sortSmem = (size_t)kSortTokens * K * sizeof(uint32_t);
    RowTile *tiles = reinterpret_cast<RowTile *>(ctx->units);
    const uint32_t maxTiles = ctx->maxUnits / 2;  // first half of the tile buffer
    {
        LaunchScope scope(ctx, stream, "route_count");
        k_route_count<<<blocks, 256, sortSmem, stream>>>(ids, T, K, E, ctx->blockCounts);
    }
    {
        LaunchScope scope(ctx, stream, "route_scan");
        k_route_scan<<<1, 256, 0, stream>>>(ctx->blockCounts, (int)blocks, E, ctx->expertOffsets, tiles,
                                            maxTiles, ctx->unitCount);
    }
    {
        LaunchScope scope(ctx, stream, "route_scatter");
        k_route_scatter<<<blocks, 256, sortSmem, stream>>>(ids, nullptr, T, K, E, ctx->blockCounts,
                                                           ctx->expertOffsets, ctx->sortedPairs);
    }
    const uint32_t pairs = tokens * c.topK;
    {
        LaunchScope scope(ctx, stream, "gather_rows");
        k_gather_rows<<<ctx->smCount * 8, 256, 0, stream>>>(x, xStride, ctx->sortedPairs, nullptr, pairs,
                                                            (int)c.d, ctx->xSorted);
    }
    FF_CUDA_OK(cudaGetLastError(), error);

    const uint32_t tileBound = pairs / kRowTile + (uint32_t)E;
    CUtensorMap mapX, mapActs;
    if (!make_activation_map(&mapX, ctx->xSorted, (uint64_t)pairs + 256, c.d, c.d, error)) return false;
    if (!make_activation_map(&mapActs, ctx->acts, (uint64_t)pairs + 256, c.f, c.f, error)) return false;

    GemmArgs a{};
    a.blobBase = L.experts;
    a.expertStride = L.stride;
    a.scaleOff[0] = L.off.gateSOff;
    a.biasOff[0] = L.off.gateBOff;
    a.scaleOff[1] = L.off.upSOff;
    a.biasOff[1] = L.off.upBOff;
    a.K = c.d;
    a.N = c.f;
    a.nTiles = (c.f + 63) / 64;
    a.tiles = tiles;
    a.counts = ctx->unitCount;
    a.out = ctx->acts;
    a.pairs = nullptr;
    a.topK = c.topK;
    a.roundGateUp = 0;
    a.errorFlag = ctx->errorFlag;
    if (!launch_gemm<kModeGateUp>(ctx, mapX, L.routedMap[0], L.routedMap[1], a, tileBound * a.nTiles,
                                  stream, error))
        return false;

    GemmArgs b = a;
    b.scaleOff[0] = b.scaleOff[1] = L.off.downSOff;
    b.biasOff[0] = b.biasOff[1] = L.off.downBOff;
    b.K = c.f;
    b.N = c.d;
    b.nTiles = (c.d + 127) / 128;
    b.out = partials;
    b.pairs = ctx->sortedPairs;
    return launch_gemm<kModeDown>(ctx, mapActs, L.routedMap[2], L.routedMap[2], b, tileBound * b.nTiles,
                                  stream, error);
}

// The stable counting sort of routes by a group id, on its own: `groupIds` [tokens][K] on the device
// (ids >= groups are dropped), `sortedPairs` receives (token, group, rank, 0) in (group, token,
// rank) order, `offsets` [groups + 1] the first row of every group.  Uses the context's permute
// scratch.
bool launch_route_sort(FFContext *ctx, const uint32_t *groupIds, uint32_t tokens, uint32_t groups,
                       FFTokenExpertPair *sortedPairs, uint32_t *offsets, cudaStream_t stream, const char **error) {
    const FFConfig &c = ctx->cfg;
    if (tokens == 0) return true;
    if (!ctx->xSorted) return fail(error, "context was created with maxTokens <= 16: no prefill scratch");
    if (groups == 0 || groups > c.experts) return fail(error, "group count must be 1..experts of the context");
    if (tokens > c.maxTokens) return fail(error, "rows exceed the context's maxTokens");
    const int T = (int)tokens, K = (int)c.topK, E = (int)groups;
    const uint32_t blocks = (tokens + kSortTokens - 1) / kSortTokens;
    const size_t sortSmem = (size_t)kSortTokens * K * sizeof(uint32_t);
    RowTile *tiles = reinterpret_cast<RowTile *>(ctx->units);
    {
        LaunchScope scope(ctx, stream, "route_count");
        k_route_count<<<blocks, 256, sortSmem, stream>>>(groupIds, T, K, E, ctx->blockCounts);
    }
    {
        LaunchScope scope(ctx, stream, "route_scan");
        k_route_scan<<<1, 256, 0, stream>>>(ctx->blockCounts, (int)blocks, E, offsets, tiles, ctx->maxUnits / 2,
                                            ctx->unitCount);
    }
    {
        LaunchScope scope(ctx, stream, "route_scatter");
        k_route_scatter<<<blocks, 256, sortSmem, stream>>>(groupIds, nullptr, T, K, E, ctx->blockCounts, offsets,
                                                           sortedPairs);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

bool launch_prefill_shared(FFContext *ctx, LayerStore &L, const uint16_t *x, uint32_t xStride,
                           uint32_t tokens, uint16_t *y, cudaStream_t stream, const char **error) {
    const FFConfig &c = ctx->cfg;
    if (tokens == 0) return true;
    if (!ctx->xSorted) return fail(error, "context was created with maxTokens <= 16: no prefill scratch");
    if (!L.shared) return fail(error, "layer has no resident shared FFN");
    if (!check_gemm_shapes(c, c.sharedF, error) || !prefill_prepare_layer(ctx, L, error)) return false;
    // dense problem: its row tiles live behind the routed ones in the units buffer
    RowTile *tiles = reinterpret_cast<RowTile *>(ctx->units) + ctx->maxUnits / 2;
    uint32_t *counts = ctx->unitCount + 4;
    {
        LaunchScope scope(ctx, stream, "dense_tiles");
        k_dense_tiles<<<1, 256, 0, stream>>>((int)tokens, tiles, counts);
    }
    {
        LaunchScope scope(ctx, stream, "gather_rows");
        k_gather_rows<<<ctx->smCount * 8, 256, 0, stream>>>(x, xStride, nullptr, nullptr, tokens,
                                                            (int)c.d, ctx->xSorted);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    const uint32_t rowTiles = (tokens + kRowTile - 1) / kRowTile;
    CUtensorMap mapX, mapActs;
    if (!make_activation_map(&mapX, ctx->xSorted, (uint64_t)tokens + 256, c.d, c.d, error)) return false;
    if (!make_activation_map(&mapActs, ctx->sharedActs, (uint64_t)tokens + 256, c.sharedF, c.sharedF, error))
        return false;
    uint64_t payload = 0;
    packed_offsets(c.d, c.sharedF, &payload);
    GemmArgs a{};
    a.blobBase = L.shared;
    a.expertStride = (payload + 15) & ~15ull;
    a.scaleOff[0] = L.sharedOff.gateSOff;
    a.biasOff[0] = L.sharedOff.gateBOff;
    a.scaleOff[1] = L.sharedOff.upSOff;
    a.biasOff[1] = L.sharedOff.upBOff;
    a.K = c.d;
    a.N = c.sharedF;
    a.nTiles = (c.sharedF + 63) / 64;
    a.tiles = tiles;
    a.counts = counts;
    a.out = ctx->sharedActs;
    a.topK = c.topK;
    a.roundGateUp = 1;
    a.errorFlag = ctx->errorFlag;
    if (!launch_gemm<kModeGateUp>(ctx, mapX, L.sharedMap[0], L.sharedMap[1], a, rowTiles * a.nTiles, stream,
                                  error))
        return false;
    GemmArgs b = a;
    b.scaleOff[0] = b.scaleOff[1] = L.sharedOff.downSOff;
    b.biasOff[0] = b.biasOff[1] = L.sharedOff.downBOff;
    b.K = c.sharedF;
    b.N = c.d;
    b.nTiles = (c.d + 127) / 128;
    b.out = y;
    b.pairs = nullptr;
    return launch_gemm<kModeDown>(ctx, mapActs, L.sharedMap[2], L.sharedMap[2], b, rowTiles * b.nTiles,
                                  stream, error);
}

}  // namespace ff

extern "C" bool ff_last_prefill_routes(FFContext *ctx, FFTokenExpertPair *sortedPairs,
                                       uint32_t *offsets, const char **error) {
    using namespace ff;
    if (error) *error = nullptr;
    if (!ctx || !sortedPairs || !offsets) return fail(error, "null argument");
    if (!ctx->sortedPairs) return fail(error, "context has no prefill scratch");
    FF_CUDA_OK(cudaSetDevice(ctx->device), error);
    FF_CUDA_OK(cudaDeviceSynchronize(), error);
    uint32_t counts[4] = {0, 0, 0, 0};
    FF_CUDA_OK(cudaMemcpy(counts, ctx->unitCount, sizeof(counts), cudaMemcpyDeviceToHost), error);
    FF_CUDA_OK(cudaMemcpy(sortedPairs, ctx->sortedPairs, (size_t)counts[1] * sizeof(FFTokenExpertPair),
                          cudaMemcpyDeviceToHost),
               error);
    FF_CUDA_OK(cudaMemcpy(offsets, ctx->expertOffsets, (size_t)(ctx->cfg.experts + 1) * sizeof(uint32_t),
                          cudaMemcpyDeviceToHost),
               error);
    return true;
}
