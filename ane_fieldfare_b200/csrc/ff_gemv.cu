// Bandwidth kernels of the INT4 MoE block for 1..16 token rows: router, top-K + route plan,
// grouped INT4 GEMV (gate/up/GeGLU and down), decode combine, token-major reduce, RMSNorm and
// the dequantization probe.
//
// GEMV scheme (every matrix, every row count): a weight row of `cols` 4-bit codes is cut into
// 16-byte chunks of 32 codes.  Eight lanes share a row; lane j takes chunks j, j+8, j+16, ...
// with one 128-bit load each, unpacks the codes in registers, and for every input row
// accumulates  acc = fma(scale, sum(q*x), acc); acc = fma(bias, sum(x), acc)  per chunk; the
// eight lane sums are added by an xor butterfly (4, 2, 1).  A warp therefore covers four weight
// rows, and the per-(weight row, input row) arithmetic does not depend on how many input rows a
// job carries.  Input rows are staged once per job in shared memory as fp32, in an order that
// makes the eight lanes' 128-bit reads contiguous.
//
// Reference kernels this file stands in for (paths inside the reference project):
//   Sources/ANEFieldfareHotpath/Metal/MoE/moe.metal:65-103,186-319,382-517,548-638
//   Sources/ANEFieldfareHotpath/Metal/Prefill/prefill.metal:544-565,1246-1529
//   Sources/ANEFieldfareHotpath/Metal/Quant/dequant_int4.metal:78-347
#include <algorithm>

#include "ff_gemv_device.cuh"
#include "ff_internal.cuh"

namespace ff {

template <int NT, bool DUAL, bool STAGE_ALL>
__device__ __forceinline__ void run_item(const GemvJob &job, int row0, const float *xs,
                                         const float *xsum) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = row0 + warp * 4 + (lane >> 3);
    const bool live = row < (int)job.rows;
    // staged row each input reads: with all rows of the block staged once, the job's own row
    // numbers; otherwise the job's rows were staged compactly in order
    int sel[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int tt = t < (int)job.n ? t : 0;
        sel[t] = STAGE_ALL ? (int)job.inRow[tt] : tt;
    }
    float a0[NT], a1[NT];
    row_dot<NT, DUAL>(job.w0, job.s0, job.b0, job.w1, job.s1, job.b1, row, (int)job.cols, live, xs,
                      xsum, sel, a0, a1);
    if (live && (lane & 7) == 0) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            if (t < (int)job.n) {
                float v = a0[t];
                if (DUAL) {
                    float g = a0[t], u = a1[t];
                    if (job.flags & kJobRoundGateUp) {
                        g = bf16_round(g);
                        u = bf16_round(u);
                    }
                    v = gelu_tanh(g) * u;
                }
                job.out[(size_t)job.outRow[t] * job.outStride + row] = f2bf(v);
            }
        }
    }
}

// Persistent grouped GEMV over (job, row block) items.  With `jobs` null the single `inlineJob`
// is used.  STAGE_ALL: every job reads rows of one input block (`allRows` x `allCols`), which is
// staged once per CTA and items are dealt round robin; otherwise a job's input rows are staged
// when a CTA meets the job, and items are dealt in chunks of two so that a staging is shared.
template <int MAXNT, bool DUAL, bool STAGE_ALL>
__global__ void __launch_bounds__(kGemvThreads)
k_int4_gemv(const GemvJob *jobs, const uint32_t *items, const uint32_t *itemCountPtr,
            GemvJob inlineJob, uint32_t inlineItems, uint32_t maxCols, const uint16_t *allIn,
            uint32_t allStride, uint32_t allRows) {
    extern __shared__ float smem[];
    __shared__ GemvJob sjob;
    __shared__ uint32_t sAllRows[kMaxGemvRows];
    float *xs = smem;
    const int stagedRows = STAGE_ALL ? (int)allRows : MAXNT;
    float *xsum = smem + stagedRows * staged_stride((int)maxCols);
    const uint32_t nItems = jobs ? *itemCountPtr : inlineItems;
    if (STAGE_ALL) {
        if (threadIdx.x < kMaxGemvRows) sAllRows[threadIdx.x] = threadIdx.x;
        __syncthreads();
        stage_rows(allIn, allStride, sAllRows, (int)allRows, (int)maxCols, xs, xsum);
    }
    constexpr uint32_t kItemChunk = STAGE_ALL ? 1 : 2;
    const uint32_t nChunks = (nItems + kItemChunk - 1) / kItemChunk;
    int current = -1;
    for (uint32_t chunk = blockIdx.x; chunk < nChunks; chunk += gridDim.x)
    for (uint32_t it = chunk * kItemChunk; it < min(nItems, (chunk + 1) * kItemChunk); ++it) {
        uint32_t jobIdx = 0, block = it;
        if (jobs) {
            const uint32_t packed = items[it];
            jobIdx = packed >> 16;
            block = packed & 0xFFFFu;
        }
        if ((int)jobIdx != current) {
            __syncthreads();
            const uint32_t *src =
                reinterpret_cast<const uint32_t *>(jobs ? jobs + jobIdx : &inlineJob);
            uint32_t *dst = reinterpret_cast<uint32_t *>(&sjob);
            for (int i = threadIdx.x; i < (int)(sizeof(GemvJob) / 4); i += blockDim.x) dst[i] = src[i];
            __syncthreads();
            if (!STAGE_ALL)
                stage_rows(sjob.in, sjob.inStride, sjob.inRow, min((int)sjob.n, MAXNT), (int)sjob.cols,
                           xs, xsum);
            current = (int)jobIdx;
        }
        const int row0 = (int)block * kRowsPerItem;
        const int n = (int)sjob.n;
        if (n <= 1) {
            run_item<1, DUAL, STAGE_ALL>(sjob, row0, xs, xsum);
        } else if (MAXNT >= 2 && n <= 2) {
            run_item<(MAXNT >= 2 ? 2 : 1), DUAL, STAGE_ALL>(sjob, row0, xs, xsum);
        } else if (MAXNT >= 4 && n <= 4) {
            run_item<(MAXNT >= 4 ? 4 : 1), DUAL, STAGE_ALL>(sjob, row0, xs, xsum);
        } else if (MAXNT >= 8 && n <= 8) {
            run_item<(MAXNT >= 8 ? 8 : 1), DUAL, STAGE_ALL>(sjob, row0, xs, xsum);
        } else if (MAXNT >= 16) {
            run_item<(MAXNT >= 16 ? 16 : 1), DUAL, STAGE_ALL>(sjob, row0, xs, xsum);
        }
    }
}

// ---- router --------------------------------------------------------------------------------

// One warp per (expert, token).  The reduction order is part of the contract (top-K indices are
// compared for equality with the CPU oracle): lane l chains fmaf over elements
// [256 i + 8 l, +8) for i = 0, 1, ... in increasing index, the lane sums are added by an xor
// butterfly (16, 8, 4, 2, 1), then the per-expert logit bias is added.
__global__ void __launch_bounds__(256)
k_router_logits(const uint16_t *W, const uint16_t *scale, const float *bias, const uint16_t *x,
                uint32_t xStride, int E, int D, float *logits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    const int t = blockIdx.y;
    if (e >= E) return;
    const uint16_t *wr = W + (size_t)e * D;
    const uint16_t *xr = x + (size_t)t * xStride;
    float acc = 0.0f;
    for (int base = 8 * lane; base < D; base += 256) {
        const uint4 wv = *reinterpret_cast<const uint4 *>(wr + base);
        const uint4 xv = *reinterpret_cast<const uint4 *>(xr + base);
        uint4 sv = make_uint4(0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u);
        if (scale) sv = *reinterpret_cast<const uint4 *>(scale + base);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        const uint32_t xx[4] = {xv.x, xv.y, xv.z, xv.w};
        const uint32_t ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float x0 = __uint_as_float(xx[k] << 16), x1 = __uint_as_float(xx[k] & 0xFFFF0000u);
            if (scale) {
                x0 = x0 * __uint_as_float(ss[k] << 16);
                x1 = x1 * __uint_as_float(ss[k] & 0xFFFF0000u);
            }
            acc = fmaf(__uint_as_float(ww[k] << 16), x0, acc);
            acc = fmaf(__uint_as_float(ww[k] & 0xFFFF0000u), x1, acc);
        }
    }
#pragma unroll
    for (int offset = 16; offset >= 1; offset >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, offset);
    if (lane == 0) logits[(size_t)t * E + e] = bias ? acc + bias[e] : acc;
}

struct PlanArgs {
    const float *logits;      // [T][E] or null (ids given)
    const uint16_t *gain;
    const uint32_t *idsIn;    // used when logits is null
    uint32_t *idsOut;         // written when logits is given
    uint16_t *weightsOut;
    int T, E, K, D, F, Fs;
    const uint8_t *experts;
    uint64_t stride;
    FFExpertOffsets off;
    const uint8_t *shared;    // null: no shared job
    FFExpertOffsets sharedOff;
    const uint16_t *x;
    uint32_t xStride;
    uint16_t *acts;
    uint16_t *sharedActs;
    uint16_t *partials;       // null in decode mode: no routed down jobs
    uint16_t *sharedOut;
    GemvJob *jobs0, *jobs1;
    RoutePlan *plan;
    int buildPlan;            // 0: top-K only
    uint32_t *errorFlag;      // raised when a route names an expert that is not resident
};

// One CTA: top-K per token (when logits are given), then the route plan — the role of the
// reference's verify_bound_plan (Metal/Prefill/prefill.metal:1458-1493): per active expert the
// routes that chose it, in (token, rank) order, as one gate/up job and one down job, experts
// ascending; the shared FFN is job 0 of each phase.
__global__ void __launch_bounds__(512) k_topk_plan(PlanArgs a) {
    __shared__ uint32_t sIds[kMaxGemvRows * 8];
    __shared__ uint32_t sPos[kMaxExperts];
    __shared__ uint32_t sCount[kMaxExperts];
    __shared__ __align__(16) uint8_t sList[kMaxExperts * kMaxGemvRows];  // route numbers (< 128)
    const int warp = threadIdx.x >> 5;
    const int routes = a.T * a.K;
    if (a.logits) {
        if (warp < a.T) {
            warp_topk(a.logits + (size_t)warp * a.E, a.E, a.K, a.gain, a.idsOut + warp * a.K,
                      a.weightsOut + warp * a.K, sIds + warp * a.K);
        }
    } else {
        for (int i = threadIdx.x; i < routes; i += blockDim.x) sIds[i] = a.idsIn[i];
    }
    if (!a.buildPlan) return;
    __syncthreads();
    // Lists of routes per expert, built from the routes' side: route r's place in its expert's list
    // is the number of earlier routes with the same expert, so every list is in (token, rank) order.
    // A token's routes are distinct experts, so an expert is chosen by at most T routes; repeats
    // beyond that are dropped rather than overrunning the row class.
    for (int i = threadIdx.x; i < kMaxExperts; i += blockDim.x) sCount[i] = 0u;
    __syncthreads();
    if ((int)threadIdx.x < routes) {
        const int r = threadIdx.x;
        const uint32_t mine = sIds[r];
        int place = 0;
        for (int q = 0; q < r; ++q) place += sIds[q] == mine ? 1 : 0;
        if (mine < (uint32_t)a.E && place < a.T) {
            sList[mine * kMaxGemvRows + place] = (uint8_t)r;
            atomicAdd(&sCount[mine], 1u);
        } else {
            // the reference refuses such a route ("route expert N is out of range"); here its
            // partial row stays unwritten and the context's error flag says so
            atomicExch(a.errorFlag, 12u);
        }
    }
    __syncthreads();
    const int e = threadIdx.x;
    uint32_t list[kMaxGemvRows];
    const int n = e < a.E ? (int)sCount[e] : 0;
    {
        const uint4 packed = e < a.E ? *reinterpret_cast<const uint4 *>(&sList[e * kMaxGemvRows]) : make_uint4(0, 0, 0, 0);
        const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
        for (int i = 0; i < kMaxGemvRows; ++i) list[i] = i < n ? (words[i >> 2] >> (8 * (i & 3))) & 0xFFu : 0u;
    }
    // position of expert e among the active experts: ballots inside a warp, warp totals through
    // shared memory
    const bool isActive = e < a.E && n > 0;
    const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, isActive);
    const int lane = threadIdx.x & 31;
    if (lane == 0) sPos[warp] = __popc(ballot);
    __syncthreads();
    uint32_t before = 0, active = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
        const uint32_t c = sPos[w];
        if (w < warp) before += c;
        active += c;
    }
    const uint32_t myPos = before + __popc(ballot & ((1u << lane) - 1u));
    const uint32_t sharedJobs = a.shared ? 1u : 0u;
    if (e < a.E && n > 0) {
        const uint8_t *blob = a.experts + (size_t)e * a.stride;
        GemvJob j0{};
        j0.w0 = blob + a.off.gateWOff;
        j0.s0 = reinterpret_cast<const uint16_t *>(blob + a.off.gateSOff);
        j0.b0 = reinterpret_cast<const uint16_t *>(blob + a.off.gateBOff);
        j0.w1 = blob + a.off.upWOff;
        j0.s1 = reinterpret_cast<const uint16_t *>(blob + a.off.upSOff);
        j0.b1 = reinterpret_cast<const uint16_t *>(blob + a.off.upBOff);
        j0.in = a.x;
        j0.out = a.acts;
        j0.rows = (uint32_t)a.F;
        j0.cols = (uint32_t)a.D;
        j0.inStride = a.xStride;
        j0.outStride = (uint32_t)a.F;
        j0.n = (uint32_t)n;
        j0.flags = 0;
        for (int i = 0; i < kMaxGemvRows; ++i) {
            j0.inRow[i] = i < n ? list[i] / (uint32_t)a.K : 0u;
            j0.outRow[i] = i < n ? list[i] : 0u;
        }
        a.jobs0[sharedJobs + myPos] = j0;
        if (a.partials) {
            GemvJob j1{};
            j1.w0 = blob + a.off.downWOff;
            j1.s0 = reinterpret_cast<const uint16_t *>(blob + a.off.downSOff);
            j1.b0 = reinterpret_cast<const uint16_t *>(blob + a.off.downBOff);
            j1.in = a.acts;
            j1.out = a.partials;
            j1.rows = (uint32_t)a.D;
            j1.cols = (uint32_t)a.F;
            j1.inStride = (uint32_t)a.F;
            j1.outStride = (uint32_t)a.D;
            j1.n = (uint32_t)n;
            for (int i = 0; i < kMaxGemvRows; ++i) {
                j1.inRow[i] = i < n ? list[i] : 0u;
                j1.outRow[i] = i < n ? list[i] : 0u;
            }
            a.jobs1[sharedJobs + myPos] = j1;
        }
    }
    if (threadIdx.x == 0 && a.shared) {
        GemvJob j0{};
        j0.w0 = a.shared + a.sharedOff.gateWOff;
        j0.s0 = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.gateSOff);
        j0.b0 = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.gateBOff);
        j0.w1 = a.shared + a.sharedOff.upWOff;
        j0.s1 = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.upSOff);
        j0.b1 = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.upBOff);
        j0.in = a.x;
        j0.out = a.sharedActs;
        j0.rows = (uint32_t)a.Fs;
        j0.cols = (uint32_t)a.D;
        j0.inStride = a.xStride;
        j0.outStride = (uint32_t)a.Fs;
        j0.n = (uint32_t)a.T;
        j0.flags = kJobRoundGateUp;
        GemvJob j1{};
        j1.w0 = a.shared + a.sharedOff.downWOff;
        j1.s0 = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.downSOff);
        j1.b0 = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.downBOff);
        j1.in = a.sharedActs;
        j1.out = a.sharedOut;
        j1.rows = (uint32_t)a.D;
        j1.cols = (uint32_t)a.Fs;
        j1.inStride = (uint32_t)a.Fs;
        j1.outStride = (uint32_t)a.D;
        j1.n = (uint32_t)a.T;
        for (int i = 0; i < kMaxGemvRows; ++i) {
            j0.inRow[i] = j0.outRow[i] = j1.inRow[i] = j1.outRow[i] = i < a.T ? (uint32_t)i : 0u;
        }
        a.jobs0[0] = j0;
        a.jobs1[0] = j1;
    }
    const uint32_t routedJobs1 = a.partials ? active : 0u;
    if (threadIdx.x == 0) {
        a.plan->jobCount[0] = sharedJobs + active;
        a.plan->jobCount[1] = sharedJobs + routedJobs1;
        a.plan->itemCount[0] = 0;
        a.plan->itemCount[1] = 0;
        a.plan->activeExperts = active;
    }
}

// Metal/Prefill/prefill.metal:544-565 plus an optional residual row added after the ranks.
// rowIndex (optional): the partial row of route (t, r) is row rowIndex[t * K + r] of `partials`
// instead of row t * K + r — rows that came back from other GPUs in another order are reduced
// where they lie.
__global__ void __launch_bounds__(256)
k_reduce_token_major(const uint16_t *partials, const uint32_t *rowIndex, const uint16_t *weights,
                     const uint16_t *residual, uint16_t *y, int T, int K, int D) {
    const int t = blockIdx.y;
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (t >= T || d >= D) return;
    float acc0 = 0.0f, acc1 = 0.0f;
    for (int r = 0; r < K; ++r) {
        const float w = bf2f(weights[(size_t)t * K + r]);
        const size_t row = rowIndex ? (size_t)rowIndex[(size_t)t * K + r] : (size_t)t * K + r;
        const uint32_t two = *reinterpret_cast<const uint32_t *>(partials + row * D + d);
        acc0 = fmaf(w, __uint_as_float(two << 16), acc0);
        acc1 = fmaf(w, __uint_as_float(two & 0xFFFF0000u), acc1);
    }
    if (residual) {
        const uint32_t two = *reinterpret_cast<const uint32_t *>(residual + (size_t)t * D + d);
        acc0 += __uint_as_float(two << 16);
        acc1 += __uint_as_float(two & 0xFFFF0000u);
    }
    *reinterpret_cast<uint32_t *>(y + (size_t)t * D + d) =
        (uint32_t)f2bf(acc0) | ((uint32_t)f2bf(acc1) << 16);
}

// The same reduce, eight outputs per thread with 128-bit loads (every element's chain is the one
// above: rank ascending, then the residual); for rows that are 16-byte aligned.
__global__ void __launch_bounds__(256)
k_reduce_token_major_x8(const uint16_t *partials, const uint32_t *rowIndex, const uint16_t *weights,
                        const uint16_t *residual, uint16_t *y, int T, int K, int D) {
    const int perRow = D >> 3;
    const size_t item = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (size_t)T * perRow) return;
    const int t = (int)(item / perRow), d = (int)(item - (size_t)t * perRow) * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (int r = 0; r < K; ++r) {
        const float w = bf2f(weights[(size_t)t * K + r]);
        const size_t row = rowIndex ? (size_t)rowIndex[(size_t)t * K + r] : (size_t)t * K + r;
        const uint4 v = *reinterpret_cast<const uint4 *>(partials + row * D + d);
        const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] = fmaf(w, __uint_as_float(p[i] << 16), acc[2 * i]);
            acc[2 * i + 1] = fmaf(w, __uint_as_float(p[i] & 0xFFFF0000u), acc[2 * i + 1]);
        }
    }
    if (residual) {
        const uint4 v = *reinterpret_cast<const uint4 *>(residual + (size_t)t * D + d);
        const uint32_t p[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] += __uint_as_float(p[i] << 16);
            acc[2 * i + 1] += __uint_as_float(p[i] & 0xFFFF0000u);
        }
    }
    uint4 o;
    o.x = (uint32_t)f2bf(acc[0]) | ((uint32_t)f2bf(acc[1]) << 16);
    o.y = (uint32_t)f2bf(acc[2]) | ((uint32_t)f2bf(acc[3]) << 16);
    o.z = (uint32_t)f2bf(acc[4]) | ((uint32_t)f2bf(acc[5]) << 16);
    o.w = (uint32_t)f2bf(acc[6]) | ((uint32_t)f2bf(acc[7]) << 16);
    *reinterpret_cast<uint4 *>(y + (size_t)t * D + d) = o;
}

// y = x * w * rsqrt(mean(x^2) + eps) per row; one CTA per row, fp32 throughout.
__global__ void __launch_bounds__(256)
k_rmsnorm(const uint16_t *x, const uint16_t *w, float eps, int D, uint16_t *y) {
    __shared__ float warpSums[8];
    __shared__ float inv;
    const uint16_t *xr = x + (size_t)blockIdx.x * D;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = bf2f(xr[i]);
        sum = fmaf(v, v, sum);
    }
#pragma unroll
    for (int offset = 16; offset >= 1; offset >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, offset);
    if ((threadIdx.x & 31) == 0) warpSums[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int i = 0; i < 8; ++i) total += warpSums[i];
        inv = 1.0f / sqrtf(total / (float)D + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float wv = w ? bf2f(w[i]) : 1.0f;
        y[(size_t)blockIdx.x * D + i] = f2bf(bf2f(xr[i]) * wv * inv);
    }
}

// ---- the fused steps either side of the block ----------------------------------------------------

// Sum over the CTA (256 threads) of one float per thread; every thread gets the total.
__device__ __forceinline__ float cta_sum_256(float v, float *warpSums) {
#pragma unroll
    for (int offset = 16; offset >= 1; offset >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, offset);
    __syncthreads();  // warpSums may still be read from the previous use
    if ((threadIdx.x & 31) == 0) warpSums[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += warpSums[i];
    return total;
}

// prefill_post_attn_setup_block (Metal/Prefill/prefill.metal:244-318), one CTA per row:
//   a = r16(attn * rms_inv(attn) * w_post_attn);  hidden = r16(hidden + a);
//   n = hidden * rms_inv(hidden);  dense_x = r16(n * w_pre_ffn);  routed_x = r16(n * w_pre_ffn2);
//   router_x = r16(n).  The new hidden row is kept in shared memory between the two passes.
__global__ void __launch_bounds__(256)
k_post_attn_setup(uint16_t *hidden, const uint16_t *attn, const uint16_t *wPostAttn, const uint16_t *wPreFfn,
                  const uint16_t *wPreFfn2, float eps, int D, uint16_t *denseX, uint16_t *routedX,
                  uint16_t *routerX) {
    extern __shared__ uint16_t glueRow[];
    __shared__ float warpSums[8];
    const size_t row = (size_t)blockIdx.x * D;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = bf2f(attn[row + i]);
        sq = fmaf(v, v, sq);
    }
    const float attnInv = 1.0f / sqrtf(cta_sum_256(sq, warpSums) / (float)D + eps);
    sq = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const uint16_t an = f2bf(bf2f(attn[row + i]) * attnInv * bf2f(wPostAttn[i]));
        const uint16_t h = f2bf(bf2f(hidden[row + i]) + bf2f(an));
        glueRow[i] = h;
        hidden[row + i] = h;
        const float hf = bf2f(h);
        sq = fmaf(hf, hf, sq);
    }
    const float hiddenInv = 1.0f / sqrtf(cta_sum_256(sq, warpSums) / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float n = bf2f(glueRow[i]) * hiddenInv;
        denseX[row + i] = f2bf(n * bf2f(wPreFfn[i]));
        routedX[row + i] = f2bf(n * bf2f(wPreFfn2[i]));
        routerX[row + i] = f2bf(n);
    }
}

// prefill_layer_tail_block (Metal/Prefill/prefill.metal:321-399; one row: Metal/Fusions/fused.metal:470-474):
//   t = r16(h2 * rms_inv(h2) * w_postffn2);  h12 = r16(h1 + t);
//   u = r16(h12 * rms_inv(h12) * w_postffn);  hidden = r16(r16(hidden + u) * r16(layer_scalar)).
__global__ void __launch_bounds__(256)
k_layer_tail(const uint16_t *h2, const uint16_t *h1, uint16_t *hidden, const uint16_t *wPostFfn2,
             const uint16_t *wPostFfn, float eps, float layerScalar, int D) {
    extern __shared__ uint16_t glueRow[];
    __shared__ float warpSums[8];
    const size_t row = (size_t)blockIdx.x * D;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = bf2f(h2[row + i]);
        sq = fmaf(v, v, sq);
    }
    const float inv2 = 1.0f / sqrtf(cta_sum_256(sq, warpSums) / (float)D + eps);
    sq = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const uint16_t tmp = f2bf(bf2f(h2[row + i]) * inv2 * bf2f(wPostFfn2[i]));
        const uint16_t h12 = f2bf(bf2f(h1[row + i]) + bf2f(tmp));
        glueRow[i] = h12;
        const float v = bf2f(h12);
        sq = fmaf(v, v, sq);
    }
    const float inv12 = 1.0f / sqrtf(cta_sum_256(sq, warpSums) / (float)D + eps);
    const float scale = bf2f(f2bf(layerScalar));
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const uint16_t u = f2bf(bf2f(glueRow[i]) * inv12 * bf2f(wPostFfn[i]));
        const uint16_t sum = f2bf(bf2f(hidden[row + i]) + bf2f(u));
        hidden[row + i] = f2bf(bf2f(sum) * scale);
    }
}

bool launch_post_attn_setup(FFContext *ctx, uint16_t *hidden, const uint16_t *attn, const uint16_t *wPostAttn,
                            const uint16_t *wPreFfn, const uint16_t *wPreFfn2, float eps, uint32_t tokens,
                            uint16_t *denseX, uint16_t *routedX, uint16_t *routerX, cudaStream_t stream,
                            const char **error) {
    if (tokens == 0) return true;
    const int D = (int)ctx->cfg.d;
    if ((size_t)D * 2 > 96 * 1024) return fail(error, "model width too large for the row buffer");
    {
        LaunchScope scope(ctx, stream, "post_attn_setup");
        k_post_attn_setup<<<tokens, 256, (size_t)D * 2, stream>>>(hidden, attn, wPostAttn, wPreFfn, wPreFfn2, eps, D,
                                                                  denseX, routedX, routerX);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

bool launch_layer_tail(FFContext *ctx, const uint16_t *h2, const uint16_t *h1, uint16_t *hidden,
                       const uint16_t *wPostFfn2, const uint16_t *wPostFfn, float eps, float layerScalar,
                       uint32_t tokens, cudaStream_t stream, const char **error) {
    if (tokens == 0) return true;
    const int D = (int)ctx->cfg.d;
    if ((size_t)D * 2 > 96 * 1024) return fail(error, "model width too large for the row buffer");
    {
        LaunchScope scope(ctx, stream, "layer_tail");
        k_layer_tail<<<tokens, 256, (size_t)D * 2, stream>>>(h2, h1, hidden, wPostFfn2, wPostFfn, eps, layerScalar, D);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

// w = q*scale + bias for a whole matrix, fp32 and/or bf16 (one rounding of the exact value:
// a bf16 fused multiply-add).  One thread per 8 codes.
__global__ void __launch_bounds__(256)
k_dequant_probe(const uint8_t *w, const uint16_t *s, const uint16_t *b, int rows, int cols,
                float *out32, uint16_t *out16) {
    const size_t word = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t wordsPerRow = (size_t)cols / 8;
    if (word >= (size_t)rows * wordsPerRow) return;
    const size_t row = word / wordsPerRow;
    const int col = (int)(word - row * wordsPerRow) * 8;
    const uint32_t packed = reinterpret_cast<const uint32_t *>(w)[word];
    const size_t g = row * (size_t)(cols / kGroup) + (size_t)(col / kGroup);
    const float scale = bf2f(s[g]), bias = bf2f(b[g]);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float q = (float)((packed >> (4 * k)) & 0xFu);
        if (out32) out32[row * cols + col + k] = fmaf(q, scale, bias);
        if (out16) {
            // exact in double, then one rounding to bf16 via round-to-odd fp32
            const double exact = (double)q * (double)scale + (double)bias;
            float f = __double2float_rz(exact);
            if ((double)f != exact) f = __uint_as_float(__float_as_uint(f) | 1u);
            out16[row * cols + col + k] = f2bf(f);
        }
    }
}

// ---- host launchers ------------------------------------------------------------------------

static size_t gemv_smem_bytes(int rows, uint32_t maxCols) {
    return (size_t)rows * (staged_stride((int)maxCols) + (maxCols >> 5)) * sizeof(float);
}

constexpr size_t kGemvSmemLimit = 200 * 1024;
static uint32_t gemv_rows_class(uint32_t n) { return n <= 1 ? 1 : n <= 2 ? 2 : n <= 4 ? 4 : n <= 8 ? 8 : 16; }
// Input rows one launch can stage for a job of `n` rows and `cols` columns: the job's row class,
// or the largest smaller class that fits in shared memory; 0 when not even one row fits.
static uint32_t gemv_pass_rows(uint32_t n, uint32_t cols) {
    for (uint32_t c = gemv_rows_class(n); c >= 1; c >>= 1)
        if (gemv_smem_bytes((int)c, cols) <= kGemvSmemLimit) return c;
    return 0;
}

// The input block all jobs of a launch read (staged once per CTA), or null.
struct StageAll {
    const uint16_t *in = nullptr;
    uint32_t stride = 0, rows = 0;
};

template <int MAXNT, bool DUAL, bool STAGE_ALL>
static bool launch_gemv_kernel(FFContext *ctx, const GemvJob *jobs, const uint32_t *items,
                               const uint32_t *itemCountPtr, const GemvJob &inlineJob,
                               uint32_t inlineItems, uint32_t maxCols, uint32_t itemBound,
                               const StageAll &all, cudaStream_t stream, const char **error) {
    auto kernel = k_int4_gemv<MAXNT, DUAL, STAGE_ALL>;
    const size_t smem = gemv_smem_bytes(STAGE_ALL ? (int)all.rows : MAXNT, maxCols);
    if (smem > kGemvSmemLimit)
        return fail(error, "input rows do not fit in shared memory: " + std::to_string(MAXNT) +
                               " rows x " + std::to_string(maxCols) + " columns");
    // attribute + occupancy are looked up once per (kernel, device, shared-memory size): nothing but
    // the launch itself happens on later calls, which keeps the call legal under stream capture
    static KernelSmemMemo memo;
    int perSm = 0;
    if (!memo.prepare(kernel, ctx->device, smem, kGemvThreads, &perSm, error)) return false;
    if (perSm < 1) return fail(error, "GEMV kernel does not fit on an SM");
    uint32_t grid = (uint32_t)(ctx->smCount * perSm);
    if (itemBound < grid) grid = itemBound;
    if (grid == 0) return true;
    {
        LaunchScope scope(ctx, stream, DUAL ? "int4_gemv_gate_up_act" : "int4_gemv_down");
        kernel<<<grid, kGemvThreads, smem, stream>>>(jobs, items, itemCountPtr, inlineJob,
                                                     inlineItems, maxCols, all.in, all.stride, all.rows);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

template <bool DUAL>
static bool launch_gemv_class(FFContext *ctx, uint32_t rowsClass, const GemvJob *jobs,
                              const uint32_t *items, const uint32_t *itemCountPtr,
                              const GemvJob &inlineJob, uint32_t inlineItems, uint32_t maxCols,
                              uint32_t itemBound, cudaStream_t stream, const char **error,
                              const StageAll &all = StageAll()) {
#define FF_GEMV_DISPATCH(NTV)                                                                   \
    return launch_gemv_kernel<NTV, DUAL, false>(ctx, jobs, items, itemCountPtr, inlineJob, inlineItems, \
                                                maxCols, itemBound, all, stream, error)
    if (rowsClass <= 1) FF_GEMV_DISPATCH(1);
    if (rowsClass <= 2) FF_GEMV_DISPATCH(2);
    if (rowsClass <= 4) FF_GEMV_DISPATCH(4);
    if (rowsClass <= 8) FF_GEMV_DISPATCH(8);
    FF_GEMV_DISPATCH(16);
#undef FF_GEMV_DISPATCH
}

static uint32_t blocks_of(uint32_t rows) { return (rows + kRowsPerItem - 1) / kRowsPerItem; }

// One job given by value (a matrix, or a gate/up pair, against job.n <= 16 input rows).  When the
// rows of the job's class do not fit in shared memory together (wide matrices), the job runs as
// passes of fewer rows: the arithmetic per (weight row, input row) does not depend on how many
// rows a launch carries, so the bits are those of a single pass.
template <bool DUAL>
static bool launch_inline_job(FFContext *ctx, const GemvJob &job, cudaStream_t stream, const char **error) {
    const uint32_t pass = gemv_pass_rows(job.n, job.cols);
    if (pass == 0)
        return fail(error, "one input row of " + std::to_string(job.cols) + " columns does not fit in shared memory");
    for (uint32_t first = 0; first < job.n; first += pass) {
        GemvJob part = job;
        part.n = std::min(pass, job.n - first);
        for (uint32_t i = 0; i < (uint32_t)kMaxGemvRows; ++i) {
            part.inRow[i] = i < part.n ? job.inRow[first + i] : 0u;
            part.outRow[i] = i < part.n ? job.outRow[first + i] : 0u;
        }
        if (!launch_gemv_class<DUAL>(ctx, part.n, nullptr, nullptr, nullptr, part, blocks_of(part.rows), part.cols,
                                     blocks_of(part.rows), stream, error))
            return false;
    }
    return true;
}

// INT8 affine router (the shipped checkpoints' form), one warp per expert row and up to four
// tokens.  The order of the reference's kernel (Metal/MoE/moe.metal:65-103) is kept and made
// definite: lane l takes elements 64 g + 2 l and 64 g + 2 l + 1 of every group g in increasing g,
// with x' = float(x) * float(effective scale): acc = fma(s_g, fma(q1, x1', q0 * x0'), acc), then
// acc = fma(b_g, x0' + x1', acc); the lane sums are added by an xor butterfly (16, 8, 4, 2, 1) and the
// per-expert logit bias comes last.
constexpr int kInt8RouterTokens = 4;
__global__ void __launch_bounds__(256)
k_router_logits_int8(const uint8_t *W, const uint16_t *scales, const uint16_t *biases, const uint16_t *effScale,
                     const float *bias, const uint16_t *x, uint32_t xStride, int T, int E, int D, float *logits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    const int t0 = blockIdx.y * kInt8RouterTokens;
    if (e >= E) return;
    const int groups = D / 64;
    const uint8_t *wr = W + (size_t)e * D;
    const uint16_t *sr = scales + (size_t)e * groups, *br = biases + (size_t)e * groups;
    float acc[kInt8RouterTokens];
#pragma unroll
    for (int r = 0; r < kInt8RouterTokens; ++r) acc[r] = 0.0f;
    for (int g = 0; g < groups; ++g) {
        const int idx = g * 64 + 2 * lane;
        const uint32_t q = *reinterpret_cast<const uint16_t *>(wr + idx);
        const float q0 = (float)(q & 0xFFu), q1 = (float)(q >> 8);
        const float s = bf2f(sr[g]), b = bf2f(br[g]);
        float e0 = 1.0f, e1 = 1.0f;
        if (effScale) {
            const uint32_t ev = *reinterpret_cast<const uint32_t *>(effScale + idx);
            e0 = __uint_as_float(ev << 16);
            e1 = __uint_as_float(ev & 0xFFFF0000u);
        }
#pragma unroll
        for (int r = 0; r < kInt8RouterTokens; ++r) {
            const int t = min(t0 + r, T - 1);
            const uint32_t xv = *reinterpret_cast<const uint32_t *>(x + (size_t)t * xStride + idx);
            float x0 = __uint_as_float(xv << 16), x1 = __uint_as_float(xv & 0xFFFF0000u);
            if (effScale) {
                x0 = x0 * e0;
                x1 = x1 * e1;
            }
            acc[r] = fmaf(s, fmaf(q1, x1, q0 * x0), acc[r]);
            acc[r] = fmaf(b, x0 + x1, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < kInt8RouterTokens; ++r) {
        float v = acc[r];
#pragma unroll
        for (int offset = 16; offset >= 1; offset >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, offset);
        if (lane == 0 && t0 + r < T) logits[(size_t)(t0 + r) * E + e] = bias ? v + bias[e] : v;
    }
}

// INT8 affine shared FFN (Metal/Quant/dequant_int8.metal:41-138; Kernels/MoE/SharedExpertInt8.swift),
// one warp per output row and up to four input rows, in the reference kernels' order made definite:
// lane l takes elements 64 g + 2 l and + 1 of every group g in increasing g,
//   acc = fma(s_g, fma(q1, x1, q0 * x0), acc);  acc = fma(b_g, x0 + x1, acc);
// lane sums by an xor butterfly (16..1).  DUAL: gate and up rows of the same index, both rounded to
// 16 bits, then act = r16(gelu_tanh(gate) * up); otherwise one matrix, out = r16(sum).
template <bool DUAL>
__global__ void __launch_bounds__(256)
k_int8_rows(const uint8_t *W0, const uint16_t *S0, const uint16_t *B0, const uint8_t *W1, const uint16_t *S1,
            const uint16_t *B1, const uint16_t *x, uint32_t xStride, int T, int rows, int cols, uint16_t *out,
            uint32_t outStride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    const int t0 = blockIdx.y * kInt8RouterTokens;
    if (r >= rows) return;
    const int groups = cols / 64;
    const uint8_t *w0 = W0 + (size_t)r * cols, *w1 = DUAL ? W1 + (size_t)r * cols : nullptr;
    const uint16_t *s0 = S0 + (size_t)r * groups, *b0 = B0 + (size_t)r * groups;
    const uint16_t *s1 = DUAL ? S1 + (size_t)r * groups : nullptr, *b1 = DUAL ? B1 + (size_t)r * groups : nullptr;
    float acc0[kInt8RouterTokens], acc1[kInt8RouterTokens];
#pragma unroll
    for (int i = 0; i < kInt8RouterTokens; ++i) acc0[i] = acc1[i] = 0.0f;
    for (int g = 0; g < groups; ++g) {
        const int idx = g * 64 + 2 * lane;
        const uint32_t q = *reinterpret_cast<const uint16_t *>(w0 + idx);
        const float q00 = (float)(q & 0xFFu), q01 = (float)(q >> 8);
        const float sa = bf2f(s0[g]), ba = bf2f(b0[g]);
        float q10 = 0.0f, q11 = 0.0f, sb = 0.0f, bb = 0.0f;
        if (DUAL) {
            const uint32_t p = *reinterpret_cast<const uint16_t *>(w1 + idx);
            q10 = (float)(p & 0xFFu);
            q11 = (float)(p >> 8);
            sb = bf2f(s1[g]);
            bb = bf2f(b1[g]);
        }
#pragma unroll
        for (int i = 0; i < kInt8RouterTokens; ++i) {
            const int t = min(t0 + i, T - 1);
            const uint32_t xv = *reinterpret_cast<const uint32_t *>(x + (size_t)t * xStride + idx);
            const float x0 = __uint_as_float(xv << 16), x1 = __uint_as_float(xv & 0xFFFF0000u);
            const float sumX = x0 + x1;
            acc0[i] = fmaf(sa, fmaf(q01, x1, q00 * x0), acc0[i]);
            acc0[i] = fmaf(ba, sumX, acc0[i]);
            if (DUAL) {
                acc1[i] = fmaf(sb, fmaf(q11, x1, q10 * x0), acc1[i]);
                acc1[i] = fmaf(bb, sumX, acc1[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kInt8RouterTokens; ++i) {
        float a = acc0[i], b = acc1[i];
#pragma unroll
        for (int offset = 16; offset >= 1; offset >>= 1) {
            a += __shfl_xor_sync(0xFFFFFFFFu, a, offset);
            if (DUAL) b += __shfl_xor_sync(0xFFFFFFFFu, b, offset);
        }
        if (lane == 0 && t0 + i < T) {
            uint16_t v;
            if (DUAL) v = f2bf(gelu_tanh(bf16_round(a)) * bf16_round(b));
            else v = f2bf(a);
            out[(size_t)(t0 + i) * outStride + r] = v;
        }
    }
}

// y = down(r16(gelu_tanh(r16(gate x)) * r16(up x))) for any number of rows; the activations go through
// the context's shared-activation scratch.
bool launch_shared_int8(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride, uint32_t tokens,
                        uint16_t *y, cudaStream_t stream, const char **error) {
    if (tokens == 0) return true;
    if (!L.has_shared8()) return fail(error, "layer has no resident shared FFN");
    const int D = (int)ctx->cfg.d, Fs = (int)ctx->cfg.sharedF;
    if (D % 64 || Fs % 64) return fail(error, "widths must be multiples of 64");
    if (xStride % 2 || ((uintptr_t)x & 3)) return fail(error, "input rows must be 4-byte aligned");
    if (tokens > ctx->cfg.maxTokens) return fail(error, "rows exceed the context's maxTokens");
    uint16_t *acts = ctx->sharedActs;
    const unsigned tokenBlocks = (tokens + kInt8RouterTokens - 1) / kInt8RouterTokens;
    {
        LaunchScope scope(ctx, stream, "shared_int8_gate_up_act");
        k_int8_rows<true><<<dim3((Fs + 7) / 8, tokenBlocks), 256, 0, stream>>>(
            L.shared8W[0], L.shared8S[0], L.shared8B[0], L.shared8W[1], L.shared8S[1], L.shared8B[1], x, xStride,
            (int)tokens, Fs, D, acts, (uint32_t)Fs);
    }
    {
        LaunchScope scope(ctx, stream, "shared_int8_down");
        k_int8_rows<false><<<dim3((D + 7) / 8, tokenBlocks), 256, 0, stream>>>(
            L.shared8W[2], L.shared8S[2], L.shared8B[2], nullptr, nullptr, nullptr, acts, (uint32_t)Fs, (int)tokens, D,
            Fs, y, (uint32_t)D);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

// Top-K of logits rows, one warp per row (the rows' logits are in global memory).
__global__ void __launch_bounds__(256)
k_topk_rows(const float *logits, const uint16_t *gain, int T, int E, int K, uint32_t *ids, uint16_t *weights) {
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= T) return;
    warp_topk(logits + (size_t)t * E, E, K, gain, ids + (size_t)t * K, weights + (size_t)t * K);
}

bool launch_router_logits_int8(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                               uint32_t tokens, float *logits, cudaStream_t stream, const char **error) {
    const int E = (int)L.routerExperts, D = (int)ctx->cfg.d;
    if (xStride % 2 || ((uintptr_t)x & 3)) return fail(error, "input rows must be 4-byte aligned");
    dim3 grid((E + 7) / 8, (tokens + kInt8RouterTokens - 1) / kInt8RouterTokens);
    {
        LaunchScope scope(ctx, stream, "router_logits_int8");
        k_router_logits_int8<<<grid, 256, 0, stream>>>(L.routerQ, L.routerQScale, L.routerQBias, L.routerScale,
                                                       L.logitBias, x, xStride, (int)tokens, E, D, logits);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

bool launch_router_topk(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                        uint32_t tokens, uint32_t *ids, uint16_t *weights, float *logits,
                        cudaStream_t stream, const char **error) {
    if (tokens == 0) return true;
    if (!L.has_router()) return fail(error, "layer has no resident router");
    const int E = (int)L.routerExperts, D = (int)ctx->cfg.d;
    if (L.routerQ && tokens > kMaxGemvRows) {
        float *lg = logits ? logits : ctx->logitsRows;
        if (!launch_router_logits_int8(ctx, L, x, xStride, tokens, lg, stream, error)) return false;
        {
            LaunchScope scope(ctx, stream, "topk_rows");
            k_topk_rows<<<(tokens + 7) / 8, 256, 0, stream>>>(lg, L.gain, (int)tokens, E, (int)ctx->cfg.topK, ids,
                                                             weights);
        }
        FF_CUDA_OK(cudaGetLastError(), error);
        return true;
    }
    if (tokens > kMaxGemvRows)
        return launch_router_prefill(ctx, L, x, xStride, tokens, ids, weights, logits, stream, error);
    float *lg = logits ? logits : ctx->logits;
    if (L.routerQ) {
        if (!launch_router_logits_int8(ctx, L, x, xStride, tokens, lg, stream, error)) return false;
    } else {
        dim3 grid((E + 7) / 8, tokens);
        LaunchScope scope(ctx, stream, "router_logits");
        k_router_logits<<<grid, 256, 0, stream>>>(L.routerW, L.routerScale, L.logitBias, x, xStride,
                                                  E, D, lg);
    }
    PlanArgs a{};
    a.logits = lg;
    a.gain = L.gain;
    a.idsOut = ids;
    a.weightsOut = weights;
    a.T = (int)tokens;
    a.E = E;
    a.K = (int)ctx->cfg.topK;
    a.buildPlan = 0;
    a.errorFlag = ctx->errorFlag;
    {
        LaunchScope scope(ctx, stream, "topk_plan");
        k_topk_plan<<<1, 512, 0, stream>>>(a);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

// Router top-K (when ids is null) + routed experts (+ shared FFN) for up to 16 rows.
//   decodeCombine: one row; y = bf16(residual' + sum_k w_k v_k), residual' = shared output when
//                  withShared else `residual`.
//   otherwise:     partial rows are written; sharedOut receives the shared FFN rows.
bool launch_block_small(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                        uint32_t tokens, const uint32_t *ids, const uint16_t *weights,
                        bool withShared, bool decodeCombine, const uint16_t *residual,
                        uint16_t *partials, uint16_t *sharedOut, uint16_t *y,
                        cudaStream_t stream, const char **error) {
    const FFConfig &c = ctx->cfg;
    if (tokens == 0) return true;
    if (tokens > kMaxGemvRows) return fail(error, "more than 16 rows in a decode/verify block");
    if (decodeCombine && tokens != 1) return fail(error, "decode combine takes exactly one row");
    if (!L.experts) return fail(error, "layer has no resident experts");
    if (withShared && !L.shared) return fail(error, "layer has no resident shared FFN");
    if (decodeCombine)
        return launch_decode_fused(ctx, L, x, ids, weights, withShared, true, residual, y, stream, error);
    const int E = (int)L.expertCount;
    PlanArgs a{};
    uint32_t *idsDev = ctx->ids;
    uint16_t *weightsDev = ctx->weights;
    if (!ids) {
        if (!L.has_router()) return fail(error, "layer has no resident router");
        if (L.routerExperts != L.expertCount) return fail(error, "router and layer disagree on the expert count");
        if (L.routerQ) {
            if (!launch_router_logits_int8(ctx, L, x, xStride, tokens, ctx->logits, stream, error)) return false;
        } else {
            dim3 grid((L.routerExperts + 7) / 8, tokens);
            LaunchScope scope(ctx, stream, "router_logits");
            k_router_logits<<<grid, 256, 0, stream>>>(L.routerW, L.routerScale, L.logitBias, x,
                                                      xStride, (int)L.routerExperts, (int)c.d,
                                                      ctx->logits);
        }
        a.logits = ctx->logits;
        a.gain = L.gain;
        a.idsOut = idsDev;
        a.weightsOut = weightsDev;
    } else {
        a.idsIn = ids;
        idsDev = const_cast<uint32_t *>(ids);
        weightsDev = const_cast<uint16_t *>(weights);
    }
    a.T = (int)tokens;
    a.E = E;
    a.K = (int)c.topK;
    a.D = (int)c.d;
    a.F = (int)c.f;
    a.Fs = (int)c.sharedF;
    a.experts = L.experts;
    a.stride = L.stride;
    a.off = L.off;
    a.shared = withShared ? L.shared : nullptr;
    a.sharedOff = L.sharedOff;
    a.x = x;
    a.xStride = xStride;
    a.acts = ctx->acts;
    a.sharedActs = ctx->sharedActs;
    a.partials = decodeCombine ? nullptr : partials;
    a.sharedOut = sharedOut;
    a.jobs0 = ctx->jobs[0];
    a.jobs1 = ctx->jobs[1];
    a.plan = ctx->plan;
    a.buildPlan = 1;
    a.errorFlag = ctx->errorFlag;
    {
        LaunchScope scope(ctx, stream, "topk_plan");
        k_topk_plan<<<1, 512, 0, stream>>>(a);
    }
    FF_CUDA_OK(cudaGetLastError(), error);

    // the planned jobs run on the tensor-core block kernels
    return launch_block_mma(ctx, x, xStride, tokens, withShared, withShared || !decodeCombine, stream, error);
}

bool launch_reduce(FFContext *ctx, const uint16_t *partials, const uint16_t *weights,
                   const uint16_t *residual, uint16_t *y, uint32_t tokens, cudaStream_t stream,
                   const char **error, const uint32_t *rowIndex) {
    if (tokens == 0) return true;
    const int D = (int)ctx->cfg.d;
    const bool wide = D % 8 == 0 && !((reinterpret_cast<uintptr_t>(partials) | reinterpret_cast<uintptr_t>(y) |
                                        reinterpret_cast<uintptr_t>(residual)) & 15u);
    {
        LaunchScope scope(ctx, stream, "reduce_token_major");
        if (wide) {
            const size_t items = (size_t)tokens * (D / 8);
            k_reduce_token_major_x8<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(
                partials, rowIndex, weights, residual, y, (int)tokens, (int)ctx->cfg.topK, D);
        } else {
            dim3 grid((D / 2 + 255) / 256, tokens);
            k_reduce_token_major<<<grid, 256, 0, stream>>>(partials, rowIndex, weights, residual, y, (int)tokens,
                                                           (int)ctx->cfg.topK, D);
        }
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

bool launch_gemv_rows(FFContext *ctx, const FFProjection &p, const uint16_t *x, uint32_t xStride,
                      uint32_t rows, uint16_t *y, uint32_t yStride, cudaStream_t stream,
                      const char **error) {
    if (rows == 0) return true;
    if (rows > kMaxGemvRows) return fail(error, "ff_int4_gemv_rows takes at most 16 input rows");
    if (p.cols % kGroup != 0) return fail(error, "columns must be a multiple of 64");
    if ((reinterpret_cast<uintptr_t>(p.weights) & 15u) || (p.cols / 2) % 16 != 0)
        return fail(error, "packed weights must be 16-byte aligned with 16-byte-multiple rows");
    GemvJob job{};
    job.w0 = static_cast<const uint8_t *>(p.weights);
    job.s0 = static_cast<const uint16_t *>(p.scales);
    job.b0 = static_cast<const uint16_t *>(p.biases);
    job.in = x;
    job.out = y;
    job.rows = p.rows;
    job.cols = p.cols;
    job.inStride = xStride;
    job.outStride = yStride;
    job.n = rows;
    for (uint32_t i = 0; i < kMaxGemvRows; ++i) job.inRow[i] = job.outRow[i] = i < rows ? i : 0u;
    return launch_inline_job<false>(ctx, job, stream, error);
}

// Shared FFN for up to 16 rows without a route plan: gate/up/GeGLU job, then the down job.
bool launch_shared_small(FFContext *ctx, const LayerStore &L, const uint16_t *x, uint32_t xStride,
                         uint32_t tokens, uint16_t *y, cudaStream_t stream, const char **error) {
    const FFConfig &c = ctx->cfg;
    if (tokens == 0) return true;
    if (!L.shared) return fail(error, "layer has no resident shared FFN");
    GemvJob j0{};
    j0.w0 = L.shared + L.sharedOff.gateWOff;
    j0.s0 = reinterpret_cast<const uint16_t *>(L.shared + L.sharedOff.gateSOff);
    j0.b0 = reinterpret_cast<const uint16_t *>(L.shared + L.sharedOff.gateBOff);
    j0.w1 = L.shared + L.sharedOff.upWOff;
    j0.s1 = reinterpret_cast<const uint16_t *>(L.shared + L.sharedOff.upSOff);
    j0.b1 = reinterpret_cast<const uint16_t *>(L.shared + L.sharedOff.upBOff);
    j0.in = x;
    j0.out = ctx->sharedActs;
    j0.rows = c.sharedF;
    j0.cols = c.d;
    j0.inStride = xStride;
    j0.outStride = c.sharedF;
    j0.n = tokens;
    j0.flags = kJobRoundGateUp;
    GemvJob j1{};
    j1.w0 = L.shared + L.sharedOff.downWOff;
    j1.s0 = reinterpret_cast<const uint16_t *>(L.shared + L.sharedOff.downSOff);
    j1.b0 = reinterpret_cast<const uint16_t *>(L.shared + L.sharedOff.downBOff);
    j1.in = ctx->sharedActs;
    j1.out = y;
    j1.rows = c.d;
    j1.cols = c.sharedF;
    j1.inStride = c.sharedF;
    j1.outStride = c.d;
    j1.n = tokens;
    for (uint32_t i = 0; i < kMaxGemvRows; ++i)
        j0.inRow[i] = j0.outRow[i] = j1.inRow[i] = j1.outRow[i] = i < tokens ? i : 0u;
    if (!launch_inline_job<true>(ctx, j0, stream, error)) return false;
    return launch_inline_job<false>(ctx, j1, stream, error);
}

bool launch_rmsnorm(FFContext *ctx, const uint16_t *x, const uint16_t *w, float eps,
                    uint32_t tokens, uint16_t *y, cudaStream_t stream, const char **error) {
    if (tokens == 0) return true;
    {
        LaunchScope scope(ctx, stream, "rmsnorm");
        k_rmsnorm<<<tokens, 256, 0, stream>>>(x, w, eps, (int)ctx->cfg.d, y);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

bool launch_dequant_probe(FFContext *ctx, const uint8_t *w, const uint16_t *s, const uint16_t *b,
                          uint32_t rows, uint32_t cols, float *out32, uint16_t *out16,
                          cudaStream_t stream, const char **error) {
    const size_t words = (size_t)rows * cols / 8;
    {
        LaunchScope scope(ctx, stream, "dequant_probe");
        k_dequant_probe<<<(unsigned)((words + 255) / 256), 256, 0, stream>>>(w, s, b, (int)rows,
                                                                             (int)cols, out32, out16);
    }
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

}  // namespace ff

// ---- shared FFN without any allocation -----------------------------------------------------

// Scratch for ff_shared_ffn_noalloc: the GeGLU activations between the gate/up kernel and the
// down kernel, [kNoAllocMaxRows][kNoAllocMaxIntermediate] bf16 = 128 KiB.  It is part of the
// library image, so every GPU that loads the library holds it until the process exits.
constexpr uint32_t kNoAllocMaxRows = 16;
constexpr uint32_t kNoAllocMaxIntermediate = 4096;
constexpr uint32_t kNoAllocMaxWidth = 16384;
static __device__ __align__(256) uint16_t g_noAllocActs[kNoAllocMaxRows * kNoAllocMaxIntermediate];

extern "C" bool ff_shared_ffn_noalloc(const FFProjection *gate, const FFProjection *up,
                                      const FFProjection *down, const uint16_t *x,
                                      uint32_t xStride, uint32_t rows, uint16_t *y,
                                      uint32_t yStride, void *stream, const char **error) {
    using namespace ff;
    if (error) *error = nullptr;
    if (!gate || !up || !down || !x || !y) return fail(error, "null argument");
    if (rows == 0) return true;
    if (rows > kNoAllocMaxRows)
        return fail(error, "ff_shared_ffn_noalloc takes at most " + std::to_string(kNoAllocMaxRows) +
                               " rows, got " + std::to_string(rows));
    const uint32_t d = gate->cols, f = gate->rows;
    if (f > kNoAllocMaxIntermediate)
        return fail(error, "intermediate width " + std::to_string(f) +
                               " exceeds the static scratch's maximum of " +
                               std::to_string(kNoAllocMaxIntermediate));
    if (d > kNoAllocMaxWidth)
        return fail(error, "model width " + std::to_string(d) + " exceeds the maximum of " +
                               std::to_string(kNoAllocMaxWidth) + " (one input row must fit in shared memory)");
    if (up->rows != f || up->cols != d || down->rows != d || down->cols != f)
        return fail(error, "SharedExpert dimension mismatch: gate=(" + std::to_string(gate->rows) + "," +
                               std::to_string(gate->cols) + ") up=(" + std::to_string(up->rows) + "," +
                               std::to_string(up->cols) + ") down=(" + std::to_string(down->rows) + "," +
                               std::to_string(down->cols) + ")");
    if (d % kGroup || f % kGroup || d == 0 || f == 0)
        return fail(error, "widths must be non-zero multiples of the group size 64");
    if (xStride < d || yStride < d || xStride % 2) return fail(error, "row stride is too small or odd");
    if ((reinterpret_cast<uintptr_t>(x) & 3u) || (reinterpret_cast<uintptr_t>(y) & 1u))
        return fail(error, "input rows must be 4-byte aligned and output rows 2-byte aligned");
    const FFProjection *ps[3] = {gate, up, down};
    for (const FFProjection *p : ps)
        if (!p->weights || !p->scales || !p->biases || (reinterpret_cast<uintptr_t>(p->weights) & 15u) ||
            (reinterpret_cast<uintptr_t>(p->scales) & 1u) || (reinterpret_cast<uintptr_t>(p->biases) & 1u))
            return fail(error, "projection pointers must be non-null, the weights 16-byte aligned, scales and "
                               "biases 2-byte aligned");
    // both kernels' staging must fit before anything is enqueued (wide matrices run as passes of
    // fewer rows; kNoAllocMaxWidth and kNoAllocMaxIntermediate guarantee that one row always fits)
    if (gemv_pass_rows(rows, d) == 0 || gemv_pass_rows(rows, f) == 0)
        return fail(error, "one input row does not fit in shared memory");

    // Per-device set-up, done by the first call on each device with that device current: the
    // array's name is only a host-side handle, so its device address is looked up here.
    struct DeviceSetup {
        uint16_t *scratch = nullptr;
        int smCount = 0;
    };
    static DeviceSetup setups[kMaxDevices];
    static std::mutex setupLock;
    int device = 0;
    FF_CUDA_OK(cudaGetDevice(&device), error);
    if (device < 0 || device >= kMaxDevices) return fail(error, "device ordinal out of range");
    DeviceSetup setup;
    {
        std::lock_guard<std::mutex> guard(setupLock);
        if (!setups[device].scratch) {
            void *ptr = nullptr;
            FF_CUDA_OK(cudaGetSymbolAddress(&ptr, g_noAllocActs), error);
            int sms = 0;
            FF_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), error);
            if (!ptr || sms <= 0) return fail(error, "could not set up the static scratch on this device");
            setups[device].smCount = sms;
            setups[device].scratch = static_cast<uint16_t *>(ptr);
        }
        setup = setups[device];
    }

    FFContext local;  // launch bookkeeping only: owns nothing on the device
    local.device = device;
    local.smCount = setup.smCount;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    GemvJob j0{}, j1{};
    j0.w0 = static_cast<const uint8_t *>(gate->weights);
    j0.s0 = static_cast<const uint16_t *>(gate->scales);
    j0.b0 = static_cast<const uint16_t *>(gate->biases);
    j0.w1 = static_cast<const uint8_t *>(up->weights);
    j0.s1 = static_cast<const uint16_t *>(up->scales);
    j0.b1 = static_cast<const uint16_t *>(up->biases);
    j0.in = x;
    j0.out = setup.scratch;
    j0.rows = f;
    j0.cols = d;
    j0.inStride = xStride;
    j0.outStride = f;
    j0.n = rows;
    j0.flags = kJobRoundGateUp;
    j1.w0 = static_cast<const uint8_t *>(down->weights);
    j1.s0 = static_cast<const uint16_t *>(down->scales);
    j1.b0 = static_cast<const uint16_t *>(down->biases);
    j1.in = setup.scratch;
    j1.out = y;
    j1.rows = d;
    j1.cols = f;
    j1.inStride = f;
    j1.outStride = yStride;
    j1.n = rows;
    for (uint32_t i = 0; i < (uint32_t)kMaxGemvRows; ++i)
        j0.inRow[i] = j0.outRow[i] = j1.inRow[i] = j1.outRow[i] = i < rows ? i : 0u;
    if (!launch_inline_job<true>(&local, j0, s, error)) return false;
    return launch_inline_job<false>(&local, j1, s, error);
}

