// One token through the whole MoE block in ONE cooperative kernel: router, top-8, routed
// gate/up/GeGLU, shared FFN, routed down and the weighted combine.
//
// The step streams 37.5 MB of weights once; at B200's HBM rate that is under 6 us, so separate
// kernels (launch gaps, cold starts) cannot come near the roofline.  Here one CTA per SM runs
// three phases separated by two grid-wide barriers:
//   A  L2 prefetch of everything known up front (router, shared FFN); router logits (one warp per
//      expert) and the shared gate/up/GeGLU rows;
//   B  every CTA ranks the 128 logits itself (top-8, softmax, gain), issues L2 prefetches for
//      the eight chosen experts' blobs, then routed gate/up/GeGLU rows and the shared down rows;
//   C  routed down rows, warp = slot, fixed-order combine onto the shared output (or the
//      caller's residual).
// The prefetches (one bulk L2 prefetch instruction per 8 KiB) keep HBM busy independently of how
// many loads the compute warps have in flight; the compute loads then hit L2.
// Row arithmetic is row_dot<1, ...> of the generic GEMV kernels, so the result is bitwise the one
// the split operators (ff_router_topk, ff_shared_ffn, ff_moe_decode) produce.
//
// The grid barrier is a sense-reversing counter in global memory; cooperative launch guarantees
// that all CTAs are resident.  Its spin is bounded: on running out it raises the context's error
// flag and the CTA returns.
//
// Reference kernels replaced (paths inside the reference project):
//   Sources/ANEFieldfareHotpath/Metal/MoE/moe.metal:65-120,242-319,500-517,548-570,597-638
//   Sources/ANEFieldfareHotpath/Metal/Quant/dequant_int4.metal:78-169
#include <algorithm>
#include <cstdlib>

#include "ff_gemv_device.cuh"
#include "ff_internal.cuh"

namespace ff {

constexpr int kFusedThreads = 512;
constexpr int kFusedWarps = kFusedThreads / 32;
constexpr uint32_t kBarrierSpinLimit = 1u << 24;

struct DecodeArgs {
    const uint16_t *routerW, *routerScale, *gain;
    const float *logitBias;
    const uint8_t *experts;
    uint64_t stride;
    FFExpertOffsets off;
    const uint8_t *shared;  // null: no shared FFN, `residual` is added instead
    FFExpertOffsets sharedOff;
    uint64_t sharedBytes;
    const uint16_t *x;
    const uint16_t *residual;
    const uint32_t *idsIn;  // non-null: routes are given, the router is skipped
    const uint16_t *weightsIn;
    float *logits;
    uint32_t *ids;
    uint16_t *weights;
    uint16_t *acts, *sharedActs, *h1, *y;
    uint32_t *barrier;  // [0] arrivals, [1] sense
    uint32_t *errorFlag;
    unsigned long long *stamps;  // null, or 8 slots for block 0's phase timestamps (ns)
    int E, D, F, Fs, K;
    int prefetch;  // 0: no L2 prefetch (diagnostic)
};

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bulk L2 prefetch of [p, p + bytes); bytes a multiple of 16, p 16-byte aligned.
__device__ __forceinline__ void prefetch_l2_bulk(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// The grid prefetches [base, base+bytes) in 8 KiB pieces.  Piece i belongs to CTA (i + cursor) mod
// gridDim and to one thread of it, so every SM issues the same share: a bulk prefetch is executed
// by the issuing SM's copy engine, whose throughput is a small fraction of HBM's.
__device__ __forceinline__ void prefetch_region(const uint8_t *base, uint64_t bytes, uint32_t &cursor) {
    constexpr uint32_t kPiece = 8192;
    const uint32_t pieces = (uint32_t)((bytes + kPiece - 1) / kPiece);
    const uint32_t first = (blockIdx.x + gridDim.x - cursor % gridDim.x) % gridDim.x;
    for (uint32_t i = first + threadIdx.x * gridDim.x; i < pieces; i += gridDim.x * blockDim.x) {
        const uint64_t offset = (uint64_t)i * kPiece;
        const uint32_t len = (uint32_t)min((uint64_t)kPiece, bytes - offset) & ~15u;
        if (len) prefetch_l2_bulk(base + offset, len);
    }
    cursor += pieces;
}

// Sense-reversing grid barrier with a bounded spin.  Returns false when the wait ran out.
__device__ bool grid_barrier(uint32_t *bar, uint32_t &sense, uint32_t *errorFlag, volatile uint32_t *sOk) {
    __syncthreads();
    if (threadIdx.x == 0) {
        sense ^= 1u;
        __threadfence();
        const uint32_t arrived = atomicAdd(&bar[0], 1u);
        uint32_t ok = 1u;
        if (arrived == gridDim.x - 1) {
            bar[0] = 0u;
            __threadfence();
            atomicExch(&bar[1], sense);
        } else {
            uint32_t spins = 0;
            while (ld_acquire_u32(&bar[1]) != sense) {
                if (++spins > kBarrierSpinLimit) {
                    atomicExch(errorFlag, 9u);
                    ok = 0u;
                    break;
                }
            }
        }
        __threadfence();
        *sOk = ok;
    }
    __syncthreads();
    return *sOk != 0u;
}

__device__ __forceinline__ void stamp(const DecodeArgs &a, int slot) {
    if (a.stamps && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        a.stamps[slot] = t;
    }
}

__global__ void __launch_bounds__(kFusedThreads, 1) k_decode_fused(const DecodeArgs a) {
    extern __shared__ float smem[];
    __shared__ float sLogits[kMaxExperts];
    __shared__ uint32_t sIds[8];
    __shared__ float sWeights[8];
    __shared__ float sScore[8];
    __shared__ uint32_t sRowIdx[8];
    __shared__ volatile uint32_t sOk;
    __shared__ uint32_t sSense;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // consecutive tasks go to different SMs: global warp w is warp (w / gridDim) of CTA (w % gridDim)
    const int gwarp = warp * (int)gridDim.x + (int)blockIdx.x;
    const int totalWarps = gridDim.x * kFusedWarps;
    const int D = a.D, F = a.F, Fs = a.Fs, K = a.K, E = a.E;

    // shared-memory regions: x (kept through phase B), then a region reused by phases B and C
    float *xs = smem;
    float *xsum = xs + staged_stride(D);
    float *region = xsum + (D >> 5);

    if (threadIdx.x == 0) sSense = ld_acquire_u32(&a.barrier[1]);
    if (threadIdx.x < 8) sRowIdx[threadIdx.x] = threadIdx.x;
    uint32_t cursor = 0;
    stamp(a, 0);
    // ---------------- phase A ----------------
    if (a.prefetch && a.shared) prefetch_region(a.shared, a.sharedBytes, cursor);
    if (a.prefetch && !a.idsIn) prefetch_region(reinterpret_cast<const uint8_t *>(a.routerW), (uint64_t)E * D * 2, cursor);
    __syncthreads();
    uint32_t sense = sSense;
    {
        const uint32_t zero = 0;
        stage_rows(a.x, (uint32_t)D, &zero, 1, D, xs, xsum);
    }
    if (!a.idsIn) {
        for (int e = gwarp; e < E; e += totalWarps) {
            const uint16_t *wr = a.routerW + (size_t)e * D;
            float acc = 0.0f;
            for (int base = 8 * lane; base < D; base += 256) {
                const uint4 wv = *reinterpret_cast<const uint4 *>(wr + base);
                const uint4 xv = *reinterpret_cast<const uint4 *>(a.x + base);
                uint4 sv = make_uint4(0, 0, 0, 0);
                if (a.routerScale) sv = *reinterpret_cast<const uint4 *>(a.routerScale + base);
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
                const uint32_t xx[4] = {xv.x, xv.y, xv.z, xv.w};
                const uint32_t ss[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float x0 = __uint_as_float(xx[k] << 16), x1 = __uint_as_float(xx[k] & 0xFFFF0000u);
                    if (a.routerScale) {
                        x0 = x0 * __uint_as_float(ss[k] << 16);
                        x1 = x1 * __uint_as_float(ss[k] & 0xFFFF0000u);
                    }
                    acc = fmaf(__uint_as_float(ww[k] << 16), x0, acc);
                    acc = fmaf(__uint_as_float(ww[k] & 0xFFFF0000u), x1, acc);
                }
            }
#pragma unroll
            for (int offset = 16; offset >= 1; offset >>= 1)
                acc += __shfl_xor_sync(0xFFFFFFFFu, acc, offset);
            if (lane == 0) a.logits[e] = a.logitBias ? acc + a.logitBias[e] : acc;
        }
    }
    if (a.shared) {
        // shared gate/up/GeGLU: four rows per warp task, interleaved after the router's warps
        const uint8_t *gw = a.shared + a.sharedOff.gateWOff, *uw = a.shared + a.sharedOff.upWOff;
        const uint16_t *gs = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.gateSOff);
        const uint16_t *gb = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.gateBOff);
        const uint16_t *us = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.upSOff);
        const uint16_t *ub = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.upBOff);
        const int tasks = (Fs + 3) / 4;
        const int skew = a.idsIn ? 0 : E % totalWarps;
        for (int t = (gwarp + totalWarps - skew) % totalWarps; t < tasks; t += totalWarps) {
            const int row = t * 4 + (lane >> 3);
            float g[1], u[1];
            row_dot<1, true>(gw, gs, gb, uw, us, ub, row, D, row < Fs, xs, xsum, 1, g, u);
            if (row < Fs && (lane & 7) == 0)
                a.sharedActs[row] = f2bf(gelu_tanh(bf16_round(g[0])) * bf16_round(u[0]));
        }
    }
    stamp(a, 1);
    if (!grid_barrier(a.barrier, sense, a.errorFlag, &sOk)) return;
    stamp(a, 2);

    // ---------------- phase B ----------------
    if (!a.idsIn) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) sLogits[e] = a.logits[e];
        if (threadIdx.x < 8) {
            sIds[threadIdx.x] = 0u;
            sScore[threadIdx.x] = -INFINITY;
        }
        __syncthreads();
        // rank of every logit under (higher score, then lower expert id); scores of -inf or NaN
        // are never taken — the order of the serial top-8 (moe.metal:269-303)
        // four threads per expert, each counting a quarter of the competitors
        for (int idx = threadIdx.x; idx < 4 * ((E + 127) & ~127); idx += blockDim.x) {
            const int e = idx >> 2, part = idx & 3;
            const float v = e < E ? sLogits[e] : -INFINITY;
            const int span = (E + 3) >> 2;
            int rank = 0;
            if (v > -INFINITY) {
                const int end = min(E, (part + 1) * span);
                for (int o = part * span; o < end; ++o) {
                    const float w = sLogits[o];
                    rank += (w > -INFINITY && (w > v || (w == v && o < e))) ? 1 : 0;
                }
            }
            rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 1);
            rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 2);
            if (part == 0 && v > -INFINITY && rank < K) {
                sIds[rank] = (uint32_t)e;
                sScore[rank] = v;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float ex[8], sum = 0.0f;
            for (int r = 0; r < K; ++r) {
                ex[r] = expf(sScore[r] - sScore[0]);
                sum += ex[r];
            }
            for (int r = 0; r < K; ++r) {
                float w = ex[r] / sum;
                if (a.gain) w = w * bf2f(a.gain[sIds[r]]);
                const uint16_t wb = f2bf(w);
                sWeights[r] = bf2f(wb);
                if (blockIdx.x == 0) {
                    a.ids[r] = sIds[r];
                    a.weights[r] = wb;
                }
            }
        }
    } else if (threadIdx.x < K) {
        sIds[threadIdx.x] = a.idsIn[threadIdx.x];
        sWeights[threadIdx.x] = bf2f(a.weightsIn[threadIdx.x]);
    }
    __syncthreads();
    stamp(a, 3);
    for (int k = 0; k < K && a.prefetch; ++k) {
        const uint8_t *blob = a.experts + (size_t)sIds[k] * a.stride;
        prefetch_region(blob, (uint64_t)a.off.downBOff + (uint64_t)D * F / kGroup * 2, cursor);
    }
    {
        // routed gate/up/GeGLU: task = (slot, four rows)
        const int perSlot = (F + 3) / 4;
        const int tasks = K * perSlot;
        for (int t = gwarp; t < tasks; t += totalWarps) {
            const int slot = t / perSlot;
            const int row = (t - slot * perSlot) * 4 + (lane >> 3);
            const uint8_t *blob = a.experts + (size_t)sIds[slot] * a.stride;
            float g[1], u[1];
            row_dot<1, true>(blob + a.off.gateWOff, reinterpret_cast<const uint16_t *>(blob + a.off.gateSOff),
                             reinterpret_cast<const uint16_t *>(blob + a.off.gateBOff), blob + a.off.upWOff,
                             reinterpret_cast<const uint16_t *>(blob + a.off.upSOff),
                             reinterpret_cast<const uint16_t *>(blob + a.off.upBOff), row, D, row < F, xs,
                             xsum, 1, g, u);
            if (row < F && (lane & 7) == 0) a.acts[slot * F + row] = f2bf(gelu_tanh(g[0]) * u[0]);
        }
    }
    if (a.shared) {
        // shared down rows from the activations phase A wrote
        float *as = region;
        float *asum = as + staged_stride(Fs);
        const uint32_t zero = 0;
        stage_rows(a.sharedActs, (uint32_t)Fs, &zero, 1, Fs, as, asum);
        const uint8_t *dw = a.shared + a.sharedOff.downWOff;
        const uint16_t *ds = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.downSOff);
        const uint16_t *db = reinterpret_cast<const uint16_t *>(a.shared + a.sharedOff.downBOff);
        const int tasks = (D + 3) / 4;
        const int skew = (K * ((F + 3) / 4)) % totalWarps;
        for (int t = (gwarp + totalWarps - skew) % totalWarps; t < tasks; t += totalWarps) {
            const int row = t * 4 + (lane >> 3);
            float v[1], unused[1];
            row_dot<1, false>(dw, ds, db, nullptr, nullptr, nullptr, row, Fs, row < D, as, asum, 1, v, unused);
            if (row < D && (lane & 7) == 0) a.h1[row] = f2bf(v[0]);
        }
    }
    stamp(a, 4);
    if (!grid_barrier(a.barrier, sense, a.errorFlag, &sOk)) return;
    stamp(a, 5);

    // ---------------- phase C ----------------
    {
        float *as = region;
        const int strideF = staged_stride(F);
        float *asum = as + 8 * strideF;
        stage_rows(a.acts, (uint32_t)F, sRowIdx, K, F, as, asum);
        const uint16_t *res = a.shared ? a.h1 : a.residual;
        const int chunks = F >> 5, groups = F >> 6, j = lane & 7;
        const int tasks = (D + 3) / 4;
        for (int t = gwarp; t < tasks; t += totalWarps) {
            const int row = t * 4 + (lane >> 3);
            const bool live = row < D;
            float acc = (live && res) ? bf2f(res[row]) : 0.0f;
            if (chunks <= 24) {
                // every slot's row is at most three 16-byte chunks per lane: the next slot's chunks
                // are fetched while this slot's are accumulated (rolled loop, generic order)
                uint4 wv[3], wn[3];
                uint32_t sbv[3], sbn[3];  // scale | bias << 16
                auto fetch = [&](int k, uint4 (&w)[3], uint32_t (&sb)[3]) {
                    const uint8_t *blob = a.experts + (size_t)sIds[k] * a.stride;
                    const uint4 *p = reinterpret_cast<const uint4 *>(blob + a.off.downWOff + (size_t)row * (F >> 1));
                    const uint16_t *sr = reinterpret_cast<const uint16_t *>(blob + a.off.downSOff) + (size_t)row * groups;
                    const uint16_t *br = reinterpret_cast<const uint16_t *>(blob + a.off.downBOff) + (size_t)row * groups;
#pragma unroll
                    for (int it = 0; it < 3; ++it) {
                        const int c = j + 8 * it;
                        if (c < chunks) {
                            w[it] = load_stream(p + c);
                            sb[it] = (uint32_t)sr[c >> 1] | ((uint32_t)br[c >> 1] << 16);
                        }
                    }
                };
                if (live) fetch(0, wv, sbv);
#pragma unroll 1
                for (int k = 0; k < K; ++k) {
                    if (live && k + 1 < K) fetch(k + 1, wn, sbn);
                    float part = 0.0f;
                    if (live) {
                        const float *xk = as + k * strideF;
                        const float *sk = asum + k * chunks;
#pragma unroll
                        for (int it = 0; it < 3; ++it) {
                            const int c = j + 8 * it;
                            if (c < chunks) {
                                const float sc = __uint_as_float(sbv[it] << 16);
                                const float bi = fmaf(-16.0f, sc, __uint_as_float(sbv[it] & 0xFFFF0000u));
                                const float *xc = xk + ((c >> 3) << 8) + ((c & 7) << 2);
                                const uint32_t words[4] = {wv[it].x, wv[it].y, wv[it].z, wv[it].w};
                                float d = 0.0f;
#pragma unroll
                                for (int w4 = 0; w4 < 4; ++w4) {
                                    float qf[8];
                                    unpack8_plus16(words[w4], qf);
                                    const float4 xa = *reinterpret_cast<const float4 *>(xc + (w4 << 6));
                                    const float4 xb = *reinterpret_cast<const float4 *>(xc + (w4 << 6) + 32);
                                    d = fmaf(qf[0], xa.x, d);
                                    d = fmaf(qf[1], xa.y, d);
                                    d = fmaf(qf[2], xa.z, d);
                                    d = fmaf(qf[3], xa.w, d);
                                    d = fmaf(qf[4], xb.x, d);
                                    d = fmaf(qf[5], xb.y, d);
                                    d = fmaf(qf[6], xb.z, d);
                                    d = fmaf(qf[7], xb.w, d);
                                }
                                part = fmaf(sc, d, part);
                                part = fmaf(bi, sk[c], part);
                            }
                        }
                    }
                    part += __shfl_xor_sync(0xFFFFFFFFu, part, 4);
                    part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
                    part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
                    acc = __fadd_rn(acc, __fmul_rn(sWeights[k], part));
#pragma unroll
                    for (int it = 0; it < 3; ++it) {
                        wv[it] = wn[it];
                        sbv[it] = sbn[it];
                    }
                }
            } else {
#pragma unroll 1
                for (int k = 0; k < K; ++k) {
                    const uint8_t *blob = a.experts + (size_t)sIds[k] * a.stride;
                    float v[1], unused[1];
                    row_dot<1, false>(blob + a.off.downWOff, reinterpret_cast<const uint16_t *>(blob + a.off.downSOff),
                                      reinterpret_cast<const uint16_t *>(blob + a.off.downBOff), nullptr, nullptr,
                                      nullptr, row, F, live, as + k * strideF, asum + k * chunks, 1, v, unused);
                    acc = __fadd_rn(acc, __fmul_rn(sWeights[k], v[0]));
                }
            }
            if (live && j == 0) a.y[row] = f2bf(acc);
        }
    }
    stamp(a, 6);
}

static size_t fused_smem_bytes(const FFConfig &c) {
    const size_t xPart = (size_t)staged_stride((int)c.d) + (c.d >> 5);
    const size_t sharedPart = c.sharedF ? (size_t)staged_stride((int)c.sharedF) + (c.sharedF >> 5) : 0;
    const size_t actsPart = (size_t)8 * (staged_stride((int)c.f) + (c.f >> 5));
    return (xPart + std::max(sharedPart, actsPart)) * sizeof(float);
}

// One decode row through router (unless ids are given), routed experts and the shared FFN (or
// the caller's residual), as one cooperative launch.
bool launch_decode_fused(FFContext *ctx, const LayerStore &L, const uint16_t *x, const uint32_t *idsIn,
                         const uint16_t *weightsIn, bool withShared, const uint16_t *residual,
                         uint16_t *y, cudaStream_t stream, const char **error) {
    const FFConfig &c = ctx->cfg;
    if (!L.experts) return fail(error, "layer has no resident experts");
    if (!idsIn && !L.routerW) return fail(error, "layer has no resident router");
    if (withShared && !L.shared) return fail(error, "layer has no resident shared FFN");
    if (c.topK > 8) return fail(error, "decode supports at most 8 routes");
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
    uint64_t payload = 0;
    if (c.sharedF) packed_offsets(c.d, c.sharedF, &payload);
    a.sharedBytes = payload;
    a.x = x;
    a.residual = residual;
    a.idsIn = idsIn;
    a.weightsIn = weightsIn;
    a.logits = ctx->logits;
    a.ids = ctx->ids;
    a.weights = ctx->weights;
    a.acts = ctx->acts;
    a.sharedActs = ctx->sharedActs;
    a.h1 = ctx->h1;
    a.y = y;
    a.barrier = ctx->gridBarrier;
    a.errorFlag = ctx->errorFlag;
    a.stamps = ctx->tracing ? ctx->phaseStamps : nullptr;
    static int prefetchMode = -1;
    if (prefetchMode < 0) {
        const char *env = getenv("FF_DECODE_PREFETCH");
        prefetchMode = env ? atoi(env) : 1;
    }
    a.prefetch = prefetchMode;
    a.E = idsIn ? (int)L.expertCount : (int)L.routerExperts;
    a.D = (int)c.d;
    a.F = (int)c.f;
    a.Fs = (int)c.sharedF;
    a.K = (int)c.topK;
    const size_t smem = fused_smem_bytes(c);
    static size_t configured[8] = {0};
    static int gridFor[8] = {0};
    const int slot = ctx->device & 7;
    if (configured[slot] != smem) {
        FF_CUDA_OK(cudaFuncSetAttribute(k_decode_fused, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem),
                   error);
        int perSm = 0;
        FF_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, k_decode_fused, kFusedThreads,
                                                                 smem),
                   error);
        if (perSm < 1) return fail(error, "fused decode kernel does not fit on an SM");
        gridFor[slot] = ctx->smCount;
        configured[slot] = smem;
    }
    void *params[] = {&a};
    {
        LaunchScope scope(ctx, stream, "decode_fused");
        FF_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(k_decode_fused), dim3(gridFor[slot]),
                                               dim3(kFusedThreads), params, smem, stream),
                   error);
    }
    return true;
}

}  // namespace ff
