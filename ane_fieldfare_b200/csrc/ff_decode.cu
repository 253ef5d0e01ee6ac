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
    uint32_t slotsOffset, bigBytes, smallBytes;  // shared-memory staging slots (fused_layout)
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

// ---- per-warp staging of weight rows in shared memory ----------------------------------------
// A warp task covers four consecutive weight rows.  All of their bytes are requested at once with
// asynchronous copies (16 bytes per lane and request, contiguous across the warp; 8 bytes for the
// scale/bias runs whose start is only 8-byte aligned), so a warp has its whole task in flight
// instead of a few loads; the arithmetic then reads the rows from shared memory.

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.wait_all;" ::: "memory");
}
__device__ __forceinline__ uint32_t sm_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void warp_copy16(uint8_t *dst, const uint8_t *src, int bytes) {
    const int lane = threadIdx.x & 31;
    for (int off = lane * 16; off < bytes; off += 512) cp_async16(sm_addr(dst + off), src + off);
}
__device__ __forceinline__ void warp_copy8(uint8_t *dst, const uint8_t *src, int bytes) {
    const int lane = threadIdx.x & 31;
    for (int off = lane * 8; off < bytes; off += 256) cp_async8(sm_addr(dst + off), src + off);
}
__host__ __device__ inline int pad16(int bytes) { return (bytes + 15) & ~15; }

// Shared-memory image of up to four rows of one matrix: packed codes, then scales, then biases.
struct RowsImage {
    int wBytes, sBytes;  // per image: 4 * cols/2 and pad16(4 * groups * 2)
    __host__ __device__ int bytes() const { return wBytes + 2 * sBytes; }
};
__host__ __device__ inline RowsImage rows_image(int cols) {
    return RowsImage{4 * (cols >> 1), pad16(4 * (cols >> 6) * 2)};
}

// Requests rows [row0, row0+4) (clipped to `rows`) of the matrix at (w, s, b) into `dst`.
__device__ __forceinline__ void stage_matrix_rows(uint8_t *dst, const RowsImage &im, const uint8_t *w,
                                                  const uint8_t *s, const uint8_t *b, int row0, int rows,
                                                  int cols) {
    const int n = min(4, rows - row0);
    if (n <= 0) return;
    const int groups = cols >> 6;
    warp_copy16(dst, w + (size_t)row0 * (cols >> 1), n * (cols >> 1));
    warp_copy8(dst + im.wBytes, s + (size_t)row0 * groups * 2, n * groups * 2);
    warp_copy8(dst + im.wBytes + im.sBytes, b + (size_t)row0 * groups * 2, n * groups * 2);
}

constexpr int kBigWarps = 10;  // warps with a large staging slot (gate/up pairs, down x 8 slots)

__global__ void __launch_bounds__(kFusedThreads, 1) k_decode_fused(const DecodeArgs a) {
    const int kSelZero[1] = {0};
    extern __shared__ __align__(16) uint8_t smemRaw[];
    __shared__ float sLogits[kMaxExperts];
    __shared__ uint32_t sIds[8];
    __shared__ float sWeights[8];
    __shared__ float sScore[8];
    __shared__ uint32_t sRowIdx[8];
    __shared__ volatile uint32_t sOk;
    __shared__ uint32_t sSense;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = (int)gridDim.x, cta = (int)blockIdx.x;
    const int D = a.D, F = a.F, Fs = a.Fs, K = a.K, E = a.E;
    const int j = lane & 7, r4 = lane >> 3;

    // shared memory: x (fp32, staged order) | region for the shared / routed activations |
    // kBigWarps big staging slots | small staging slots for the remaining warps
    float *xs = reinterpret_cast<float *>(smemRaw);
    float *xsum = xs + staged_stride(D);
    float *region = xsum + (D >> 5);
    uint8_t *slots = smemRaw + a.slotsOffset;
    uint8_t *mySlot = warp < kBigWarps ? slots + (size_t)warp * a.bigBytes
                                        : slots + (size_t)kBigWarps * a.bigBytes + (size_t)(warp - kBigWarps) * a.smallBytes;
    const RowsImage imD = rows_image(D), imF = rows_image(F), imFs = rows_image(Fs);

    if (threadIdx.x == 0) sSense = ld_acquire_u32(&a.barrier[1]);
    if (threadIdx.x < 8) sRowIdx[threadIdx.x] = threadIdx.x;
    uint32_t cursor = 0;
    stamp(a, 0);

    // ---------------- phase A: router logits, shared gate/up/GeGLU ----------------
    const uint8_t *sh = a.shared;
    const int tasksSharedGU = a.shared ? (Fs + 3) / 4 : 0;
    const int tasksSharedDown = a.shared ? (D + 3) / 4 : 0;
    // requests first: shared gate/up rows (warps 0..3), router rows (warps 4..9), and already the
    // shared down rows of phase B (warps 10..15): none of them depends on the routing
    auto issue_shared_gu = [&](int t) {
        stage_matrix_rows(mySlot, imD, sh + a.sharedOff.gateWOff, sh + a.sharedOff.gateSOff,
                          sh + a.sharedOff.gateBOff, t * 4, Fs, D);
        stage_matrix_rows(mySlot + imD.bytes(), imD, sh + a.sharedOff.upWOff, sh + a.sharedOff.upSOff,
                          sh + a.sharedOff.upBOff, t * 4, Fs, D);
    };
    auto issue_shared_down = [&](int t) {
        stage_matrix_rows(mySlot, imFs, sh + a.sharedOff.downWOff, sh + a.sharedOff.downSOff,
                          sh + a.sharedOff.downBOff, t * 4, D, Fs);
    };
    int tA = warp < 4 ? warp * G + cta : 0x7FFFFFFF;
    if (tA < tasksSharedGU) issue_shared_gu(tA);
    int eA = (!a.idsIn && warp >= 4 && warp < kBigWarps) ? (warp - 4) * G + cta : 0x7FFFFFFF;
    if (eA < E) warp_copy16(mySlot, reinterpret_cast<const uint8_t *>(a.routerW + (size_t)eA * D), D * 2);
    int tSD = warp >= kBigWarps ? (warp - kBigWarps) * G + cta : 0x7FFFFFFF;
    if (tSD < tasksSharedDown) issue_shared_down(tSD);
    if (a.prefetch && a.shared) prefetch_region(a.shared, a.sharedBytes, cursor);
    warp_stamp(a, 0, 0);
    __syncthreads();
    uint32_t sense = sSense;
    {
        const uint32_t zero = 0;
        stage_rows(a.x, (uint32_t)D, &zero, 1, D, xs, xsum);
    }
    for (; tA < tasksSharedGU; tA += 4 * G) {
        cp_async_wait_all();
        __syncwarp();
        warp_stamp(a, 0, 1);
        const int row = tA * 4 + r4;
        const uint8_t *g0 = mySlot, *u0 = mySlot + imD.bytes();
        float g[1], u[1];
        row_dot<1, true, true>(g0, reinterpret_cast<const uint16_t *>(g0 + imD.wBytes),
                               reinterpret_cast<const uint16_t *>(g0 + imD.wBytes + imD.sBytes), u0,
                               reinterpret_cast<const uint16_t *>(u0 + imD.wBytes),
                               reinterpret_cast<const uint16_t *>(u0 + imD.wBytes + imD.sBytes), r4, D, row < Fs,
                               xs, xsum, kSelZero, g, u);
        if (row < Fs && j == 0) a.sharedActs[row] = f2bf(gelu_tanh(bf16_round(g[0])) * bf16_round(u[0]));
        __syncwarp();
        if (tA + 4 * G < tasksSharedGU) issue_shared_gu(tA + 4 * G);
    }
    for (; eA < E; eA += (kBigWarps - 4) * G) {
        cp_async_wait_all();
        __syncwarp();
        warp_stamp(a, 0, 1);
        const uint16_t *wr = reinterpret_cast<const uint16_t *>(mySlot);
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
        for (int offset = 16; offset >= 1; offset >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, offset);
        if (lane == 0) a.logits[eA] = a.logitBias ? acc + a.logitBias[eA] : acc;
        __syncwarp();
        const int next = eA + (kBigWarps - 4) * G;
        if (next < E) warp_copy16(mySlot, reinterpret_cast<const uint8_t *>(a.routerW + (size_t)next * D), D * 2);
    }
    warp_stamp(a, 0, 2);
    stamp(a, 1);
    if (!grid_barrier(a.barrier, sense, a.errorFlag, &sOk)) {
        cp_async_wait_all();
        return;
    }
    stamp(a, 2);

    // ---------------- phase B: top-8, routed gate/up/GeGLU, shared down ----------------
    if (!a.idsIn) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) sLogits[e] = a.logits[e];
        if (threadIdx.x < 8) {
            sIds[threadIdx.x] = 0u;
            sScore[threadIdx.x] = -INFINITY;
        }
        __syncthreads();
        // rank of every logit under (higher score, then lower expert id); scores of -inf or NaN
        // are never taken — the order of the serial top-8 (moe.metal:269-303).  Four threads per
        // expert, each counting a quarter of the competitors.
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
    const int perSlot = (F + 3) / 4;
    const int tasksRouted = K * perSlot;
    auto stage_routed = [&](int t) {
        const int slot = t / perSlot, row0 = (t - slot * perSlot) * 4;
        const uint8_t *blob = a.experts + (size_t)sIds[slot] * a.stride;
        stage_matrix_rows(mySlot, imD, blob + a.off.gateWOff, blob + a.off.gateSOff, blob + a.off.gateBOff,
                          row0, F, D);
        stage_matrix_rows(mySlot + imD.bytes(), imD, blob + a.off.upWOff, blob + a.off.upSOff,
                          blob + a.off.upBOff, row0, F, D);
    };
    int tB = warp < kBigWarps ? warp * G + cta : 0x7FFFFFFF;
    if (tB < tasksRouted) stage_routed(tB);
    warp_stamp(a, 1, 0);
    if (a.prefetch) {
        // the down projections of the chosen experts go to L2 now and are read in phase C
        for (int k = 0; k < K; ++k) {
            const uint8_t *blob = a.experts + (size_t)sIds[k] * a.stride;
            prefetch_region(blob + a.off.downWOff,
                            (uint64_t)a.off.downBOff - a.off.downWOff + (uint64_t)D * F / kGroup * 2, cursor);
        }
    }
    float *as = region;
    if (a.shared) {
        const uint32_t zero = 0;
        stage_rows(a.sharedActs, (uint32_t)Fs, &zero, 1, Fs, as, as + staged_stride(Fs));
    }
    for (; tB < tasksRouted; tB += kBigWarps * G) {
        cp_async_wait_all();
        __syncwarp();
        warp_stamp(a, 1, 1);
        const int slot = tB / perSlot;
        const int row = (tB - slot * perSlot) * 4 + r4;
        const uint8_t *g0 = mySlot, *u0 = mySlot + imD.bytes();
        float g[1], u[1];
        row_dot<1, true, true>(g0, reinterpret_cast<const uint16_t *>(g0 + imD.wBytes),
                               reinterpret_cast<const uint16_t *>(g0 + imD.wBytes + imD.sBytes), u0,
                               reinterpret_cast<const uint16_t *>(u0 + imD.wBytes),
                               reinterpret_cast<const uint16_t *>(u0 + imD.wBytes + imD.sBytes), r4, D, row < F,
                               xs, xsum, kSelZero, g, u);
        if (row < F && j == 0) a.acts[slot * F + row] = f2bf(gelu_tanh(g[0]) * u[0]);
        __syncwarp();
        if (tB + kBigWarps * G < tasksRouted) stage_routed(tB + kBigWarps * G);
    }
    for (; tSD < tasksSharedDown; tSD += (kFusedWarps - kBigWarps) * G) {
        cp_async_wait_all();
        __syncwarp();
        warp_stamp(a, 1, 1);
        const int row = tSD * 4 + r4;
        float v[1], unused[1];
        row_dot<1, false, true>(mySlot, reinterpret_cast<const uint16_t *>(mySlot + imFs.wBytes),
                                reinterpret_cast<const uint16_t *>(mySlot + imFs.wBytes + imFs.sBytes), nullptr,
                                nullptr, nullptr, r4, Fs, row < D, as, as + staged_stride(Fs), kSelZero, v, unused);
        if (row < D && j == 0) a.h1[row] = f2bf(v[0]);
        __syncwarp();
        const int next = tSD + (kFusedWarps - kBigWarps) * G;
        if (next < tasksSharedDown) issue_shared_down(next);
    }
    warp_stamp(a, 1, 2);
    stamp(a, 4);
    if (!grid_barrier(a.barrier, sense, a.errorFlag, &sOk)) {
        cp_async_wait_all();
        return;
    }
    stamp(a, 5);

    // ---------------- phase C: routed down rows and the combine ----------------
    {
        const int tasksDown = (D + 3) / 4;
        const int imgBytes = imF.bytes();
        auto stage_down = [&](int t) {
            for (int k = 0; k < K; ++k) {
                const uint8_t *blob = a.experts + (size_t)sIds[k] * a.stride;
                stage_matrix_rows(mySlot + (size_t)k * imgBytes, imF, blob + a.off.downWOff,
                                  blob + a.off.downSOff, blob + a.off.downBOff, t * 4, D, F);
            }
        };
        int tC = warp < kBigWarps ? warp * G + cta : 0x7FFFFFFF;
        if (tC < tasksDown) stage_down(tC);
        warp_stamp(a, 2, 0);
        const int strideF = staged_stride(F);
        float *asum = as + 8 * strideF;
        stage_rows(a.acts, (uint32_t)F, sRowIdx, K, F, as, asum);
        const uint16_t *res = a.shared ? a.h1 : a.residual;
        for (; tC < tasksDown; tC += kBigWarps * G) {
            cp_async_wait_all();
            __syncwarp();
            warp_stamp(a, 2, 1);
            const int row = tC * 4 + r4;
            const bool live = row < D;
            float acc = (live && res) ? bf2f(res[row]) : 0.0f;
#pragma unroll 1
            for (int k = 0; k < K; ++k) {
                const uint8_t *img = mySlot + (size_t)k * imgBytes;
                float v[1], unused[1];
                row_dot<1, false, true>(img, reinterpret_cast<const uint16_t *>(img + imF.wBytes),
                                        reinterpret_cast<const uint16_t *>(img + imF.wBytes + imF.sBytes),
                                        nullptr, nullptr, nullptr, r4, F, live, as + k * strideF,
                                        asum + k * (F >> 5), kSelZero, v, unused);
                acc = __fadd_rn(acc, __fmul_rn(sWeights[k], v[0]));
            }
            if (live && j == 0) a.y[row] = f2bf(acc);
            __syncwarp();
            if (tC + kBigWarps * G < tasksDown) stage_down(tC + kBigWarps * G);
        }
    }
    warp_stamp(a, 2, 2);
    stamp(a, 6);
}

struct FusedLayout {
    size_t slotsOffset, bigBytes, smallBytes, total;
};

static FusedLayout fused_layout(const FFConfig &c) {
    const size_t xPart = ((size_t)staged_stride((int)c.d) + (c.d >> 5)) * sizeof(float);
    const size_t sharedPart =
        c.sharedF ? ((size_t)staged_stride((int)c.sharedF) + (c.sharedF >> 5)) * sizeof(float) : 0;
    const size_t actsPart = (size_t)8 * (staged_stride((int)c.f) + (c.f >> 5)) * sizeof(float);
    FusedLayout l{};
    l.slotsOffset = (xPart + std::max(sharedPart, actsPart) + 127) & ~(size_t)127;
    const size_t gateUp = 2 * (size_t)rows_image((int)c.d).bytes();
    const size_t down8 = 8 * (size_t)rows_image((int)c.f).bytes();
    l.bigBytes = (std::max({gateUp, down8, (size_t)c.d * 2}) + 127) & ~(size_t)127;
    l.smallBytes = c.sharedF ? (((size_t)rows_image((int)c.sharedF).bytes() + 127) & ~(size_t)127) : 128;
    l.total = l.slotsOffset + kBigWarps * l.bigBytes + (kFusedWarps - kBigWarps) * l.smallBytes;
    return l;
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
    const FusedLayout lay = fused_layout(c);
    const size_t smem = lay.total;
    if (smem > 227 * 1024)
        return fail(error, "model shape too large for the fused decode kernel's shared memory");
    // the asynchronous 8-byte copies need 8-byte aligned scale/bias runs
    const uint32_t *ro = &L.off.gateWOff, *so = &L.sharedOff.gateWOff;
    for (int i = 0; i < 9; ++i)
        if (ro[i] % 8 || (withShared && so[i] % 8) || L.stride % 8)
            return fail(error, "sub-tensor offsets must be multiples of 8 bytes for the decode kernel");
    a.slotsOffset = (uint32_t)lay.slotsOffset;
    a.bigBytes = (uint32_t)lay.bigBytes;
    a.smallBytes = (uint32_t)lay.smallBytes;
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
