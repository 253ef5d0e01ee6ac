// Device functions shared by the GEMV kernels: bf16 helpers, the GeGLU activation, input staging
// and the one-weight-row dot product every 1..16-row kernel is built from.
#pragma once

#include "ff_internal.cuh"

namespace ff {

constexpr int kGemvThreads = 256;
constexpr int kRowsPerItem = (kGemvThreads / 32) * 4;
constexpr int kDecodeDownRows = 8;  // output rows per CTA of the decode combine kernel

__device__ __forceinline__ float bf2f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// Round-half-even on the dropped 16 bits: Quantization.bf16Bits
// (Sources/ANEFieldfareHotpath/Infrastructure/ModelIO/Quantization.swift:9-16).
__device__ __forceinline__ uint16_t f2bf(float f) {
    uint32_t u = __float_as_uint(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float bf16_round(float f) { return bf2f(f2bf(f)); }

// gelu_pytorch_tanh with the kernels' clamp (Metal/MoE/moe.metal:40-47).
__device__ __forceinline__ float gelu_tanh(float x) {
    const float x3 = x * x * x;
    float inner = 0.7978845608028654f * (x + 0.044715f * x3);
    inner = fminf(fmaxf(inner, -20.0f), 20.0f);
    return 0.5f * x * (1.0f + tanhf(inner));
}

// The same activation with the hardware's tanh approximation (relative error about 2^-11, below
// the bf16 rounding that follows it): for the prefill GEMM's epilogue, where the exact tanhf is a
// measurable share of the step.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    const float x3 = x * x * x;
    float inner = 0.7978845608028654f * (x + 0.044715f * x3);
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(inner));
    return 0.5f * x * (1.0f + th);
}

// Position of input element e inside a staged row: chunks are interleaved in blocks of eight so
// that lanes j = 0..7 (chunks c = 8i + j) read one contiguous 128 bytes per 128-bit load.
__device__ __forceinline__ int staged_index(int e) {
    const int c = e >> 5;
    return ((c >> 3) << 8) + (((e >> 2) & 7) << 5) + ((c & 7) << 2) + (e & 3);
}
__host__ __device__ inline int staged_stride(int cols) { return (cols + 255) & ~255; }

// Eight codes of one 32-bit word as the floats 16+q: the code goes into the top mantissa bits of
// a float whose exponent is 2^4 (bits 0x41800000 | q << 19).  The surplus 16*sum(x) is taken out
// once per chunk through the bias term, so no per-code subtraction is needed.
// Twelve integer instructions for eight codes, written as PTX so the count is what runs: the even
// codes (low nibbles) and the odd codes (high nibbles) are each moved to bits 3..6 of their byte
// and given bit 7 (two shifts, two lop3), then one byte permute per code drops that byte into
// byte 2 of the float and 0x41 into byte 3.
__device__ __forceinline__ void unpack8_plus16(uint32_t w, float (&q)[8]) {
    uint32_t even, odd, sl, sr;
    asm("shl.b32 %0, %1, 3;" : "=r"(sl) : "r"(w));
    asm("shr.b32 %0, %1, 1;" : "=r"(sr) : "r"(w));
    // (a & b) | c  ->  lop3 immLut 0xEA
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(even) : "r"(sl), "r"(0x78787878u), "r"(0x80808080u));
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(odd) : "r"(sr), "r"(0x78787878u), "r"(0x80808080u));
    const uint32_t hi = 0x41000000u;
    uint32_t r0, r1, r2, r3, r4, r5, r6, r7;
    asm("prmt.b32 %0, %1, %2, 0x7044;" : "=r"(r0) : "r"(even), "r"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7044;" : "=r"(r1) : "r"(odd), "r"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7144;" : "=r"(r2) : "r"(even), "r"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7144;" : "=r"(r3) : "r"(odd), "r"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7244;" : "=r"(r4) : "r"(even), "r"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7244;" : "=r"(r5) : "r"(odd), "r"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7344;" : "=r"(r6) : "r"(even), "r"(hi));
    asm("prmt.b32 %0, %1, %2, 0x7344;" : "=r"(r7) : "r"(odd), "r"(hi));
    q[0] = __uint_as_float(r0);
    q[1] = __uint_as_float(r1);
    q[2] = __uint_as_float(r2);
    q[3] = __uint_as_float(r3);
    q[4] = __uint_as_float(r4);
    q[5] = __uint_as_float(r5);
    q[6] = __uint_as_float(r6);
    q[7] = __uint_as_float(r7);
}

// Packed fp32 pairs for fma.rn.f32x2 (low half = first value).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ float pair_sum(uint64_t v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return lo + hi;
}

__device__ __forceinline__ uint4 load_stream(const uint4 *p) { return __ldcs(p); }

// Stages n bf16 input rows (indices rowIdx[0..n)) as fp32 in chunk-interleaved order, then the
// per-chunk sums of each row.  All threads of the CTA take part.
__device__ inline void stage_rows(const uint16_t *in, uint32_t inStride, const uint32_t *rowIdx, int n,
                           int cols, float *xs, float *xsum) {
    const int stride = staged_stride(cols);
    const int chunks = cols >> 5;
    const int pairsPerRow = cols >> 1;
    for (int i = threadIdx.x; i < n * pairsPerRow; i += blockDim.x) {
        const int r = i / pairsPerRow, p = i - r * pairsPerRow;
        const uint32_t two =
            *reinterpret_cast<const uint32_t *>(in + (size_t)rowIdx[r] * inStride + 2 * p);
        float *dst = xs + r * stride + staged_index(2 * p);
        dst[0] = __uint_as_float(two << 16);
        dst[1] = __uint_as_float(two & 0xFFFF0000u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n * chunks; i += blockDim.x) {
        const int r = i / chunks, c = i - r * chunks;
        const float *src = xs + r * stride + ((c >> 3) << 8) + ((c & 7) << 2);
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float4 v = *reinterpret_cast<const float4 *>(src + (k << 5));
            s += v.x;
            s += v.y;
            s += v.z;
            s += v.w;
        }
        xsum[r * chunks + c] = s;
    }
    __syncthreads();
}

// One 16-byte chunk (32 codes) of a weight row (or of a gate/up row pair) against NT staged input
// rows: acc = fma(scale, sum(q*x), acc); acc = fma(bias - 16*scale, sum(x), acc).  `sb` packs the
// group's scale (low 16 bits) and bias (high 16 bits) as bf16.  Every kernel that multiplies an
// INT4 row by 1..16 input rows goes through this function, in chunk-ascending order per lane.
// sel[t] is the staged row that input t reads.
template <int NT, bool DUAL>
__device__ __forceinline__ void chunk_accumulate(const uint4 &v0, const uint4 &v1, uint32_t sb0v,
                                                 uint32_t sb1v, int c, const float *xs, const float *xsum,
                                                 int stride, int chunks, const int (&sel)[NT],
                                                 float (&a0)[NT], float (&a1)[NT]) {
    const float sc0 = __uint_as_float(sb0v << 16);
    const float bi0 = fmaf(-16.0f, sc0, __uint_as_float(sb0v & 0xFFFF0000u));
    float sc1 = 0.0f, bi1 = 0.0f;
    if (DUAL) {
        sc1 = __uint_as_float(sb1v << 16);
        bi1 = fmaf(-16.0f, sc1, __uint_as_float(sb1v & 0xFFFF0000u));
    }
    // Two running sums per (matrix, input row), held as one packed fp32 pair and advanced by
    // packed fused multiply-adds (fma.rn.f32x2: two fp32 FMAs per instruction): the even codes of
    // the chunk accumulate in the low half, the odd codes in the high half; the halves are added
    // once per chunk.
    uint64_t d0[NT], d1[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        d0[t] = 0ull;
        d1[t] = 0ull;
    }
    const float *xc = xs + ((c >> 3) << 8) + ((c & 7) << 2);
    const uint32_t words0[4] = {v0.x, v0.y, v0.z, v0.w};
    const uint32_t words1[4] = {v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float q0[8], q1[8];
        unpack8_plus16(words0[k], q0);
        if (DUAL) unpack8_plus16(words1[k], q1);
        uint64_t p0[4], p1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            p0[i] = pack2(q0[2 * i], q0[2 * i + 1]);
            if (DUAL) p1[i] = pack2(q1[2 * i], q1[2 * i + 1]);
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float *xt = xc + sel[t] * stride + (k << 6);
            const float4 xa = *reinterpret_cast<const float4 *>(xt);
            const float4 xb = *reinterpret_cast<const float4 *>(xt + 32);
            const uint64_t x01 = pack2(xa.x, xa.y), x23 = pack2(xa.z, xa.w);
            const uint64_t x45 = pack2(xb.x, xb.y), x67 = pack2(xb.z, xb.w);
            uint64_t acc = d0[t];
            acc = fma2(p0[0], x01, acc);
            acc = fma2(p0[1], x23, acc);
            acc = fma2(p0[2], x45, acc);
            acc = fma2(p0[3], x67, acc);
            d0[t] = acc;
            if (DUAL) {
                uint64_t acu = d1[t];
                acu = fma2(p1[0], x01, acu);
                acu = fma2(p1[1], x23, acu);
                acu = fma2(p1[2], x45, acu);
                acu = fma2(p1[3], x67, acu);
                d1[t] = acu;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const float sx = xsum[sel[t] * chunks + c];
        a0[t] = fmaf(sc0, pair_sum(d0[t]), a0[t]);
        a0[t] = fmaf(bi0, sx, a0[t]);
        if (DUAL) {
            a1[t] = fmaf(sc1, pair_sum(d1[t]), a1[t]);
            a1[t] = fmaf(bi1, sx, a1[t]);
        }
    }
}

// One weight row (or a gate/up row pair) against NT staged input rows; returns the full sums in
// every lane of the row's eight-lane group.  SMEM: the weight pointers address a copy of the rows
// in shared memory (plain loads) instead of global memory (streaming loads).  `live` false skips the loads but keeps the
// shuffles convergent.
template <int NT, bool DUAL, bool SMEM = false>
__device__ __forceinline__ void row_dot(const uint8_t *w0, const uint16_t *s0, const uint16_t *b0,
                                        const uint8_t *w1, const uint16_t *s1, const uint16_t *b1,
                                        int row, int cols, bool live, const float *xs,
                                        const float *xsum, const int (&sel)[NT], float (&a0)[NT],
                                        float (&a1)[NT]) {
    const int lane = threadIdx.x & 31;
    const int j = lane & 7;
    const int chunks = cols >> 5;
    const int groups = cols >> 6;
    const int stride = staged_stride(cols);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        a0[t] = 0.0f;
        a1[t] = 0.0f;
    }
    if (live) {
        const uint4 *p0 = reinterpret_cast<const uint4 *>(w0 + (size_t)row * (cols >> 1));
        const uint4 *p1 = DUAL ? reinterpret_cast<const uint4 *>(w1 + (size_t)row * (cols >> 1)) : p0;
        const uint16_t *sr0 = s0 + (size_t)row * groups, *br0 = b0 + (size_t)row * groups;
        const uint16_t *sr1 = DUAL ? s1 + (size_t)row * groups : sr0;
        const uint16_t *br1 = DUAL ? b1 + (size_t)row * groups : br0;
        // Software pipeline in a rolled loop: the 128-bit loads (and scales) of the next kDepth
        // chunks are in flight while one chunk is unpacked and accumulated.  The loop body stays
        // small enough for the instruction cache; the accumulation order (chunks ascending) does
        // not depend on kDepth.
        constexpr int kDepth = NT <= 2 ? 3 : 2;
        uint4 v0b[kDepth], v1b[kDepth];
        uint32_t sb0[kDepth], sb1[kDepth];  // scale | bias << 16
        auto fetch = [&](int c, int slot) {
            v0b[slot] = SMEM ? p0[c] : load_stream(p0 + c);
            sb0[slot] = (uint32_t)sr0[c >> 1] | ((uint32_t)br0[c >> 1] << 16);
            if (DUAL) {
                v1b[slot] = SMEM ? p1[c] : load_stream(p1 + c);
                sb1[slot] = (uint32_t)sr1[c >> 1] | ((uint32_t)br1[c >> 1] << 16);
            }
        };
#pragma unroll
        for (int u = 0; u < kDepth; ++u)
            if (j + 8 * u < chunks) fetch(j + 8 * u, u);
#pragma unroll 1
        for (int c0 = j; c0 < chunks; c0 += 8 * kDepth) {
#pragma unroll
            for (int u = 0; u < kDepth; ++u) {
                const int c = c0 + 8 * u;
                if (c < chunks) {
                    const uint4 v0 = v0b[u];
                    const uint4 v1 = DUAL ? v1b[u] : v0b[u];
                    const uint32_t p0sb = sb0[u], p1sb = DUAL ? sb1[u] : 0u;
                    if (c + 8 * kDepth < chunks) fetch(c + 8 * kDepth, u);
                    chunk_accumulate<NT, DUAL>(v0, v1, p0sb, p1sb, c, xs, xsum, stride, chunks, sel, a0, a1);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
#pragma unroll
        for (int offset = 4; offset >= 1; offset >>= 1) {
            a0[t] += __shfl_xor_sync(0xFFFFFFFFu, a0[t], offset);
            if (DUAL) a1[t] += __shfl_xor_sync(0xFFFFFFFFu, a1[t], offset);
        }
    }
}

// Warp-wide top-K over E <= 256 logits held four-plus per lane: K rounds of argmax (higher score,
// then lower expert id), softmax over the selected scores, times the per-expert gain.  Selection
// rule and softmax: Metal/MoE/moe.metal:186-237,269-319.
// sharedIds: optional copy of the ids in shared memory.
__device__ inline void warp_topk(const float *logits, int E, int K, const uint16_t *gain, uint32_t *ids,
                          uint16_t *weights, uint32_t *sharedIds = nullptr) {
    const int lane = threadIdx.x & 31;
    float v[8];
    uint32_t live = 0;  // bit j: candidate j of this lane is still in the race (a register, not an indexed array)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int e = j * 32 + lane;
        v[j] = e < E ? logits[e] : -INFINITY;
        if (e < E && v[j] > -INFINITY) live |= 1u << j;
    }
    float topScore[8];
    uint32_t topIdx[8];
    for (int r = 0; r < 8; ++r) {
        float best = -INFINITY;
        uint32_t bestE = 0xFFFFFFFFu;
        if (r < K) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t e = (uint32_t)(j * 32 + lane);
                if (((live >> j) & 1u) && (v[j] > best || (v[j] == best && e < bestE))) {
                    best = v[j];
                    bestE = e;
                }
            }
        }
#pragma unroll
        for (int offset = 16; offset >= 1; offset >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, offset);
            const uint32_t oe = __shfl_xor_sync(0xFFFFFFFFu, bestE, offset);
            if (oe != 0xFFFFFFFFu && (bestE == 0xFFFFFFFFu || ob > best || (ob == best && oe < bestE))) {
                best = ob;
                bestE = oe;
            }
        }
        if (bestE != 0xFFFFFFFFu && (bestE & 31u) == (uint32_t)lane) live &= ~(1u << (bestE >> 5));
        topIdx[r] = bestE == 0xFFFFFFFFu ? 0u : bestE;
        topScore[r] = bestE == 0xFFFFFFFFu ? -INFINITY : best;
    }
    // softmax over the chosen scores: lane r holds route r; exponentials in parallel, the sum in
    // rank order (the same additions as a serial loop)
    float myScore = -INFINITY;
    uint32_t myIdx = 0;
#pragma unroll
    for (int r = 0; r < 8; ++r)
        if (lane == r) {
            myScore = topScore[r];
            myIdx = topIdx[r];
        }
    const float ex = lane < K ? expf(myScore - topScore[0]) : 0.0f;
    float sum = 0.0f;
    for (int r = 0; r < K; ++r) sum += __shfl_sync(0xFFFFFFFFu, ex, r);
    if (lane < K) {
        float w = ex / sum;
        if (gain) w = w * bf2f(gain[myIdx]);
        ids[lane] = myIdx;
        weights[lane] = f2bf(w);
        if (sharedIds) sharedIds[lane] = myIdx;
    }
}

}  // namespace ff
