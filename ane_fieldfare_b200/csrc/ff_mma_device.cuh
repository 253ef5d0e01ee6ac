// Device helpers shared by the kernels that multiply packed INT4 rows on the tensor cores without
// dequantizing them (the one-token decode kernel and the 2..16-row block kernels): bulk copies into
// a warp's shared-memory slot with completion on the warp's mbarrier, the code -> bf16 conversion,
// the m16n8k16 MMA over groups of 64 codes, and the staging of bf16 input rows.
#pragma once

#include "ff_gemv_device.cuh"
#include "ff_internal.cuh"

namespace ff {

constexpr uint32_t kCopySpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t sm_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- bulk copies into a warp's slot, completion on the warp's mbarrier -------------------------

__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint32_t bar, uint32_t parity) {
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
// 16-byte aligned source and destination, size a multiple of 16.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Called by the whole warp when it has used its slot's contents, before the next copies into the
// slot are requested.  The values read from the slot have been consumed by then (the arithmetic
// depends on them), so the reads are complete; the warp barrier orders every lane's reads before
// the requesting lane's next copy — the consumer-release / producer-acquire hand-off of a copy
// pipeline, with the warp barrier in place of the "empty" mbarrier.  (A proxy fence here would also
// wait for the warp's outstanding L2 prefetches.)
__device__ __forceinline__ void slot_release() { __syncwarp(); }
// Bounded wait for the warp's copies; flips the parity.  On running out the error flag is raised
// and the warp carries on (its rows are then wrong, the launch still ends).
static __device__ __noinline__ bool slot_wait_slow(uint32_t bar, uint32_t parity) {
    bool done = false;
    for (uint32_t i = 0; i < kCopySpinLimit && !done; ++i) done = bar_try_wait(bar, parity);
    return done;
}
// (The first poll stands alone: a poll inside the bounded loop measured about 200 cycles on a
// barrier that was already complete, a stand-alone one 7.)
__device__ __forceinline__ void slot_wait(uint32_t bar, uint32_t &parity, uint32_t *errorFlag) {
    bool done = bar_try_wait(bar, parity);
    if (!done) done = slot_wait_slow(bar, parity);
    if (!done && (threadIdx.x & 31) == 0) atomicExch(errorFlag, 10u);
    parity ^= 1u;
    __syncwarp();
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- tensor-core row arithmetic on packed codes ------------------------------------------------

// Codes i and i+4 of a word (already shifted so that they sit at bits 3..6 of each half) as the
// bf16 pair (16+q_i, 16+q_{i+4}): (s & 0x00780078) | 0x41804180.
__device__ __forceinline__ uint32_t code_pair(uint32_t shifted) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(shifted), "r"(0x00780078u), "r"(0x41804180u));
    return r;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// N consecutive groups of 64 codes of a 16-row tile against the (up to eight) input columns.
//   lo / hi: this thread's eight packed bytes of tile rows g and g+8 (g = lane / 4) for the first
//            group: bytes [8 t, 8 t + 8) of the group's 32, t = lane % 4; next group 32 bytes on;
//   xg:      this thread's 32 bytes of input column lane / 4: elements [16 t, 16 t + 16) of the
//            group, every aligned run of eight stored in the order 0,4,1,5,2,6,3,7; next group 128
//            bytes on.
// Word j of the eight bytes feeds MMAs 2j and 2j+1; MMA 2j+h multiplies codes (2h, 2h+4 | 2h+1,
// 2h+5) of the word with input register pair h of the run — the same elements, whatever position
// the MMA gives them.  d[u]: group u's sums for rows g (d[u][0], d[u][1]) and g+8 (d[u][2],
// d[u][3]), columns 2t and 2t+1.  The N accumulator chains are independent, so their MMAs overlap.
template <int N>
__device__ __forceinline__ void groups_mma(const uint8_t *lo, const uint8_t *hi, const uint8_t *xg, float (&d)[N][4]) {
    uint2 wl[N], wh[N];
    uint4 x0[N], x1[N];
#pragma unroll
    for (int u = 0; u < N; ++u) {
        wl[u] = *reinterpret_cast<const uint2 *>(lo + 32 * u);
        wh[u] = *reinterpret_cast<const uint2 *>(hi + 32 * u);
        x0[u] = *reinterpret_cast<const uint4 *>(xg + 128 * u);
        x1[u] = *reinterpret_cast<const uint4 *>(xg + 128 * u + 16);
        d[u][0] = d[u][1] = d[u][2] = d[u][3] = 0.0f;
    }
#pragma unroll
    for (int u = 0; u < N; ++u)
        mma_16816(d[u], code_pair(wl[u].x << 3), code_pair(wh[u].x << 3), code_pair(wl[u].x >> 1),
                  code_pair(wh[u].x >> 1), x0[u].x, x0[u].y);
#pragma unroll
    for (int u = 0; u < N; ++u)
        mma_16816(d[u], code_pair(wl[u].x >> 5), code_pair(wh[u].x >> 5), code_pair(wl[u].x >> 9),
                  code_pair(wh[u].x >> 9), x0[u].z, x0[u].w);
#pragma unroll
    for (int u = 0; u < N; ++u)
        mma_16816(d[u], code_pair(wl[u].y << 3), code_pair(wh[u].y << 3), code_pair(wl[u].y >> 1),
                  code_pair(wh[u].y >> 1), x1[u].x, x1[u].y);
#pragma unroll
    for (int u = 0; u < N; ++u)
        mma_16816(d[u], code_pair(wl[u].y >> 5), code_pair(wh[u].y >> 5), code_pair(wl[u].y >> 9),
                  code_pair(wh[u].y >> 9), x1[u].z, x1[u].w);
}

// acc += scale * sum((16+q) x) + (bias - 16 scale) * sum(x)
__device__ __forceinline__ float group_scale(float acc, uint16_t scale, uint16_t bias, float dsum, float xsum) {
    const float s = bf2f(scale);
    acc = fmaf(s, dsum, acc);
    return fmaf(fmaf(-16.0f, s, bf2f(bias)), xsum, acc);
}

// Run `i` (eight bf16 values `v`) of a staged input: stored in the order 0,4,1,5,2,6,3,7 at row
// i / runsPerRow, and its values summed into the group's fp32 sum by a fixed butterfly over the
// eight adjacent lanes that hold the group's runs.  Called by whole warps.
__device__ __forceinline__ void stage_put(int i, bool valid, const uint4 &v, int runsPerRow, uint8_t *dst,
                                          uint32_t dstStride, float *sums) {
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    float s = 0.0f;
    if (valid) {
        const int r = i / runsPerRow;
        *reinterpret_cast<uint4 *>(dst + (size_t)r * dstStride + (size_t)(i - r * runsPerRow) * 16) = o;
        s = __uint_as_float(o.x << 16);
        s += __uint_as_float(o.x & 0xFFFF0000u);
        s += __uint_as_float(o.y << 16);
        s += __uint_as_float(o.y & 0xFFFF0000u);
        s += __uint_as_float(o.z << 16);
        s += __uint_as_float(o.z & 0xFFFF0000u);
        s += __uint_as_float(o.w << 16);
        s += __uint_as_float(o.w & 0xFFFF0000u);
    }
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
    if (valid && (i & 7) == 0) sums[i >> 3] = s;
}

// Copies `rows` bf16 rows of `n` values (n a multiple of 64, rows contiguous at the source,
// `dstStride` bytes apart in shared memory) with every aligned run of eight stored in the order
// 0,4,1,5,2,6,3,7, then the fp32 sum of each group of 64 (sums[row * n/64 + group]).  All threads
// of the CTA take part; ends with a CTA barrier.
// `first`: the run with index threadIdx.x, already loaded by the caller (or null).  `srcStride`:
// elements between source rows (0: the rows are contiguous).
__device__ __forceinline__ void stage_input(const uint16_t *src, int rows, int n, uint8_t *dst, uint32_t dstStride,
                                            float *sums, bool plainLoads = false, const uint4 *first = nullptr,
                                            uint32_t srcStride = 0) {
    const int runsPerRow = n >> 3, runs = rows * runsPerRow;
    const uint32_t rowRuns = srcStride ? srcStride >> 3 : (uint32_t)runsPerRow;  // 16-byte units between source rows
    // Two runs per thread and step, both loads issued before either is used.  A run's eight values
    // are summed while they are in registers (in stored order), the eight runs of a group sit in
    // eight adjacent lanes and are added by a fixed butterfly: one pass, one CTA barrier.  The loop
    // bound is the same for all lanes of a warp.
    auto fetch = [&](int i) {
        const int sr = i / runsPerRow;
        const size_t si = (size_t)sr * rowRuns + (size_t)(i - sr * runsPerRow);
        // plain loads for a source outside global memory (kernel parameters)
        return (first && i == (int)threadIdx.x) ? *first
               : plainLoads                      ? reinterpret_cast<const uint4 *>(src)[si]
                                                 : __ldcg(reinterpret_cast<const uint4 *>(src) + si);
    };
    auto put = [&](int i, bool valid, const uint4 &v) { stage_put(i, valid, v, runsPerRow, dst, dstStride, sums); };
    for (int base = (threadIdx.x >> 5) << 5; base < runs; base += 2 * blockDim.x) {
        const int i = base + (threadIdx.x & 31), j = i + blockDim.x;
        const bool vi = i < runs, vj = j < runs;
        uint4 v0 = make_uint4(0, 0, 0, 0), v1 = make_uint4(0, 0, 0, 0);
        if (vi) v0 = fetch(i);
        if (vj) v1 = fetch(j);
        put(i, vi, v0);
        if (base + (int)blockDim.x < runs) put(j, vj, v1);  // warp-uniform condition
    }
    __syncthreads();
}

__host__ __device__ inline uint32_t pad16u(uint32_t bytes) { return (bytes + 15u) & ~15u; }
// Row-piece stride in a slot: at least `bytes`, a multiple of 16, and 32 or 96 modulo 128 so that
// the four tile rows a half-warp reads with 64-bit loads fall into different bank octets.
__host__ __device__ inline uint32_t piece_stride(uint32_t bytes) {
    uint32_t s = pad16u(bytes);
    while ((s & 127u) != 32u && (s & 127u) != 96u) s += 16u;
    return s;
}
// Groups [begin, end) of part p when `groups` are split into `parts` runs of (almost) equal length.
__host__ __device__ inline void part_range(int groups, int parts, int p, int &begin, int &end) {
    const int per = (groups + parts - 1) / parts;
    begin = min(groups, p * per);
    end = min(groups, begin + per);
}

}  // namespace ff
