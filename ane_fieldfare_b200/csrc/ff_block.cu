// INT4 matrices against 2..16 input rows (a verify block): gate/up + GeGLU jobs and down jobs of
// the routed experts a block touches and of the shared FFN, on the tensor cores without
// dequantizing (see ff_mma_device.cuh), replacing the per-row GEMV kernels for these sizes.
//
// A job (GemvJob, built on the device by the route plan) is one matrix (or a gate/up pair) and the
// 1..16 input rows that use it.  A warp task is one tile of the job's weight rows (8 gate + 8 up
// rows, or 16 down rows) against up to eight of the job's input rows — the eight columns of
// mma.sync m16n8k16; a job with more than eight rows yields two tasks per tile.  A task walks its
// K range in parts: the part's packed rows (and, once, the tile's scales and biases) come in as
// bulk asynchronous copies into the warp's shared-memory slot, then every group of 64 codes is
// multiplied as bf16(16+q) and scaled (acc += s * sum((16+q) x) + (b - 16 s) * sum(x)).  All parts
// of a task accumulate in the same registers, so no partial sums cross warps and results do not
// depend on scheduling.  Persistent CTAs of 16 (gate/up) or 10 (down) warps deal tasks round robin;
// the slots of an SM keep 100 KB and more of weights in flight.
//
// Gate/up jobs read the block's input rows, staged once per CTA as bf16 with every aligned run of
// eight in the order 0,4,1,5,2,6,3,7 (the order the MMA operands use), with their per-group sums.
// Their GeGLU outputs are written in the same run order, so a down task can copy its input pieces
// straight into its slot; the group sums of those inputs come from one extra MMA per K slice
// against all-ones rows.
//
// Reference kernels replaced (paths inside the reference project):
//   Sources/ANEFieldfareHotpath/Metal/Prefill/prefill.metal:1246-1529 (verify grouped GEMV)
//   Sources/ANEFieldfareHotpath/Metal/Quant/dequant_int4.metal:230-459 (multi-row INT4 GEMV)
#include <algorithm>

#include "ff_mma_device.cuh"

namespace ff {

// warps (= slots) per CTA: the gate/up kernel shares its shared memory with the staged input rows
// and takes short K parts in many slots; the down kernel's slots also hold the input pieces
constexpr int kGateUpWarps = 16;
constexpr int kDownWarps = 10;
constexpr int kMaxBlockJobs = kMaxExperts + 1;

struct BlockArgs {
    const GemvJob *jobs;
    const uint32_t *jobCountPtr;
    const uint16_t *allIn;  // gate/up: the block's input rows
    uint32_t allStride, allRows, cols;
    uint32_t maxPartGroups;  // groups of 64 per K part
    uint32_t xPitch;         // gate/up: bytes between staged input rows in shared memory
    uint32_t pieceStride;    // bytes between the 16 row pieces of a slot
    uint32_t scaleArea;      // bytes of one scale (or bias) run in a slot
    uint32_t inputPitch;     // down: bytes between a slot's input pieces
    uint32_t slotBytes, slotsOffset;
    uint32_t *errorFlag;
};

// N consecutive groups: as groups_mma, plus (ONES) the sums of the inputs themselves from MMAs
// against rows of ones: ones[u][0], ones[u][1] = sum over group u of input columns 2t, 2t+1.
template <int N, bool ONES>
__device__ __forceinline__ void groups_mma_cols(const uint8_t *lo, const uint8_t *hi, const uint8_t *xg,
                                                float (&d)[N][4], float (&ones)[N][4]) {
    groups_mma<N>(lo, hi, xg, d);
    if (ONES) {
        constexpr uint32_t kOne2 = 0x3F803F80u;  // bf16 (1.0, 1.0)
#pragma unroll
        for (int u = 0; u < N; ++u) {
            const uint4 x0 = *reinterpret_cast<const uint4 *>(xg + 128 * u);
            const uint4 x1 = *reinterpret_cast<const uint4 *>(xg + 128 * u + 16);
            ones[u][0] = ones[u][1] = ones[u][2] = ones[u][3] = 0.0f;
            mma_16816(ones[u], kOne2, kOne2, kOne2, kOne2, x0.x, x0.y);
            mma_16816(ones[u], kOne2, kOne2, kOne2, kOne2, x0.z, x0.w);
            mma_16816(ones[u], kOne2, kOne2, kOne2, kOne2, x1.x, x1.y);
            mma_16816(ones[u], kOne2, kOne2, kOne2, kOne2, x1.z, x1.w);
        }
    }
}

// `n` consecutive groups of a 16-row tile against two input columns per thread: acc[0], acc[1] =
// tile row g, columns 2t and 2t+1; acc[2], acc[3] = tile row g+8.  s0/b0, s1/b1: the two rows'
// scales and biases; xs0/xs1: the two columns' group sums (ignored with ONES).  Groups are taken
// in ascending order whatever the batching.
template <bool ONES>
__device__ __noinline__ void tile_rows_cols(const uint8_t *lo, const uint8_t *hi, const uint8_t *xg,
                                            const uint16_t *s0, const uint16_t *b0, const uint16_t *s1,
                                            const uint16_t *b1, const float *xs0, const float *xs1, int n,
                                            float (&acc)[4]) {
    float v[4] = {acc[0], acc[1], acc[2], acc[3]};
    auto apply = [&](const float (&d)[4], const float (&o)[4], int i) {
        const float x0 = ONES ? o[0] : xs0[i], x1 = ONES ? o[1] : xs1[i];
        v[0] = group_scale(v[0], s0[i], b0[i], d[0], x0);
        v[1] = group_scale(v[1], s0[i], b0[i], d[1], x1);
        v[2] = group_scale(v[2], s1[i], b1[i], d[2], x0);
        v[3] = group_scale(v[3], s1[i], b1[i], d[3], x1);
    };
    int i = 0;
#pragma unroll 1
    for (; i + 2 <= n; i += 2) {
        float d[2][4], o[2][4];
        groups_mma_cols<2, ONES>(lo + 32 * i, hi + 32 * i, xg + 128 * i, d, o);
        apply(d[0], o[0], i);
        apply(d[1], o[1], i + 1);
    }
    if (i < n) {
        float d[1][4], o[1][4];
        groups_mma_cols<1, ONES>(lo + 32 * i, hi + 32 * i, xg + 128 * i, d, o);
        apply(d[0], o[0], i);
    }
    acc[0] = v[0];
    acc[1] = v[1];
    acc[2] = v[2];
    acc[3] = v[3];
}

template <bool DUAL>
__global__ void __launch_bounds__((DUAL ? kGateUpWarps : kDownWarps) * 32, 1) k_block_mma(const BlockArgs a) {
    constexpr int kBlockWarps = DUAL ? kGateUpWarps : kDownWarps;
    extern __shared__ __align__(128) uint8_t smemRaw[];
    __shared__ uint32_t sPrefix[kMaxBlockJobs + 1];
    __shared__ __align__(8) uint64_t sCopyBar[kBlockWarps];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t nJobs = min(*a.jobCountPtr, (uint32_t)kMaxBlockJobs);
    uint8_t *mySlot = smemRaw + a.slotsOffset + (size_t)warp * a.slotBytes;
    const uint32_t slotAddr = sm_addr(mySlot);
    const uint32_t myBar = sm_addr(&sCopyBar[warp]);
    uint32_t parity = 0;

    if (threadIdx.x == 0) {
        for (int w = 0; w < kBlockWarps; ++w) bar_init(sm_addr(&sCopyBar[w]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // tasks per job: tiles x column halves; prefix sums by one thread (at most 257 jobs)
    for (uint32_t j = threadIdx.x; j < nJobs; j += blockDim.x) {
        const uint32_t tiles = DUAL ? a.jobs[j].rows >> 3 : a.jobs[j].rows >> 4;
        sPrefix[j + 1] = tiles * ((a.jobs[j].n + 7u) >> 3);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        sPrefix[0] = 0;
        for (uint32_t j = 0; j < nJobs; ++j) sPrefix[j + 1] += sPrefix[j];
    }
    __syncthreads();
    uint8_t *xAll = smemRaw;
    float *xSumAll = reinterpret_cast<float *>(smemRaw + (size_t)a.allRows * a.xPitch);
    const int groupsIn = (int)(a.cols >> 6);
    if (DUAL) stage_input(a.allIn, (int)a.allRows, (int)a.cols, xAll, a.xPitch, xSumAll, false, nullptr, a.allStride);
    const uint32_t total = sPrefix[nJobs];

    for (uint32_t task = (uint32_t)warp * gridDim.x + blockIdx.x; task < total; task += kBlockWarps * gridDim.x) {
        // job of the task: last j with prefix[j] <= task
        uint32_t loJ = 0, hiJ = nJobs;
        while (hiJ - loJ > 1) {
            const uint32_t mid = (loJ + hiJ) >> 1;
            if (sPrefix[mid] <= task) loJ = mid;
            else hiJ = mid;
        }
        const GemvJob &job = a.jobs[loJ];
        const uint32_t local = task - sPrefix[loJ];
        const uint32_t halves = (job.n + 7u) >> 3;
        const uint32_t tile = local / halves, colBase = (local - tile * halves) * 8u;
        const int nc = min(8, (int)job.n - (int)colBase);
        const int groups = (int)(job.cols >> 6);
        const int parts = (groups + (int)a.maxPartGroups - 1) / (int)a.maxPartGroups;
        const uint32_t sb = DUAL ? (uint32_t)groups * 16u : (uint32_t)groups * 32u;  // one scale run of the tile
        // this thread's input columns: g supplies the MMA's column g, results are columns 2t, 2t+1
        const uint32_t colRowG = job.inRow[colBase + (uint32_t)(g < nc ? g : 0)];
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int p = 0; p < parts; ++p) {
            int gb, ge;
            part_range(groups, parts, p, gb, ge);
            const uint32_t piece = (uint32_t)(ge - gb) * 32u;
            const uint32_t inPiece = (uint32_t)(ge - gb) * 128u;
            if (lane == 0)
                bar_expect(myBar, 16u * piece + (p == 0 ? (DUAL ? 4u : 2u) * sb : 0u) + (DUAL ? 0u : (uint32_t)nc * inPiece));
            __syncwarp();
            if (lane < 16) {
                const uint32_t row = DUAL ? tile * 8u + ((uint32_t)lane & 7u) : tile * 16u + (uint32_t)lane;
                const uint8_t *w = ((DUAL && lane >= 8) ? job.w1 : job.w0) + (size_t)row * (job.cols >> 1) + gb * 32;
                bulk_copy(slotAddr + (uint32_t)lane * a.pieceStride, w, piece, myBar);
            } else if (p == 0 && lane < (DUAL ? 20 : 18)) {
                const uint32_t which = (uint32_t)lane - 16u;
                const uint16_t *src = which == 0 ? job.s0 : which == 1 ? job.b0 : which == 2 ? job.s1 : job.b1;
                bulk_copy(slotAddr + 16u * a.pieceStride + which * a.scaleArea,
                          reinterpret_cast<const uint8_t *>(src) + (size_t)tile * sb, sb, myBar);
            } else if (!DUAL && lane >= 20 && lane < 20 + nc) {
                const uint32_t c = (uint32_t)lane - 20u;
                const uint16_t *src = job.in + (size_t)job.inRow[colBase + c] * job.inStride + (size_t)gb * 64;
                bulk_copy(slotAddr + 16u * a.pieceStride + 2u * a.scaleArea + c * a.inputPitch, src, inPiece, myBar);
            }
            slot_wait(myBar, parity, a.errorFlag);
            const uint8_t *lo = mySlot + (size_t)g * a.pieceStride + 8 * t;
            const uint8_t *hi = mySlot + (size_t)(g + 8) * a.pieceStride + 8 * t;
            const uint16_t *sc = reinterpret_cast<const uint16_t *>(mySlot + 16u * a.pieceStride);
            const uint32_t run = a.scaleArea >> 1;  // elements per scale run
            if (DUAL) {
                // rows g: gate row, g+8: up row of the same index; runs: gate s, gate b, up s, up b
                const uint16_t *gS = sc + g * groups + gb, *gB = gS + run, *uS = gB + run, *uB = uS + run;
                const uint8_t *xq = xAll + (size_t)colRowG * a.xPitch + (size_t)gb * 128 + t * 32;
                const uint32_t r0 = job.inRow[colBase + (uint32_t)min(2 * t, nc - 1)];
                const uint32_t r1 = job.inRow[colBase + (uint32_t)min(2 * t + 1, nc - 1)];
                tile_rows_cols<false>(lo, hi, xq, gS, gB, uS, uB, xSumAll + (size_t)r0 * groupsIn + gb,
                                      xSumAll + (size_t)r1 * groupsIn + gb, ge - gb, acc);
            } else {
                const uint16_t *s0 = sc + g * groups + gb, *b0 = s0 + run;
                const uint16_t *s1 = sc + (g + 8) * groups + gb, *b1 = s1 + run;
                const uint8_t *xq = mySlot + 16u * a.pieceStride + 2u * a.scaleArea + (size_t)(g < nc ? g : 0) * a.inputPitch + t * 32;
                tile_rows_cols<true>(lo, hi, xq, s0, b0, s1, b1, nullptr, nullptr, ge - gb, acc);
            }
            slot_release();
        }
        // epilogue: this thread holds columns 2t, 2t+1 of tile rows g and g+8
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int c = 2 * t + k;
            if (c >= nc) continue;
            uint16_t *dst = job.out + (size_t)job.outRow[colBase + (uint32_t)c] * job.outStride;
            if (DUAL) {
                float gate = acc[k], up = acc[2 + k];
                if (job.flags & kJobRoundGateUp) {
                    gate = bf16_round(gate);
                    up = bf16_round(up);
                }
                // run order 0,4,1,5,2,6,3,7: the order the down tasks' operands use
                dst[tile * 8u + (uint32_t)((g & 3) * 2 + (g >> 2))] = f2bf(gelu_tanh(gate) * up);
            } else {
                dst[tile * 16u + (uint32_t)g] = f2bf(acc[k]);
                dst[tile * 16u + 8u + (uint32_t)g] = f2bf(acc[2 + k]);
            }
        }
    }
}

struct BlockLayout {
    uint32_t maxPartGroups, xPitch, pieceStride, scaleArea, inputPitch, slotBytes, slotsOffset;
    size_t total;
};

// dual: gate/up jobs over `cols` input columns and `rows` staged input rows; otherwise down jobs
// whose widest matrix has `cols` columns.  Picks the largest K part that fits 227 KB.
static bool block_layout(bool dual, uint32_t cols, uint32_t rows, BlockLayout *out) {
    const uint32_t groups = cols / 64;
    const uint32_t kBlockWarps = dual ? kGateUpWarps : kDownWarps;
    for (uint32_t mpg = std::min(groups, 22u); mpg >= 1; --mpg) {
        BlockLayout l{};
        l.maxPartGroups = mpg;
        l.pieceStride = piece_stride(mpg * 32);
        l.scaleArea = dual ? groups * 16 : groups * 32;
        l.inputPitch = mpg * 128 + 16;
        l.xPitch = cols * 2 + 16;
        uint32_t slot = 16 * l.pieceStride + (dual ? 4u : 2u) * l.scaleArea + (dual ? 0u : 8u * l.inputPitch);
        l.slotBytes = (slot + 127u) & ~127u;
        l.slotsOffset = dual ? ((rows * l.xPitch + rows * groups * 4 + 127u) & ~127u) : 0u;
        l.total = (size_t)l.slotsOffset + (size_t)kBlockWarps * l.slotBytes;
        if (l.total + 2048 <= 227 * 1024) {  // 2 KB kept for the static arrays
            *out = l;
            return true;
        }
    }
    return false;
}

template <bool DUAL>
static bool launch_block_class(FFContext *ctx, const GemvJob *jobs, const uint32_t *jobCountPtr,
                               const uint16_t *allIn, uint32_t allStride, uint32_t allRows, uint32_t cols,
                               const char *name, cudaStream_t stream, const char **error) {
    BlockLayout lay{};
    if (!block_layout(DUAL, cols, allRows, &lay))
        return fail(error, "model shape too large for the block kernels' shared memory");
    BlockArgs a{};
    a.jobs = jobs;
    a.jobCountPtr = jobCountPtr;
    a.allIn = allIn;
    a.allStride = allStride;
    a.allRows = allRows;
    a.cols = cols;
    a.maxPartGroups = lay.maxPartGroups;
    a.xPitch = lay.xPitch;
    a.pieceStride = lay.pieceStride;
    a.scaleArea = lay.scaleArea;
    a.inputPitch = lay.inputPitch;
    a.slotBytes = lay.slotBytes;
    a.slotsOffset = lay.slotsOffset;
    a.errorFlag = ctx->errorFlag;
    static KernelSmemMemo memo;
    if (!memo.prepare(k_block_mma<DUAL>, ctx->device, lay.total, (DUAL ? kGateUpWarps : kDownWarps) * 32, nullptr, error))
        return false;
    LaunchScope scope(ctx, stream, name);
    k_block_mma<DUAL><<<ctx->smCount, (DUAL ? kGateUpWarps : kDownWarps) * 32, lay.total, stream>>>(a);
    FF_CUDA_OK(cudaGetLastError(), error);
    return true;
}

// The gate/up + GeGLU jobs and then the down jobs of a planned block (jobs[0], jobs[1] of the
// context, counts in its route plan).  x: the block's `tokens` input rows.
bool launch_block_mma(FFContext *ctx, const uint16_t *x, uint32_t xStride, uint32_t tokens, bool withShared,
                      bool haveDownJobs, cudaStream_t stream, const char **error) {
    const FFConfig &c = ctx->cfg;
    if (c.d % 64 || c.f % 64 || c.sharedF % 64) return fail(error, "widths must be multiples of 64");
    if (((uintptr_t)x & 15) || (xStride % 8)) return fail(error, "input rows must be 16-byte aligned");
    if (!launch_block_class<true>(ctx, ctx->jobs[0], &ctx->plan->jobCount[0], x, xStride, tokens, c.d,
                                  "int4_block_gate_up_act", stream, error))
        return false;
    if (!haveDownJobs) return true;
    const uint32_t maxCols = withShared ? std::max(c.f, c.sharedF) : c.f;
    return launch_block_class<false>(ctx, ctx->jobs[1], &ctx->plan->jobCount[1], nullptr, 0, 0, maxCols,
                                     "int4_block_down", stream, error);
}

}  // namespace ff
