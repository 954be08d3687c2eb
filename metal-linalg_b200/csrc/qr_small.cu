// The small-matrix kernel: a matrix of at most 32 x 32 in the registers of half a
// warp, a quarter or an eighth of one (two, four or eight ... matrices a warp).
//
// It takes the place of the reference's register kernel qr_householder_simd
// (shaders/QR_Householder.metal:189-300; host side src/qr_householder.mm:86-98,
// 263-381) and keeps its contract: per matrix a scan for the largest magnitude
// and for NaN/Inf (such a matrix gives all-NaN Q and R), scaling by a power of
// two into [0.5, 1), LAPACK's sgeqr2 (reflectors with slarfg's signs), R
// written with exact zeros below the diagonal and multiplied back by the power
// of two, Q formed backward as sorg2r does.
//
// The mapping is not the reference's. There a lane holds rows and every dot
// product is a reduction across lanes. Here a lane holds COLUMNS (C of them, R
// rows each, in registers: lane l of a group of G has columns l, l + G, ...), so
// a reflector's dot products with the columns right of it are each lane's own
// FMAs with no reduction at all. What crosses lanes is the reflector: the lane
// that owns column j writes it to shared memory once (16 bytes an instruction)
// and every lane reads it back as broadcast 16-byte words, four rows an
// instruction; it stays there for the Q pass, which therefore only reads. The
// arithmetic on rows is packed two to an instruction (fma.rn.f32x2, the
// Blackwell packed FP32 FMA). The reflector is kept unnormalised, H = I - g v
// v^T with v = (alpha - beta; tail): one reciprocal a column, no pass to scale
// the tail, and the pivot row is updated by the same packed instructions as the
// rest.
//
// The kernel is bound by instruction issue and by the FMA pipe, not by memory
// (its DRAM traffic is the algorithmic 12 KB per 32 x 32 matrix), so the design
// minimises warp instructions per matrix. Two columns a lane (C = 2) halve what
// does not scale with the columns: with G = 16 a warp factors two 32 x 32
// matrices at once, so every scalar instruction of a step (the reflector's
// norm, its square root and reciprocal, the publication, the broadcast loads)
// serves two matrices, and once the step has passed column G the first column
// of every lane is finished and its arithmetic is skipped altogether.
//
// Global memory: lanes of a group read consecutive floats of a row, so a warp's
// load instruction covers whole 64- or 128-byte runs; stores the same.
#include "kernels.h"
#include "qr_small_steps.cuh"

#include <cstdlib>

namespace mlb {

using namespace small;

namespace {

struct SmallParams {
    const float* a;
    float*       q;
    float*       r;
    uint32_t     batch;
    int          m, n, K, qc, rr;
};

// Blocks of up to kMaxWarps warps; how many of them a multiprocessor is to hold, by the registers
// a lane needs for its R * C matrix entries.
constexpr int kMaxWarps = 8;
constexpr uint32_t kPrefetchBlocks = 74;   // how far ahead, in blocks, a block prefetches input into L2
__host__ __device__ constexpr int min_blocks(int R, int C) { return R * C > 64 ? 1 : R * C > 32 ? 2 : 3; }

// R: rows held per lane (row capacity, a multiple of 4). G: lanes per matrix. C: columns per lane
// (column capacity G * C; lane l holds columns l, l + G, ...).
// Square: the matrix is exactly R x R with R = G * C (and Q, where asked for, R x R), so every bound
// is known when the kernel is compiled and no load, store or step is guarded.
template <int R, int G, int C, bool Square>
__global__ void __launch_bounds__(kMaxWarps * 32, min_blocks(R, C)) qr_small_kernel(const SmallParams p) {
    constexpr int kCols  = G * C;
    constexpr int kSteps = R < kCols ? R : kCols;
    constexpr int kSlot = slot_floats(R, kSteps);
    extern __shared__ __align__(16) float smem[];
    const int lane  = threadIdx.x & 31;
    const int l     = lane % G;          // this lane's first column
    const uint32_t group = threadIdx.x / G;                       // matrix slot within the block
    uint32_t mat = blockIdx.x * (blockDim.x / G) + group;
    const bool live = mat < p.batch;
    if (!live) mat = p.batch - 1;        // keeps the group in step with the warp; stores are masked
    const int m = Square ? R : p.m, n = Square ? R : p.n, K = Square ? R : p.K;
    const int rr = Square ? R : p.rr, qc = Square && p.qc ? R : p.qc;

    const float* src = p.a + (size_t)mat * m * n;

    // 0. The input of the block kPrefetchBlocks further on goes to L2 now: that block starts while this one
    // is still computing, and its loads then take an L2 hit's time instead of a trip to HBM, during which
    // a warp holds its registers and does nothing (measured on 262 144 matrices of 32 x 32: 1.26 -> 1.15 ms,
    // the same for any distance from 18 to 148 blocks; beyond a wave of blocks, 296, the lines are evicted
    // again before they are used).
    {
        const uint32_t per_block = blockDim.x / G;
        const size_t first = (size_t)(blockIdx.x + kPrefetchBlocks) * per_block;
        if (first < p.batch) {
            const size_t left = p.batch - first;
            const size_t bytes = (left < per_block ? left : per_block) * (size_t)m * n * sizeof(float);
            const char* base = reinterpret_cast<const char*>(p.a + first * m * n);
            for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)blockDim.x * 128)
                asm volatile("prefetch.global.L2 [%0];" :: "l"(base + off));
        }
    }

    // 1. load; rows 2p and 2p+1 of column l + c G packed in x2[c][p]
    pair_t x2[C][R / 2];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int col = l + c * G;
#pragma unroll
        for (int i = 0; i < R / 2; ++i) {
            float a = 0.0f, b = 0.0f;
            if (2 * i < m && col < n) a = src[(2 * i) * n + col];
            if (2 * i + 1 < m && col < n) b = src[(2 * i + 1) * n + col];
            x2[c][i] = pack(a, b);
        }
    }
    bool bad;
    int  expo;
    scan_scale<R, G, C>(x2, bad, expo);

    // 2. factor
    float* slot = smem + (size_t)group * kSlot;
    factor<R, G, C>(x2, slot, l, K);

    // 3. R: row i across the lanes, exact zeros below the diagonal
    {
        scale_up<R, G, C>(x2, expo, bad);
        const float zero = bad ? qnan() : 0.0f;
        float* dst = p.r + (size_t)mat * rr * n;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = l + c * G;
            if (live && col < n) {
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const float v = (i & 1) ? hi_of(x2[c][i / 2]) : lo_of(x2[c][i / 2]);
                    if (i < rr) __stcs(&dst[i * n + col], (i < K && col >= i) ? v : zero);
                }
            }
        }
    }
    if (qc == 0) return;

    // 4. Q's columns
    pair_t q2[C][R / 2];
    form_q<R, G, C>(q2, slot, l, K, bad, [] {});

    // 5. Q
    if (live) {
        float* dst = p.q + (size_t)mat * m * qc;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = l + c * G;
            if (col < qc) {
#pragma unroll
                for (int i = 0; i < R / 2; ++i) {
                    float a, b;
                    unpack(q2[c][i], a, b);
                    if (2 * i < m) __stcs(&dst[(2 * i) * qc + col], a);      // written once, not read again here: evict first
                    if (2 * i + 1 < m) __stcs(&dst[(2 * i + 1) * qc + col], b);
                }
            }
        }
    }
}

template <int R, int G, int C, bool Square>
void launch(cudaStream_t stream, const SmallParams& p, int sm_count, int device) {
    constexpr int per_warp = 32 / G;
    constexpr int steps = R < G * C ? R : G * C;
    static const int max_warps = [] {
        const char* e = std::getenv("QR_SMALL_WARPS");
        const int w = e ? std::atoi(e) : kMaxWarps;
        return w >= 1 && w <= kMaxWarps ? w : kMaxWarps;
    }();
    // a small batch in smaller blocks, so that it reaches every multiprocessor
    int warps_per_block = max_warps;
    while (warps_per_block > 1 && (p.batch + per_warp * warps_per_block - 1) / (per_warp * warps_per_block) < 2u * sm_count)
        warps_per_block /= 2;
    const uint32_t per_block = per_warp * warps_per_block;
    const uint32_t blocks = (p.batch + per_block - 1) / per_block;
    const size_t smem = (size_t)per_block * slot_floats(R, steps) * sizeof(float);
    static PerDeviceOnce once;      // the opt-in is recorded per GPU
    if (once.first(device)) {
        cuda_check(cudaFuncSetAttribute(qr_small_kernel<R, G, C, Square>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (32 / G) * kMaxWarps * slot_floats(R, steps) * (int)sizeof(float)),
                   "qr_small shared memory");
        cuda_check(cudaFuncSetAttribute(qr_small_kernel<R, G, C, Square>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared),
                   "qr_small shared memory carveout");
        once.mark(device);
    }
    qr_small_kernel<R, G, C, Square><<<blocks, 32 * warps_per_block, smem, stream>>>(p);
}

// Columns a lane (1, 2 or 4), for measurements: QR_SMALL_COLS. 0: the default of the shape.
int forced_columns_a_lane() {
    static const int v = [] {
        const char* e = std::getenv("QR_SMALL_COLS");
        const int c = e ? std::atoi(e) : 0;
        return c == 1 || c == 2 || c == 4 ? c : 0;
    }();
    return v;
}

int pow2_at_least(uint32_t v, int lo) {
    int c = lo;
    while ((uint32_t)c < v) c *= 2;
    return c;
}

} // namespace

bool qr_small_fits(uint32_t m, uint32_t n, uint32_t qc) { return m <= 32 && n <= 32 && qc <= 32 && m > 0 && n > 0; }

void launch_qr_small(DeviceContext& ctx, cudaStream_t stream, const QrProblem& pr) {
    if (pr.batch == 0) return;
    if (launch_qr_small_stream(ctx, stream, pr)) return;
    SmallParams p{pr.a, pr.q, pr.r, pr.batch, (int)pr.m, (int)pr.n, (int)qr_k(pr), (int)pr.qc, (int)pr.rr};
    const int R   = pow2_at_least(pr.m, 8);
    const int cap = pow2_at_least(pr.n > pr.qc ? pr.n : pr.qc, 8);      // column capacity
    int C = forced_columns_a_lane() ? forced_columns_a_lane() : 2;
    while (C > 1 && cap / C < 4) C /= 2;
    if (cap == 8 && !forced_columns_a_lane()) C = 1;
    // a batch too small to give every multiprocessor a warp at two columns a lane: one column a lane
    // (twice the warps, each half as long)
    if (!forced_columns_a_lane() && C == 2 && (uint64_t)pr.batch * (cap / 2) < (uint64_t)32 * 4 * ctx.sm_count) C = 1;
    const int G = cap / C;
    const bool square = pr.m == pr.n && (int)pr.m == R && cap == R && pr.rr == pr.m && (pr.qc == 0 || pr.qc == pr.m);
#define MLB_SMALL(RR, GG, CC)                                                    \
    if (R == RR && G == GG && C == CC) {                                         \
        if constexpr (RR == GG * CC) {                                           \
            if (square) launch<RR, GG, CC, true>(stream, p, ctx.sm_count, ctx.device);       \
            else launch<RR, GG, CC, false>(stream, p, ctx.sm_count, ctx.device);             \
        } else launch<RR, GG, CC, false>(stream, p, ctx.sm_count, ctx.device);               \
    }
#define MLB_SMALL_ROWS(RR)                                                                        \
    MLB_SMALL(RR, 8, 1) MLB_SMALL(RR, 16, 1) MLB_SMALL(RR, 32, 1) /* one column a lane */        \
    MLB_SMALL(RR, 4, 2) MLB_SMALL(RR, 8, 2) MLB_SMALL(RR, 16, 2)  /* two */                       \
    MLB_SMALL(RR, 4, 4) MLB_SMALL(RR, 8, 4)                       /* four */
    MLB_SMALL_ROWS(8) MLB_SMALL_ROWS(16) MLB_SMALL_ROWS(32)
#undef MLB_SMALL_ROWS
#undef MLB_SMALL
    cuda_check(cudaGetLastError(), "qr_small launch");
}

} // namespace mlb
