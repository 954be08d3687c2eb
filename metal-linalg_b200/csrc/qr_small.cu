// The small-matrix kernel: a matrix of at most 32 x 32 in the registers of one
// warp, or of a half or a quarter of one (two or four matrices a warp).
//
// It takes the place of the reference's register kernel qr_householder_simd
// (shaders/QR_Householder.metal:189-300; host side src/qr_householder.mm:86-98,
// 263-381) and keeps its contract: per matrix a scan for the largest magnitude
// and for NaN/Inf (such a matrix gives all-NaN Q and R), scaling by a power of
// two into [0.5, 1), LAPACK's sgeqr2 (reflectors with slarfg's signs), R
// written with exact zeros below the diagonal and multiplied back by the power
// of two, Q formed backward in place as sorg2r does.
//
// The mapping is not the reference's. There a lane holds rows and every dot
// product is a reduction across lanes. Here a lane holds a COLUMN (R rows of it
// in registers), so a reflector's dot products with the columns right of it are
// each lane's own FMAs with no reduction at all; what crosses lanes is the
// reflector itself, broadcast from the lane that owns it, one shuffle a row.
// The reflector's tail is left unscaled in its lane (the factor 1/(alpha-beta)
// is carried as a scalar), which saves a pass over it.
//
// Global memory: lanes of a group read consecutive floats of a row, so a warp's
// load instruction covers whole 128-byte lines (32-column matrices) or whole
// 32-byte sectors (narrower ones); stores the same.
#include "common.cuh"
#include "kernels.h"

#include <cstdlib>

namespace mlb {

namespace {

struct SmallParams {
    const float* a;
    float*       q;
    float*       r;
    uint32_t     batch;
    int          m, n, K, qc, rr;
};

// R: rows held per lane (row capacity). G: lanes per matrix (column capacity).
template <int R, int G>
__global__ void __launch_bounds__(512) qr_small_kernel(const SmallParams p) {
    constexpr int kSteps = R < G ? R : G;
    const int lane  = threadIdx.x & 31;
    const int l     = lane % G;          // this lane's column
    const int gbase = lane - l;          // first lane of the group
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    uint32_t mat = warp * (32 / G) + lane / G;
    const bool live = mat < p.batch;
    if (!live) mat = p.batch - 1;        // keeps the group in step with the warp's shuffles; stores are masked
    const int m = p.m, n = p.n, K = p.K;

    const float* src = p.a + (size_t)mat * m * n;

    // 1. load, scan, scale
    float x[R];
    float amax = 0.0f;
    bool  bad  = false;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        float v = 0.0f;
        if (i < m && l < n) v = src[i * n + l];
        x[i] = v;
        amax = fmaxf(amax, fabsf(v));
        bad |= nonfinite(v);
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        bad |= (bool)__shfl_xor_sync(0xffffffffu, (int)bad, o);
    }
    int expo = 0;
    if (bad) {
        // a finite, harmless stand-in keeps the arithmetic quiet; the outputs are NaN
#pragma unroll
        for (int i = 0; i < R; ++i) x[i] = 0.0f;
    } else {
        expo = amax_exponent(amax);
        const Pow2 down(-expo);
#pragma unroll
        for (int i = 0; i < R; ++i) x[i] = down(x[i]);
    }

    // 2. factor. After step j, lane j holds beta in x[j] and the reflector's
    // unscaled tail below it; lanes right of j hold their updated columns.
    float tau_own = 0.0f, sc_own = 0.0f;   // of the reflector this lane owns
    float u[R];
#pragma unroll
    for (int j = 0; j < kSteps; ++j) {
        if (j < K) {
            float ss = 0.0f;
#pragma unroll
            for (int i = j + 1; i < R; ++i) ss = fmaf(x[i], x[i], ss);
            const float alpha = __shfl_sync(0xffffffffu, x[j], gbase + j);
            ss = __shfl_sync(0xffffffffu, ss, gbase + j);
            float beta, tau, sc;
            reflector(alpha, ss, beta, tau, sc);
            float s = 0.0f;
#pragma unroll
            for (int i = j + 1; i < R; ++i) {
                u[i] = __shfl_sync(0xffffffffu, x[i], gbase + j);
                s = fmaf(u[i], x[i], s);
            }
            const float dot = fmaf(sc, s, x[j]);
            const float w   = l > j ? tau * dot : 0.0f;
            x[j] = l == j ? beta : x[j] - w;
            const float ws = w * sc;
#pragma unroll
            for (int i = j + 1; i < R; ++i) x[i] = fmaf(-ws, u[i], x[i]);
            if (l == j) {
                tau_own = tau;
                sc_own  = sc;
            }
        }
    }

    // 3. R: row i is x[i] across the lanes
    const Pow2 up(expo);
    if (live && l < n) {
        float* dst = p.r + (size_t)mat * p.rr * n;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            if (i < p.rr) {
                float v = (i < K && l >= i) ? up(x[i]) : 0.0f;
                if (bad) v = qnan();
                dst[i * n + l] = v;
            }
        }
    }
    if (p.qc == 0) return;

    // 4. Q's columns, backward: lane l holds column l of Q
    float qv[R];
#pragma unroll
    for (int i = 0; i < R; ++i) qv[i] = i == l ? 1.0f : 0.0f;
#pragma unroll
    for (int j = kSteps - 1; j >= 0; --j) {
        if (j < K) {
            const float tau = __shfl_sync(0xffffffffu, tau_own, gbase + j);
            const float sc  = __shfl_sync(0xffffffffu, sc_own, gbase + j);
            float s = 0.0f;
#pragma unroll
            for (int i = j + 1; i < R; ++i) {
                u[i] = __shfl_sync(0xffffffffu, x[i], gbase + j);
                s = fmaf(u[i], qv[i], s);
            }
            const float w = tau * fmaf(sc, s, qv[j]);
            qv[j] -= w;
            const float ws = w * sc;
#pragma unroll
            for (int i = j + 1; i < R; ++i) qv[i] = fmaf(-ws, u[i], qv[i]);
        }
    }

    // 5. Q
    if (live && l < p.qc) {
        float* dst = p.q + (size_t)mat * m * p.qc;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            if (i < m) dst[i * p.qc + l] = bad ? qnan() : qv[i];
        }
    }
}

template <int R, int G>
void launch(cudaStream_t stream, const SmallParams& p) {
    constexpr int per_warp = 32 / G;
    static const int warps_per_block = [] {
        const char* e = std::getenv("QR_SMALL_WARPS");
        const int w = e ? std::atoi(e) : 8;
        return w >= 1 && w <= 16 ? w : 8;
    }();
    const uint32_t per_block = per_warp * warps_per_block;
    const uint32_t blocks = (p.batch + per_block - 1) / per_block;
    qr_small_kernel<R, G><<<blocks, 32 * warps_per_block, 0, stream>>>(p);
}

int pow2_at_least(uint32_t v, int lo) {
    int c = lo;
    while ((uint32_t)c < v) c *= 2;
    return c;
}

} // namespace

bool qr_small_fits(uint32_t m, uint32_t n, uint32_t qc) { return m <= 32 && n <= 32 && qc <= 32 && m > 0 && n > 0; }

void launch_qr_small(DeviceContext&, cudaStream_t stream, const QrProblem& pr) {
    if (pr.batch == 0) return;
    SmallParams p{pr.a, pr.q, pr.r, pr.batch, (int)pr.m, (int)pr.n, (int)qr_k(pr), (int)pr.qc, (int)pr.rr};
    const int R = pow2_at_least(pr.m, 8);
    const int G = pow2_at_least(pr.n > pr.qc ? pr.n : pr.qc, 8);
#define MLB_SMALL(RR, GG) if (R == RR && G == GG) { launch<RR, GG>(stream, p); }
    MLB_SMALL(8, 8) MLB_SMALL(8, 16) MLB_SMALL(8, 32)
    MLB_SMALL(16, 8) MLB_SMALL(16, 16) MLB_SMALL(16, 32)
    MLB_SMALL(32, 8) MLB_SMALL(32, 16) MLB_SMALL(32, 32)
#undef MLB_SMALL
    cuda_check(cudaGetLastError(), "qr_small launch");
}

} // namespace mlb
