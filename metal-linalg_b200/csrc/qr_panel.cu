// Panel factorisation for the blocked QR: a panel of up to 16384 rows x 32
// columns to compact-WY form (Y unit lower trapezoidal, T, R) in three launches.
//
// It takes the place of the reference's tall-panel kernels bd_tsqr_leaf,
// bd_tsqr_top and bd_tsqr_rebuild (shaders/Svd_Bidiag.metal:583-869, driven by
// src/band_reduce.mm:196-251): TSQR over row blocks, then Householder
// reconstruction (Ballard et al. 2014) so that the trailing update sees one
// ordinary block reflector.
//
//   panel_leaf_kernel   one thread block per block of 256 * RPT rows, a thread
//                       per row (RPT rows) held in registers. 32 column steps;
//                       a step is ONE reduction over the block of 32 numbers per
//                       thread, x[row][j] * x[row][c] for all 32 columns c: for
//                       c > j these are the reflector's dot products with the
//                       trailing columns, for c = j its norm, and for c < j its
//                       products with the earlier reflectors, which is the Gram
//                       matrix that T is built from. The current column is kept
//                       at register index 0 by rotating the row one place per
//                       step, so the step loop is not unrolled and every
//                       register index is a constant. Out: the block's V, T, R.
//   panel_top_kernel    one thread block: the same factorisation of the stacked
//                       R's (at most 512 rows), the tree's Q on the first 32
//                       rows, LU with sign choice of Q1 - S (every pivot at least
//                       1 in magnitude), T = -U S L1^-T, the panel's R = S R, and
//                       for every leaf the 32 x 32 factor B' = (its block of the
//                       top Q) U^-1.
//   panel_apply_kernel  per leaf: Y rows = [B'; 0] - V (T (V_top^T B')).
#include "common.cuh"
#include "kernels.h"
#include "qr_panel_cols.cuh"

#include <algorithm>
#include <cstdlib>

namespace mlb {

namespace {

constexpr int PT = 256;     // threads per block
constexpr unsigned kFull = 0xffffffffu;

struct PanelSmem {
    float red[2][PT / 32][32];   // each warp's column sums, by step parity
    float prow[2][32];           // the pivot row, in rotated column order, by step parity
    float wv[PT / 32][32];       // per warp: per rotated column the update coefficient (0 where nothing is to update)
    float taus[32];
    float G[32][33];          // G[k][j] = v_k^T v_j for k < j
    float T[32][33];
};

// slarfg's reflector as common.cuh's, with rsqrt / rcp and one Newton step each instead of the
// IEEE square root and divisions (it sits on the critical path of every column step).
__device__ __forceinline__ float newton_div(float a, float b) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(b));
    const float q = a * r;
    return fmaf(fmaf(-b, q, a), r, q);
}
__device__ __forceinline__ void reflector_fast(float alpha, float ss, float& beta, float& tau, float& sc) {
    beta = alpha;
    tau  = 0.0f;
    sc   = 0.0f;
    if (ss >= kTinySumsq) {
        const float n2 = fmaf(alpha, alpha, ss);
        const float y = rsqrtf(n2);
        float nrm = n2 * y;
        nrm = fmaf(fmaf(-nrm, nrm, n2), 0.5f * y, nrm);
        beta = -copysignf(nrm, alpha);
        tau  = newton_div(beta - alpha, beta);
        sc   = newton_div(1.0f, alpha - beta);
    }
}

// Sum over the warp of 32 values a lane: lane c returns the sum of p[c].
__device__ __forceinline__ float butterfly32(float (&p)[32], int lane) {
#pragma unroll
    for (int half = 16; half >= 1; half >>= 1) {
        const bool upper = (lane & half) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float send = upper ? p[i] : p[i + half];
            const float keep = upper ? p[i + half] : p[i];
            p[i] = keep + __shfl_xor_sync(kFull, send, half);
        }
    }
    return p[0];
}

// Householder QR of the rows held by the block: thread t holds rows t + 256 k, k < RPT, 32 columns
// each. Afterwards x holds R (rows < 32, on and above the diagonal) and the reflectors' tails,
// scaled to unit diagonal (below it); s.taus, s.G are set. Rows >= the block's real row count
// must be zero on entry.
template <int RPT>
__device__ __forceinline__ void factor_rows(float (&x)[RPT][32], PanelSmem& s) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
#pragma unroll 1
    for (int j = 0; j < 32; ++j) {
        // the original column (j + k) % 32 is at register index k
        float p[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) p[c] = 0.0f;
#pragma unroll
        for (int k = 0; k < RPT; ++k) {
            const float v = (t + PT * k > j) ? x[k][0] : 0.0f;
#pragma unroll
            for (int c = 0; c < 32; ++c) p[c] = fmaf(v, x[k][c], p[c]);
        }
        const int buf = j & 1;
        if (t == j) {
#pragma unroll
            for (int c = 0; c < 32; ++c) s.prow[buf][c] = x[0][c];
        }
        s.red[buf][warp][lane] = butterfly32(p, lane);
        __syncthreads();
        // every warp sums the block's columns and forms the reflector for itself: one barrier a step
        // (the buffers alternate, so the next step's writes cannot overtake this step's reads)
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < PT / 32; ++w) v += s.red[buf][w][lane];
        const float ss = __shfl_sync(kFull, v, 0);
        float beta, tau, sc;
        reflector_fast(s.prow[buf][0], ss, beta, tau, sc);
        const float val = fmaf(sc, v, s.prow[buf][lane]);
        s.wv[warp][lane] = (lane >= 1 && lane <= 31 - j) ? tau * val : 0.0f;
        if (warp == 0) {
            if (lane >= 32 - j) s.G[(j + lane) & 31][j] = val;
            if (lane == 0) s.taus[j] = tau;
        }
        __syncwarp();
        float w[32];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(&s.wv[warp][4 * q]);
            w[4 * q] = f.x; w[4 * q + 1] = f.y; w[4 * q + 2] = f.z; w[4 * q + 3] = f.w;
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < RPT; ++k) {
            const int row = t + PT * k;
            const float vr = row > j ? sc * x[k][0] : (row == j ? 1.0f : 0.0f);
            const float head = row > j ? vr : (row == j ? beta : x[k][0]);
#pragma unroll
            for (int c = 1; c < 32; ++c) x[k][c - 1] = fmaf(-w[c], vr, x[k][c]);   // update and rotate left
            x[k][31] = head;
        }
    }
}

// T from s.G and s.taus (slarft's forward recurrence), by warp 0, a row of T per lane.
template <typename Smem>
__device__ __forceinline__ void build_t(Smem& s) {
    if (threadIdx.x < 32) {
        const int i = threadIdx.x;
        float tr[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float tau = s.taus[j];
            float a = 0.0f;
#pragma unroll
            for (int k = 0; k < j; ++k) a = fmaf(tr[k], s.G[k][j], a);
            tr[j] = i < j ? -tau * a : (i == j ? tau : 0.0f);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) s.T[i][j] = tr[j];
    }
}

// The clean reflector entry of row `row`: unit diagonal, zeros above.
__device__ __forceinline__ float clean_v(float x, int row, int c) { return c < row ? x : (c == row ? 1.0f : 0.0f); }

// C (32 x 32, ld 33) = op(A) B for 32 x 32 matrices in shared memory, by the whole block.
template <bool TransA>
__device__ __forceinline__ void mat32(const float (*A)[33], const float (*B)[33], float (*C)[33]) {
    const int i = threadIdx.x >> 3, c0 = (threadIdx.x & 7) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
        const float a = TransA ? A[k][i] : A[i][k];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = fmaf(a, B[k][c0 + e], acc[e]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) C[i][c0 + e] = acc[e];
}

struct LeafParams {
    const float* panel;     // the panel's first entry in the working copy
    size_t       ldw;
    uint32_t     mp, jb, lr;   // rows and columns of the panel, rows per leaf
    float*       Vl;        // [leaves][lr][32] clean reflectors
    float*       Tl;        // [leaves][32][32]
    float*       Sl;        // [leaves * 32][32] the stack of R's
};

template <int RPT>
__global__ void __launch_bounds__(PT) panel_leaf_kernel(const LeafParams p) {
    dependency_wait();
    __shared__ __align__(16) PanelSmem s;
    const int t = threadIdx.x;
    const uint32_t blk = blockIdx.x, row0 = blk * p.lr;
    float x[RPT][32];
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
        const uint32_t gr = row0 + t + PT * k;
        const float* src = p.panel + (size_t)gr * p.ldw;
        if (gr < p.mp && p.jb == 32) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 f = *reinterpret_cast<const float4*>(src + 4 * q);
                x[k][4 * q] = f.x; x[k][4 * q + 1] = f.y; x[k][4 * q + 2] = f.z; x[k][4 * q + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) x[k][c] = (gr < p.mp && (uint32_t)c < p.jb) ? src[c] : 0.0f;
        }
    }
    factor_rows<RPT>(x, s);
    __syncthreads();
    build_t(s);
    if (t < 32) {
        float* dst = p.Sl + ((size_t)blk * 32 + t) * 32;
#pragma unroll
        for (int c = 0; c < 32; ++c) dst[c] = c >= t ? x[0][c] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
        const int row = t + PT * k;
        float* dst = p.Vl + ((size_t)blk * p.lr + row) * 32;
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(dst + 4 * q) =
                make_float4(clean_v(x[k][4 * q], row, 4 * q), clean_v(x[k][4 * q + 1], row, 4 * q + 1),
                            clean_v(x[k][4 * q + 2], row, 4 * q + 2), clean_v(x[k][4 * q + 3], row, 4 * q + 3));
    }
    __syncthreads();
    for (int idx = t; idx < 1024; idx += PT) p.Tl[(size_t)blk * 1024 + idx] = s.T[idx >> 5][idx & 31];
}

// One row of the top Q's first 32 columns, B = [I; 0] - V M with M = T V1^T, to Bp.
__device__ __forceinline__ void top_q_row(const float (&xr)[32], const int row, const float (*M4)[36], float* Bp,
                                          uint32_t S) {
    float b[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) b[c] = (row == c) ? 1.0f : 0.0f;
#pragma unroll
    for (int kk = 0; kk < 32; ++kk) {
        const float v = clean_v(xr[kk], row, kk);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 m4 = *reinterpret_cast<const float4*>(&M4[kk][4 * q]);
            b[4 * q] = fmaf(-v, m4.x, b[4 * q]); b[4 * q + 1] = fmaf(-v, m4.y, b[4 * q + 1]);
            b[4 * q + 2] = fmaf(-v, m4.z, b[4 * q + 2]); b[4 * q + 3] = fmaf(-v, m4.w, b[4 * q + 3]);
        }
    }
    if ((uint32_t)row < S) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(Bp + (size_t)row * 32 + 4 * q) =
                make_float4(b[4 * q], b[4 * q + 1], b[4 * q + 2], b[4 * q + 3]);
    }
}

struct TopParams {
    const float* Sl;        // [S][32] stacked R's
    uint32_t     S;         // rows of the stack (leaves * 32, at most 512)
    const float* Vl;        // leaf 0's clean reflectors (its first 32 rows are used)
    const float* Tl;        // leaf 0's T
    float*       Bp;        // [S][32] out: per leaf B' = (its block of the top Q) U^-1
    float*       w;         // the panel's first entry in the working copy: gets S R (upper triangle)
    size_t       ldw;
    float*       y;         // the panel's first entry in Y: gets the unit lower triangular L1
    size_t       ldy;
    float*       t;         // [32][32] out: T of the panel
    uint32_t     jb, mp;
    float*       Rt;        // [32][32] scratch: the R of the stack, from the top kernel to the finish kernel
};

// The stack of R's factored; out: its R (Rt) and the rows of its Q's first 32 columns (Bp).
template <int RPT>
__global__ void __launch_bounds__(PT, 1) panel_top_kernel(const TopParams p) {
    dependency_wait();
    __shared__ __align__(16) PanelSmem s;
    __shared__ float V1[32][33];
    __shared__ __align__(16) float M4[32][36];   // read as 16-byte words
    const int t = threadIdx.x;
    float x[RPT][32];
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
        const uint32_t r = t + PT * k;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < p.S) f = *reinterpret_cast<const float4*>(p.Sl + (size_t)r * 32 + 4 * q);
            x[k][4 * q] = f.x; x[k][4 * q + 1] = f.y; x[k][4 * q + 2] = f.z; x[k][4 * q + 3] = f.w;
        }
    }
    factor_rows<RPT>(x, s);
    __syncthreads();
    build_t(s);
    if (t < 32) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            p.Rt[t * 32 + c] = c >= t ? x[0][c] : 0.0f;
            V1[t][c] = clean_v(x[0][c], t, c);
        }
    }
    __syncthreads();
    // the top Q's rows: B = [I; 0] - V (T V1^T)
    {   // M = T V1^T: M[k][c] = sum_k' T[k][k'] V1[c][k']
        const int i = t >> 3, c0 = (t & 7) * 4;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const float a = s.T[i][k];
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(a, V1[c0 + e][k], acc[e]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) M4[i][c0 + e] = acc[e];
    }
    __syncthreads();
    // a row of B per thread and pass; the rows wait in global memory (Bp) for U
    top_q_row(x[0], t, M4, p.Bp, p.S);
    asm volatile("" ::: "memory");   // keeps the compiler from holding all of M4 in registers across the two rows
    if (RPT > 1) top_q_row(x[RPT - 1], t + PT, M4, p.Bp, p.S);
}

// Householder reconstruction from the top's Q rows (Bp) and leaf 0's reflectors: the panel's T, R
// and L1, and Bp <- Bp U^-1.
__global__ void __launch_bounds__(PT) panel_finish_kernel(const TopParams p) {
    dependency_wait();
    __shared__ float M[32][33], B0[32][33], X[32][33], V0[32][33], T0[32][33], Rm[32][33];
    __shared__ __align__(16) float Q[32][36];   // read as 16-byte words
    __shared__ float sgn[32];
    const int t = threadIdx.x;
    for (int idx = t; idx < 1024; idx += PT) {
        V0[idx >> 5][idx & 31] = p.Vl[idx];
        T0[idx >> 5][idx & 31] = p.Tl[idx];
        B0[idx >> 5][idx & 31] = p.Bp[idx];
        Rm[idx >> 5][idx & 31] = p.Rt[idx];
    }
    __syncthreads();
    // the panel's Q on its first 32 rows: Q1 = B0 - V0 (T0 (V0^T B0)), V0 and T0 leaf 0's
    mat32<true>(V0, B0, X);
    __syncthreads();
    mat32<false>(T0, X, M);
    __syncthreads();
    mat32<false>(V0, M, X);
    __syncthreads();
    for (int idx = t; idx < 1024; idx += PT) Q[idx >> 5][idx & 31] = B0[idx >> 5][idx & 31] - X[idx >> 5][idx & 31];
    __syncthreads();
    // LU of Q1 - S with S = -sgn(pivot) chosen on the way (every pivot at least 1 in magnitude): one
    // warp, a row per lane in registers, the pivot row handed round by shuffles
    if (t < 32) {
        const int i = t;
        float q[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) q[c] = Q[i][c];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float d = __shfl_sync(kFull, q[j], j);
            const float sg = d >= 0.0f ? -1.0f : 1.0f;
            const float piv = d - sg;
            if (i == j) {
                q[j] = piv;
                sgn[j] = sg;
            }
            const float l = i > j ? newton_div(q[j], piv) : 0.0f;
            if (i > j) q[j] = l;
#pragma unroll
            for (int c = j + 1; c < 32; ++c) {
                const float pc = __shfl_sync(kFull, q[c], j);
                q[c] = fmaf(-l, pc, q[c]);      // l = 0 in the rows above: unchanged
            }
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) Q[i][c] = q[c];
    }
    __syncthreads();
    // B' = B U^-1, a row per thread and pass: x U = b, eliminating with one row of U at a time
#pragma unroll 1
    for (int k = 0; k < 2; ++k) {
        const uint32_t r = t + PT * k;
        if (r >= p.S) continue;
        float b[32];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(p.Bp + (size_t)r * 32 + 4 * q);
            b[4 * q] = f.x; b[4 * q + 1] = f.y; b[4 * q + 2] = f.z; b[4 * q + 3] = f.w;
        }
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            b[kk] = newton_div(b[kk], Q[kk][kk]);
#pragma unroll
            for (int q = kk / 4; q < 8; ++q) {
                const float4 u4 = *reinterpret_cast<const float4*>(&Q[kk][4 * q]);
                if (4 * q + 0 > kk) b[4 * q + 0] = fmaf(-b[kk], u4.x, b[4 * q + 0]);
                if (4 * q + 1 > kk) b[4 * q + 1] = fmaf(-b[kk], u4.y, b[4 * q + 1]);
                if (4 * q + 2 > kk) b[4 * q + 2] = fmaf(-b[kk], u4.z, b[4 * q + 2]);
                if (4 * q + 3 > kk) b[4 * q + 3] = fmaf(-b[kk], u4.w, b[4 * q + 3]);
            }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(p.Bp + (size_t)r * 32 + 4 * q) =
                make_float4(b[4 * q], b[4 * q + 1], b[4 * q + 2], b[4 * q + 3]);
    }
    // T = -U S L1^-T, a row per lane: T L1^T = -U S forward over the columns
    if (t < 32) {
        const int i = t;
        float tr[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float a = -Q[i][c] * sgn[c];
#pragma unroll
            for (int k = 0; k < c; ++k) a = fmaf(-tr[k], Q[c][k], a);   // L1[c][k], k < c; tr[k] = 0 for k < i
            tr[c] = c >= i ? a : 0.0f;
        }
        const uint32_t jb = p.jb;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            p.t[i * 32 + c] = ((uint32_t)i < jb && (uint32_t)c < jb) ? tr[c] : 0.0f;
            if ((uint32_t)c < jb) {
                // Y's first 32 rows are L's (unit lower trapezoidal; for a panel narrower than 32 the
                // rows from jb on are ordinary rows of L)
                if ((uint32_t)i < p.mp) p.y[(size_t)i * p.ldy + c] = c < i ? Q[i][c] : (c == i ? 1.0f : 0.0f);
                if ((uint32_t)i < jb && c >= i) p.w[(size_t)i * p.ldw + c] = sgn[i] * Rm[i][c];
            }
        }
    }
}


// ---------------------------------------------------------------------------
// The leaf and the top with a column per lane (qr_panel_cols.cuh): blocks of 8 * RW rows.
// Same inputs and outputs as panel_leaf_kernel and panel_top_kernel.
// ---------------------------------------------------------------------------
template <int RW>
__global__ void __launch_bounds__(PT, 1) panel_leaf_cols_kernel(const LeafParams p) {
    dependency_wait();
    using namespace cols;
    __shared__ __align__(16) cols::Smem s;
    __shared__ __align__(16) float pub[kWarps * RW];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t blk = blockIdx.x, row0 = blk * p.lr + warp * RW;
    pair_t x2[RW / 2];
#pragma unroll
    for (int i = 0; i < RW / 2; ++i) {
        const uint32_t ra = row0 + 2 * i;
        float a = 0.0f, b = 0.0f;
        if ((uint32_t)lane < p.jb) {
            if (ra < p.mp) a = p.panel[(size_t)ra * p.ldw + lane];
            if (ra + 1 < p.mp) b = p.panel[(size_t)(ra + 1) * p.ldw + lane];
        }
        x2[i] = pack(a, b);
    }
    float my_sc;
    factor_cols<RW, false>(x2, s, pub, nullptr, my_sc);
    __syncthreads();
    build_t(s);
    if (warp == 0) {       // the first 32 rows: R for the stack, the reflectors with a unit diagonal
        float* dst = p.Sl + (size_t)blk * 1024 + lane;
        float* vdst = p.Vl + (size_t)blk * p.lr * 32 + lane;
#pragma unroll 4
        for (int r = 0; r < 32; ++r) {
            const float v = s.rows[r][lane];
            dst[r * 32]  = lane >= r ? v : 0.0f;
            vdst[r * 32] = r > lane ? v * my_sc : (r == lane ? 1.0f : 0.0f);
        }
    }
    {
        float* dst = p.Vl + ((size_t)blk * p.lr + warp * RW) * 32 + lane;
#pragma unroll
        for (int r = (RW > 32 ? 32 : RW); r < RW; ++r)       // warp 0's rows from 32 on (64 rows a lane)
            if (warp == 0) dst[r * 32] = row_of<RW>(x2, r) * my_sc;
#pragma unroll
        for (int r = 0; r < RW; ++r)
            if (warp != 0) dst[r * 32] = row_of<RW>(x2, r) * my_sc;
    }
    __syncthreads();
    for (int idx = t; idx < 1024; idx += PT) p.Tl[(size_t)blk * 1024 + idx] = s.T[idx >> 5][idx & 31];
}

template <int RW>
__global__ void __launch_bounds__(PT, 1) panel_top_cols_kernel(const TopParams p) {
    dependency_wait();
    using namespace cols;
    constexpr int kRows = kWarps * RW;
    extern __shared__ __align__(16) float Us[];          // [32][kRows]: the reflectors' tails in the rows from 32 on
    __shared__ __align__(16) cols::Smem s;
    __shared__ float V1[32][33], Mr[32][33];
    __shared__ __align__(16) float M4[32][36];           // read as 16-byte words
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    pair_t x2[RW / 2];
#pragma unroll
    for (int i = 0; i < RW / 2; ++i) {
        const uint32_t ra = warp * RW + 2 * i;
        const float a = ra < p.S ? p.Sl[(size_t)ra * 32 + lane] : 0.0f;
        const float b = ra + 1 < p.S ? p.Sl[(size_t)(ra + 1) * 32 + lane] : 0.0f;
        x2[i] = pack(a, b);
    }
    __shared__ __align__(16) float pub[RW];
    float my_sc;
    factor_cols<RW, true>(x2, s, pub, Us, my_sc);
    if (warp == 0 && RW > 32) {      // warp 0's rows from 32 on are not published into Us by the steps: their tails now
#pragma unroll
        for (int r = 32; r < RW; ++r) Us[(size_t)lane * kRows + r] = row_of<RW>(x2, r);
    }
    __syncthreads();
    build_t(s);
    if (warp == 0) {
#pragma unroll 4
        for (int r = 0; r < 32; ++r) {
            const float v = s.rows[r][lane];
            p.Rt[r * 32 + lane] = lane >= r ? v : 0.0f;
            V1[r][lane] = r > lane ? v * my_sc : (r == lane ? 1.0f : 0.0f);
        }
    }
    __syncthreads();
    // The top Q's rows, B = [I; 0] - V (T V1^T) with V the unit-diagonal reflectors: V = [I; 0] +
    // (tails) diag(sc), so B = [I - M; 0] - (tails) (diag(sc) M), M = T V1^T.
    {
        const int i = t >> 3, c0 = (t & 7) * 4;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const float a = s.T[i][k];
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(a, V1[c0 + e][k], acc[e]);
        }
        const float sci = s.sc[i];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            Mr[i][c0 + e] = acc[e];
            M4[i][c0 + e] = acc[e] * sci;
        }
    }
    __syncthreads();
#pragma unroll 1
    for (uint32_t row = t; row < p.S; row += PT) {      // a row of B per thread and pass
        float b[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) b[c] = (row == (uint32_t)c ? 1.0f : 0.0f) - (row < 32 ? Mr[row][c] : 0.0f);
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            const float v = row < 32 ? ((uint32_t)kk < row ? s.rows[row][kk] : 0.0f) : Us[kk * kRows + row];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 m4 = *reinterpret_cast<const float4*>(&M4[kk][4 * q]);
                b[4 * q] = fmaf(-v, m4.x, b[4 * q]); b[4 * q + 1] = fmaf(-v, m4.y, b[4 * q + 1]);
                b[4 * q + 2] = fmaf(-v, m4.z, b[4 * q + 2]); b[4 * q + 3] = fmaf(-v, m4.w, b[4 * q + 3]);
            }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(p.Bp + (size_t)row * 32 + 4 * q) =
                make_float4(b[4 * q], b[4 * q + 1], b[4 * q + 2], b[4 * q + 3]);
    }
}


// ---------------------------------------------------------------------------
// The whole panel in ONE launch: a thread-block cluster whose blocks hold 8 * RW rows each, the
// column steps' sums exchanged through distributed shared memory (cols::ClusterSync). This is
// LAPACK's own Householder panel (no row blocks, no tree, no reconstruction): out come R (into the
// working copy's upper triangle), Y with its unit diagonal, and T. Up to 8 blocks of 512 rows
// (4096 rows) with the portable cluster size, 16 blocks (8192 rows) with the non-portable one.
// ---------------------------------------------------------------------------
struct ClusterPanelParams {
    float*   panel;     // the panel's first entry in the working copy: in the panel, out R
    size_t   ldw;
    float*   y;         // the panel's first entry in Y
    size_t   ldy;
    float*   t;         // [32][32] out
    uint32_t mp, jb;
    int      pairs;     // 1: two columns a reduction (factor_cols2); 2: four (factor_cols4); 0: one
    int      post;      // four columns a reduction: the sums posted to mbarriers (cols::ClusterSync::post)
    unsigned* bad;      // where a wait that ran out is recorded (may be null)
};

// MODE: the columns a reduction (0: one, 1: two, 2: four), a kernel each: one kernel holding all three was larger and
// slower on every path.
template <int RW, int MODE>
__global__ void __launch_bounds__(PT, 1) panel_cluster_kernel(const ClusterPanelParams p) {
    using namespace cols;
    dependency_wait();
    __shared__ __align__(16) cols::Smem s;
    __shared__ __align__(16) cols::ClusterShared cs;
    __shared__ __align__(16) float pub[2 * kWarps * RW];
    extern __shared__ __align__(16) unsigned char quad_raw[];      // four columns a reduction: QuadShared, then 4 * kWarps * RW floats
    QuadShared* qs = reinterpret_cast<QuadShared*>(quad_raw);
    if constexpr (MODE == 2) {
        if (threadIdx.x == 0) ClusterSync::init_posts(qs);
    }
    // every block of the cluster must be running (and its mbarriers set up) before any writes into another's shared
    // memory: arrive now, wait after the loads, which hide the barrier's latency
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    float* pub4 = reinterpret_cast<float*>(quad_raw + sizeof(QuadShared));
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t rank = cluster_rank(), ncta = cluster_size();
    const uint32_t row0 = (rank * kWarps + warp) * RW;
    pair_t x2[RW / 2];
#pragma unroll
    for (int i = 0; i < RW / 2; ++i) {
        const uint32_t ra = row0 + 2 * i;
        float a = 0.0f, b = 0.0f;
        if ((uint32_t)lane < p.jb) {
            if (ra < p.mp) a = p.panel[(size_t)ra * p.ldw + lane];
            if (ra + 1 < p.mp) b = p.panel[(size_t)(ra + 1) * p.ldw + lane];
        }
        x2[i] = pack(a, b);
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    float my_sc;
    if constexpr (MODE == 2) factor_cols4<RW>(x2, s, pub4, my_sc, ClusterSync{rank, ncta, &cs, qs, p.post, p.bad});
    else if constexpr (MODE == 1) factor_cols2<RW, ClusterSync, RW == 32>(x2, s, pub, my_sc, ClusterSync{rank, ncta, &cs});      // 32 rows a lane leave the registers for it
    else factor_cols<RW, false>(x2, s, pub, nullptr, my_sc, ClusterSync{rank, ncta, &cs});
    __syncthreads();
    // T straight to global memory by the warp that recorded tau and G; rows and columns from jb on are zero (their
    // reflectors are the identity). Meanwhile block 0's first warp writes R and the other warps Y.
    if (rank + 1 == ncta && warp == kWarps - 1) build_t_to(s, p.t, 32);
    if (rank == 0 && warp == 0) {
        // the first 32 rows: R into the working copy, the reflectors with a unit diagonal into Y
#pragma unroll 4
        for (int r = 0; r < 32; ++r) {
            const float v = s.rows[r][lane];
            if ((uint32_t)lane < p.jb && (uint32_t)r < p.mp) {
                if (lane >= r) p.panel[(size_t)r * p.ldw + lane] = v;
                p.y[(size_t)r * p.ldy + lane] = r > lane ? v * my_sc : (r == lane ? 1.0f : 0.0f);
            }
        }
    }
    if ((uint32_t)lane < p.jb) {
        const bool first = rank == 0 && warp == 0;       // its rows below 32 (64 rows a lane) are ordinary rows
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const uint32_t row = row0 + r;
            if ((!first || r >= 32) && row < p.mp) p.y[(size_t)row * p.ldy + lane] = row_of<RW>(x2, r) * my_sc;
        }
    }
    // (The last write into another block's shared memory was before the last step's cluster barrier: a block may
    // leave as soon as its own stores are done.)
}

struct ApplyParams {
    const float* Vl;        // [leaves][lr][32]
    const float* Tl;        // [leaves][32][32]
    const float* Bp;        // [leaves * 32][32]
    float*       y;         // the panel's first entry in Y
    size_t       ldy;
    uint32_t     mp, jb, lr;
};

template <int RPT>
__global__ void __launch_bounds__(PT) panel_apply_kernel(const ApplyParams p) {
    dependency_wait();
    __shared__ float Vt[32][33], Ti[32][33], Bi[32][33], X[32][33], M[32][33];
    const int t = threadIdx.x;
    const uint32_t blk = blockIdx.x;
    for (int idx = t; idx < 1024; idx += PT) {
        Vt[idx >> 5][idx & 31] = p.Vl[(size_t)blk * p.lr * 32 + idx];
        Ti[idx >> 5][idx & 31] = p.Tl[(size_t)blk * 1024 + idx];
        Bi[idx >> 5][idx & 31] = p.Bp[(size_t)blk * 1024 + idx];
    }
    __syncthreads();
    mat32<true>(Vt, Bi, X);
    __syncthreads();
    mat32<false>(Ti, X, M);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
        const uint32_t row = t + PT * k, gr = blk * p.lr + row;
        if (gr >= p.mp || (blk == 0 && row < 32)) continue;   // the first 32 rows are L1, written by the top kernel
        const float* vsrc = p.Vl + ((size_t)blk * p.lr + row) * 32;
        float v[32], yv[32];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(vsrc + 4 * q);
            v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) yv[c] = row < 32 ? Bi[row][c] : 0.0f;
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
#pragma unroll
            for (int c = 0; c < 32; ++c) yv[c] = fmaf(-v[kk], M[kk][c], yv[c]);
        }
        float* dst = p.y + (size_t)gr * p.ldy;
        if (p.jb == 32 && (p.ldy & 3) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(yv[4 * q], yv[4 * q + 1], yv[4 * q + 2], yv[4 * q + 3]);
        } else {
#pragma unroll
            for (int c = 0; c < 32; ++c)
                if ((uint32_t)c < p.jb) dst[c] = yv[c];
        }
    }
}

int rows_per_thread(uint32_t mp) { return mp <= 2048 ? 1 : mp <= 8192 ? 2 : 4; }

} // namespace

bool panel_fast_fits(uint32_t mp, uint32_t jb) { return jb >= 1 && jb <= 32 && mp >= jb && mp <= 16384; }

size_t panel_fast_workspace_floats(uint32_t mp) {
    const uint32_t lr = PT * rows_per_thread(mp), leaves = (mp + lr - 1) / lr;
    return (size_t)leaves * lr * 32 + (size_t)leaves * 1024 * 3 + 1024 + 256;
}

// The panel at `panel` (mp x jb, row stride ldw, inside the working copy) to compact-WY form: its R
// (S R) into the working copy's upper triangle, Y into `y` (row stride ldy), T into t[32][32].
void panel_factor_fast(cudaStream_t stream, float* panel, size_t ldw, uint32_t mp, uint32_t jb, float* y, size_t ldy,
                       float* t, float* ws, unsigned* bad) {
    const int rpt = rows_per_thread(mp);
    const uint32_t lr = PT * rpt, leaves = (mp + lr - 1) / lr;
    float* Vl = ws;
    float* Tl = Vl + (size_t)leaves * lr * 32;
    float* Sl = Tl + (size_t)leaves * 1024;
    float* Bp = Sl + (size_t)leaves * 1024;
    float* Rt = Bp + (size_t)leaves * 1024;
    // a column per lane up to 8192 rows; a row per thread beyond, and for both with QR_PANEL_ROWS=1
    const char* env = std::getenv("QR_PANEL_ROWS");
    const bool by_columns = rpt <= 2 && !(env && env[0] == '1');
    // up to 8192 rows the whole panel in one cluster launch (QR_PANEL_CLUSTER=0: the tree of row blocks)
    const char* envc = std::getenv("QR_PANEL_CLUSTER");
    // panels of 4097 to 8192 rows: a cluster of sixteen blocks of 512 rows (the non-portable size). With two columns a
    // reduction it beats the tree of row blocks there (8192 x 8192: 35.3 -> 32.6 ms); QR_PANEL_CLUSTER=4096 keeps the tree
    const bool tall_cluster = !(envc && envc[0] == '4');
    if (by_columns && (mp <= 4096 || (tall_cluster && mp <= 8192)) && !(envc && envc[0] == '0')) {
        // 2049 to 4096 rows: sixteen blocks of 256 rows (32 rows a lane: half the arithmetic and half the shared-memory
        // reads a step, and registers left to keep the published columns from the products to the update; a cluster of
        // the non-portable size), or with QR_PANEL_CLUSTER=8 eight blocks of 512 rows (4096 x 4096: 7.67 against 7.86 ms)
        const bool sixteen = mp > 2048 && mp <= 4096 && !(envc && envc[0] == '8');
        const uint32_t rw = (mp <= 2048 || sixteen) ? 32 : 64;
        uint32_t ncta = 1;
        while (ncta * 8 * rw < mp) ncta *= 2;       // 1, 2, 4, 8 (or 16) blocks; blocks beyond the rows hold zeros
        {
            static PerDeviceOnce once;      // per GPU: the four-column kernels' static and dynamic shared memory together pass the
                                            // 48 KB that need no opt-in; sixteen blocks are a cluster of the non-portable size
            if (const int device = current_device(); once.first(device)) {
                cuda_check(cudaFuncSetAttribute(panel_cluster_kernel<32, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)(sizeof(cols::QuadShared) + 4 * cols::kWarps * 32 * sizeof(float))), "panel_cluster shared memory");
                cuda_check(cudaFuncSetAttribute(panel_cluster_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)(sizeof(cols::QuadShared) + 4 * cols::kWarps * 64 * sizeof(float))), "panel_cluster shared memory");
                const auto big = [](auto kernel) {
                    cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1),
                               "panel_cluster non-portable cluster size");
                };
                big(panel_cluster_kernel<32, 0>); big(panel_cluster_kernel<32, 1>); big(panel_cluster_kernel<32, 2>);
                big(panel_cluster_kernel<64, 0>); big(panel_cluster_kernel<64, 1>); big(panel_cluster_kernel<64, 2>);
                once.mark(device);
            }
        }
        // four columns a reduction (QR_PANEL_QUADS=0: two; QR_PANEL_PAIRS=0: one)
        const char* envp = std::getenv("QR_PANEL_PAIRS");
        const char* envq = std::getenv("QR_PANEL_QUADS");
        const int pairs = (envp && envp[0] == '0') ? 0 : (envq && envq[0] == '0') ? 1 : 2;
        // the sums of four columns posted to mbarriers (QR_PANEL_POST=0: stored, then the cluster's barrier)
        const char* envs = std::getenv("QR_PANEL_POST");
        ClusterPanelParams cp{panel, ldw, y, ldy, t, mp, jb, pairs, !(envs && envs[0] == '0'), bad};
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(ncta);
        cfg.blockDim = dim3(PT);
        cfg.dynamicSmemBytes = pairs == 2 ? sizeof(cols::QuadShared) + 4 * cols::kWarps * rw * sizeof(float) : 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = ncta;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = dependent_launches_enabled() ? 2 : 1;
        using Kernel = void (*)(ClusterPanelParams);
        static const Kernel kernels[2][3] = {{panel_cluster_kernel<32, 0>, panel_cluster_kernel<32, 1>, panel_cluster_kernel<32, 2>},
                                             {panel_cluster_kernel<64, 0>, panel_cluster_kernel<64, 1>, panel_cluster_kernel<64, 2>}};
        cuda_check(cudaLaunchKernelEx(&cfg, kernels[rw == 64][pairs], cp), "panel_cluster launch");
        return;
    }
    LeafParams lp{panel, ldw, mp, jb, lr, Vl, Tl, Sl};
    TopParams tp{Sl, leaves * 32, Vl, Tl, Bp, panel, ldw, y, ldy, t, jb, mp, Rt};
    if (by_columns) {
        static PerDeviceOnce once;      // the opt-in is recorded per GPU
        if (const int device = current_device(); once.first(device)) {
            // static and dynamic shared memory together pass the 48 KB that need no opt-in
            cuda_check(cudaFuncSetAttribute(panel_top_cols_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            32 * 256 * (int)sizeof(float)), "panel_top_cols shared memory");
            cuda_check(cudaFuncSetAttribute(panel_top_cols_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            32 * 512 * (int)sizeof(float)), "panel_top_cols shared memory");
            once.mark(device);
        }
        if (rpt == 1) launch_dependent(panel_leaf_cols_kernel<32>, leaves, PT, 0, stream, lp);
        else launch_dependent(panel_leaf_cols_kernel<64>, leaves, PT, 0, stream, lp);
        if (leaves * 32 <= PT) launch_dependent(panel_top_cols_kernel<32>, 1, PT, 32 * 256 * sizeof(float), stream, tp);
        else launch_dependent(panel_top_cols_kernel<64>, 1, PT, 32 * 512 * sizeof(float), stream, tp);
    } else {
        if (rpt == 1) launch_dependent(panel_leaf_kernel<1>, leaves, PT, 0, stream, lp);
        else if (rpt == 2) launch_dependent(panel_leaf_kernel<2>, leaves, PT, 0, stream, lp);
        else launch_dependent(panel_leaf_kernel<4>, leaves, PT, 0, stream, lp);
        if (leaves * 32 <= PT) launch_dependent(panel_top_kernel<1>, 1, PT, 0, stream, tp);
        else launch_dependent(panel_top_kernel<2>, 1, PT, 0, stream, tp);
    }
    launch_dependent(panel_finish_kernel, 1, PT, 0, stream, tp);
    ApplyParams ap{Vl, Tl, Bp, y, ldy, mp, jb, lr};
    if (rpt == 1) launch_dependent(panel_apply_kernel<1>, leaves, PT, 0, stream, ap);
    else if (rpt == 2) launch_dependent(panel_apply_kernel<2>, leaves, PT, 0, stream, ap);
    else launch_dependent(panel_apply_kernel<4>, leaves, PT, 0, stream, ap);
    cuda_check(cudaGetLastError(), "panel launch");
}

} // namespace mlb
