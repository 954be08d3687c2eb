// The mid-size kernel: one thread block per matrix, up to 1024 rows and any
// number of columns; LAPACK's blocked method (sgeqrf + sorgqr with compact-WY
// block reflectors, panels of 32 columns).
//
// It takes the place of the reference's threadgroup-per-matrix kernel
// qr_householder_wy (shaders/QR_Householder.metal:665-847; host side
// src/qr_householder.mm:128-164,293-381) and keeps its contract: scan + power-
// of-two scaling per matrix, non-finite matrix -> NaN outputs, slarfg signs, R
// with exact zeros below the diagonal, Q formed backward from [I; 0].
//
// Layout. The grid is persistent: gridDim.x blocks (as many as are resident at
// once) each loop over matrices, and each owns one scratch slot in global
// memory holding its current matrix (row-major, in the scaled domain) and the
// panels' T factors. A slot is rewritten for every matrix a block takes, so the
// slots (a few hundred KB each) live in the 126 MB L2 and the HBM traffic of a
// matrix is its input once and its outputs once.
//
// Per panel: the panel's rows are brought into shared memory column-major
// (leading dimension = 4 mod 32 floats, so that four consecutive rows of a
// column are one aligned 16-byte word and eight columns' words tile the 32
// banks), factored there one column per step with one barrier a step (a warp
// owns the columns it updates, so a dot product and its update need no
// barrier between them), T is built from the Gram matrix V^T V, and the
// trailing columns are updated tile by tile (32 columns x up to 256 rows in
// shared memory) as C -= V (T^T (V^T C)) with register-tiled FP32 FMA loops
// reading 16-byte words. Q formation runs the same tile update backward over
// the panels on the output buffer itself.
#include "common.cuh"
#include "kernels.h"
#include "qr_panel_cols.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <string>

namespace mlb {

namespace {

constexpr int NT  = 256;    // threads per block
constexpr int JB  = 32;     // panel width
constexpr int RC  = 256;    // rows of a trailing tile held in shared memory at once
constexpr int LDC = RC + 4; // its leading dimension
constexpr int LDZ = 36;     // leading dimension of the 32 x 32 blocks (T, Z, W)

struct MidParams {
    const float* a;
    float*       q;
    float*       r;
    float*       ws;            // gridDim.x slots of slot_floats
    uint32_t     batch;
    int          m, n, K, qc, rr;
    int          lda;
    unsigned long long a_stride, q_stride, r_stride, slot_floats;
    int          scale;
    int          ldv;
    int          npanels;
    int          by_columns;   // panels of at most 256 rows factored with a column per lane
    int          pairs;        // ... and two columns a reduction (factor_cols2)
    // matrix index -> (outer, inner) = (mat / inner_count, mat % inner_count) when inner_count > 0:
    // the matrix's buffers then start at outer * *_outer + inner * *_stride
    unsigned     inner_count;
    unsigned long long a_outer, q_outer, r_outer;
};

struct Smem {
    float* Vs;      // [32][ldv]   the panel / V, column-major
    float* Cs;      // [32][LDC]   a trailing tile, column-major
    float* Zp;      // [4][32][LDZ] partial V^T C of the four row groups
    float* Zs;      // [32][LDZ]   V^T C
    float* Ws;      // [32][LDZ]   op(T) V^T C
    float* Ts;      // [32][LDZ]   T
    float* taus;    // [32]
    float* scs;     // [32]
    float* betas;   // [32]
    float* colss;   // [32]
    float* red;     // [32] reductions
};

__device__ __forceinline__ Smem carve(float* base, int ldv) {
    Smem s;
    s.Vs = base;
    s.Cs = s.Vs + JB * ldv;
    s.Zp = s.Cs + 32 * LDC;
    s.Zs = s.Zp + 4 * 32 * LDZ;
    s.Ws = s.Zs + 32 * LDZ;
    s.Ts = s.Ws + 32 * LDZ;
    s.taus = s.Ts + 32 * LDZ;
    s.scs = s.taus + 32;
    s.betas = s.scs + 32;
    s.colss = s.betas + 32;
    s.red = s.colss + 32;
    return s;
}

size_t smem_bytes(int ldv) {
    return (size_t)(JB * ldv + 32 * LDC + 4 * 32 * LDZ + 3 * 32 * LDZ + 5 * 32) * sizeof(float);
}

// How an element read from global memory enters shared memory.
struct LoadPlain {
    __device__ __forceinline__ float operator()(float v, int, int) const { return v; }
};
struct LoadScaled {
    Pow2 down;
    __device__ __forceinline__ float operator()(float v, int, int) const { return down(v); }
};
// a factored panel read as its reflectors: the entries below the diagonal, a unit diagonal, zeros above
struct LoadReflector {
    __device__ __forceinline__ float operator()(float v, int r, int c) const { return r > c ? v : (r == c ? 1.0f : 0.0f); }
};

// Rows [row0, row0 + nrows) x columns [col0, col0 + ncols) of a row-major matrix
// into dst[c * lds + r], all 32 columns and rows up to the next multiple of four
// written (zeros outside). A warp reads 32 consecutive floats of four rows and
// writes one 16-byte word a lane.
//
// In two halves, so that a caller can have the next tile's loads in flight while it computes on the current one:
// tile_fetch issues the loads of up to 256 rows into registers (a warp's row quads are 8 apart: eight of them, all in
// flight together, so that a tile costs one trip to L2 and not eight), tile_commit writes them to shared memory.
struct TileRegs {
    float4 v[8];
};
__device__ __forceinline__ void tile_fetch(TileRegs& t, const float* src, size_t ld, int row0, int nrows, int col0,
                                           int ncols, int quad0) {
    const int warp = threadIdx.x >> 5, c = threadIdx.x & 31;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int r = (quad0 + warp + u * (NT / 32)) * 4;
        t.v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < ncols && r < nrows) {
            const float* s = src + (size_t)(row0 + r) * ld + col0 + c;
            t.v[u].x = s[0];
            if (r + 1 < nrows) t.v[u].y = s[ld];
            if (r + 2 < nrows) t.v[u].z = s[2 * ld];
            if (r + 3 < nrows) t.v[u].w = s[3 * ld];
        }
    }
}
template <class F>
__device__ __forceinline__ void tile_commit(const TileRegs& t, float* dst, int lds, int nrows, int ncols, int quad0, const F& f) {
    const int warp = threadIdx.x >> 5, c = threadIdx.x & 31;
    const int nq = (nrows + 3) >> 2;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int rq = quad0 + warp + u * (NT / 32), r = rq * 4;
        if (rq < nq) {
            float4 w = t.v[u];
            if (c < ncols) {
                w.x = f(w.x, r, c);
                if (r + 1 < nrows) w.y = f(w.y, r + 1, c);
                if (r + 2 < nrows) w.z = f(w.z, r + 2, c);
                if (r + 3 < nrows) w.w = f(w.w, r + 3, c);
            }
            *reinterpret_cast<float4*>(dst + c * lds + r) = w;
        }
    }
}
template <class F>
__device__ __forceinline__ void load_tile(float* dst, int lds, const float* src, size_t ld, int row0, int nrows,
                                          int col0, int ncols, const F& f) {
    const int nq = (nrows + 3) >> 2;
    for (int quad0 = 0; quad0 < nq; quad0 += 8 * (NT / 32)) {
        TileRegs t;
        tile_fetch(t, src, ld, row0, nrows, col0, ncols, quad0);
        tile_commit(t, dst, lds, nrows, ncols, quad0, f);
    }
}

// The reverse: src[c * lds + r] to rows [row0, row0 + nrows) x columns [col0, col0 + ncols).
__device__ __forceinline__ void store_tile(const float* src, int lds, float* dst, size_t ld, int row0, int nrows,
                                           int col0, int ncols) {
    const int warp = threadIdx.x >> 5, c = threadIdx.x & 31;
    const int nq = (nrows + 3) >> 2;
    if (c >= ncols) return;
    for (int rq = warp; rq < nq; rq += NT / 32) {
        const int r = rq * 4;
        const float4 v = *reinterpret_cast<const float4*>(src + c * lds + r);
        float* d = dst + (size_t)(row0 + r) * ld + col0 + c;
        if (r + 0 < nrows) d[0] = v.x;
        if (r + 1 < nrows) d[ld] = v.y;
        if (r + 2 < nrows) d[2 * ld] = v.z;
        if (r + 3 < nrows) d[3 * ld] = v.w;
    }
}

// acc[a][b] += sum over the rows of this thread's row group of V[i][r] C[c][r],
// i = ti + 8a, c = tc + 8b. V rows start at vbase (already offset to the tile's
// first row), C at cbase; nq row quads.
__device__ __forceinline__ void gemm_vtc(float (&acc)[4][4], const float* vbase, int ldv, const float* cbase,
                                         int ldc, int nq) {
    const int ti = threadIdx.x & 7, tc = (threadIdx.x >> 3) & 7, tr = threadIdx.x >> 6;
    for (int rq = tr; rq < nq; rq += 4) {
        float4 v[4], c[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) v[a] = *reinterpret_cast<const float4*>(vbase + (ti + 8 * a) * ldv + 4 * rq);
#pragma unroll
        for (int b = 0; b < 4; ++b) c[b] = *reinterpret_cast<const float4*>(cbase + (tc + 8 * b) * ldc + 4 * rq);
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                acc[a][b] = fmaf(v[a].x, c[b].x, acc[a][b]);
                acc[a][b] = fmaf(v[a].y, c[b].y, acc[a][b]);
                acc[a][b] = fmaf(v[a].z, c[b].z, acc[a][b]);
                acc[a][b] = fmaf(v[a].w, c[b].w, acc[a][b]);
            }
    }
}

// The four row groups' partial sums into Zp, then (after the caller's barrier)
// summed into Zs.
__device__ __forceinline__ void put_partials(const float (&acc)[4][4], float* Zp) {
    const int ti = threadIdx.x & 7, tc = (threadIdx.x >> 3) & 7, tr = threadIdx.x >> 6;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) Zp[(tr * 32 + ti + 8 * a) * LDZ + tc + 8 * b] = acc[a][b];
}
__device__ __forceinline__ void sum_partials(const float* Zp, float* Zs) {
    const int i = threadIdx.x >> 3, cq = threadIdx.x & 7;
    float4 s = *reinterpret_cast<const float4*>(Zp + i * LDZ + 4 * cq);
#pragma unroll
    for (int g = 1; g < 4; ++g) {
        const float4 t = *reinterpret_cast<const float4*>(Zp + (g * 32 + i) * LDZ + 4 * cq);
        s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    *reinterpret_cast<float4*>(Zs + i * LDZ + 4 * cq) = s;
}

// Ws = T^T Zs (transposed) or T Zs.
__device__ __forceinline__ void apply_t(const float* Ts, const float* Zs, float* Ws, bool transposed) {
    const int i = threadIdx.x >> 3, cq = threadIdx.x & 7;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
        const float t = transposed ? Ts[k * LDZ + i] : Ts[i * LDZ + k];
        const float4 z = *reinterpret_cast<const float4*>(Zs + k * LDZ + 4 * cq);
        s.x = fmaf(t, z.x, s.x); s.y = fmaf(t, z.y, s.y); s.z = fmaf(t, z.z, s.z); s.w = fmaf(t, z.w, s.w);
    }
    *reinterpret_cast<float4*>(Ws + i * LDZ + 4 * cq) = s;
}

// C[c][r] -= sum_i V[i][r] W[i][c] on nq row quads, in place in shared memory.
__device__ __forceinline__ void gemm_vw(const float* vbase, int ldv, const float* Ws, float* cbase, int ldc, int nq) {
    const int trq = threadIdx.x & 7;
    const int tcq = ((threadIdx.x >> 3) & 3) + 4 * ((threadIdx.x >> 5) & 1);
    const int trb = threadIdx.x >> 6;
    for (int rq = trq + 8 * trb; rq < nq; rq += 32) {
        ulonglong2 cp[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) cp[b] = *reinterpret_cast<const ulonglong2*>(cbase + (4 * tcq + b) * ldc + 4 * rq);
#pragma unroll 8
        for (int i = 0; i < 32; ++i) {
            const float4 v = *reinterpret_cast<const float4*>(vbase + i * ldv + 4 * rq);
            const float4 w = *reinterpret_cast<const float4*>(Ws + i * LDZ + 4 * tcq);
            // packed: rows (x, y) and (z, w) of V's word are pairs as they lie; W's entry goes into both halves, negated
            const ulonglong2 vv = *reinterpret_cast<const ulonglong2*>(&v);
            const small::pair_t w0 = small::pack(-w.x, -w.x), w1 = small::pack(-w.y, -w.y), w2 = small::pack(-w.z, -w.z),
                                w3 = small::pack(-w.w, -w.w);
            cp[0].x = small::fma2(vv.x, w0, cp[0].x); cp[0].y = small::fma2(vv.y, w0, cp[0].y);
            cp[1].x = small::fma2(vv.x, w1, cp[1].x); cp[1].y = small::fma2(vv.y, w1, cp[1].y);
            cp[2].x = small::fma2(vv.x, w2, cp[2].x); cp[2].y = small::fma2(vv.y, w2, cp[2].y);
            cp[3].x = small::fma2(vv.x, w3, cp[3].x); cp[3].y = small::fma2(vv.y, w3, cp[3].y);
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) *reinterpret_cast<ulonglong2*>(cbase + (4 * tcq + b) * ldc + 4 * rq) = cp[b];
    }
}

// dst[row0 + r][c] (columns [col_begin, col_end), rows row0 .. row0 + mp) <-
// (I - V op(T) V^T) src[same], 32 columns at a time. V is in s.Vs (mp rows), T
// in s.Ts. src and dst may be the same matrix.
template <class F>
__device__ void update_columns(const Smem& s, int ldv, const float* src, size_t lds, const F& f, float* dst,
                               size_t ldd, int row0, int mp, int col_begin, int col_end, bool transposed) {
    // A matrix of at most 256 rows has one tile a strip: the next strip's tile is then asked into L1 (a row of a tile
    // is one 128-byte line, a line a thread) while this strip's second product runs.
    const bool single = mp <= RC;
    for (int c0 = col_begin; c0 < col_end; c0 += 32) {
        const int tw = min(32, col_end - c0);
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
        for (int r0 = 0; r0 < mp; r0 += RC) {
            const int nr = min(RC, mp - r0);
            __syncthreads();   // the tile buffer is free
            load_tile(s.Cs, LDC, src, lds, row0 + r0, nr, c0, tw, f);
            __syncthreads();
            gemm_vtc(acc, s.Vs + r0, ldv, s.Cs, LDC, (nr + 3) >> 2);
        }
        put_partials(acc, s.Zp);
        __syncthreads();
        sum_partials(s.Zp, s.Zs);
        __syncthreads();
        apply_t(s.Ts, s.Zs, s.Ws, transposed);
        __syncthreads();
        if (single && c0 + 32 < col_end && (int)threadIdx.x < mp)
            asm volatile("prefetch.global.L1 [%0];" :: "l"(src + (size_t)(row0 + threadIdx.x) * lds + c0 + 32));
        for (int r0 = 0; r0 < mp; r0 += RC) {
            const int nr = min(RC, mp - r0);
            if (!single) {
                __syncthreads();
                load_tile(s.Cs, LDC, src, lds, row0 + r0, nr, c0, tw, f);
                __syncthreads();
            }
            gemm_vw(s.Vs + r0, ldv, s.Ws, s.Cs, LDC, (nr + 3) >> 2);
            __syncthreads();
            store_tile(s.Cs, LDC, dst, ldd, row0 + r0, nr, c0, tw);
        }
    }
    __syncthreads();
}

// Factors the panel in s.Vs (mp rows, jb columns) in place: afterwards column c
// holds R's entries above the diagonal, the reflector's unscaled tail below it;
// betas, taus, scs per column.
__device__ void factor_panel(const Smem& s, int ldv, int mp, int jb) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        float ss = 0.0f;
        for (int r = 1 + lane; r < mp; r += 32) ss = fmaf(s.Vs[r], s.Vs[r], ss);
        ss = warp_sum(ss);
        if (lane == 0) s.colss[0] = ss;
    }
    if (threadIdx.x < 32) {
        s.taus[threadIdx.x] = 0.0f;
        s.scs[threadIdx.x] = 0.0f;
        s.betas[threadIdx.x] = 0.0f;
    }
    __syncthreads();
    for (int j = 0; j < jb; ++j) {
        const float* vj = s.Vs + j * ldv;
        float beta, tau, sc;
        reflector(vj[j], s.colss[j], beta, tau, sc);
        if (threadIdx.x == 0) {
            s.taus[j] = tau;
            s.scs[j] = sc;
            s.betas[j] = beta;
        }
        for (int c = j + 1 + warp; c < jb; c += NT / 32) {
            float* xc = s.Vs + c * ldv;
            float  d = 0.0f;
            for (int r = j + 1 + lane; r < mp; r += 32) d = fmaf(vj[r], xc[r], d);
            d = warp_sum(d);
            const float head = xc[j];
            const float w = tau * fmaf(sc, d, head);
            const float ws = w * sc;
            float ss = 0.0f;
            for (int r = j + 1 + lane; r < mp; r += 32) {
                const float x = fmaf(-ws, vj[r], xc[r]);
                xc[r] = x;
                if (r > j + 1) ss = fmaf(x, x, ss);
            }
            __syncwarp();
            if (lane == 0) xc[j] = head - w;
            if (c == j + 1) {
                ss = warp_sum(ss);
                if (lane == 0) s.colss[j + 1] = ss;
            }
        }
        __syncthreads();
    }
}

// After factor_panel: writes the factored panel to the scratch matrix (R above
// the diagonal, beta on it, the scaled reflector below) and leaves the clean V
// (unit diagonal, zeros above, columns from jb on zero) in s.Vs.
__device__ void finish_panel(const Smem& s, int ldv, int mp, int jb, float* W, size_t ldw, int k0) {
    const int warp = threadIdx.x >> 5, c = threadIdx.x & 31;
    const int nq = (mp + 3) >> 2;
    const float sc = s.scs[c], beta = s.betas[c];
    for (int rq = warp; rq < nq; rq += NT / 32) {
        const int r = rq * 4;
        float4 v = *reinterpret_cast<const float4*>(s.Vs + c * ldv + r);
        float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int rr = r + t;
            const float g = rr < c ? e[t] : (rr == c ? beta : e[t] * sc);
            if (c < jb && rr < mp) W[(size_t)(k0 + rr) * ldw + k0 + c] = g;
            e[t] = (c < jb && rr < mp) ? (rr < c ? 0.0f : (rr == c ? 1.0f : g)) : 0.0f;
        }
        *reinterpret_cast<float4*>(s.Vs + c * ldv + r) = make_float4(e[0], e[1], e[2], e[3]);
    }
    __syncthreads();
}

// T of the panel from its clean V in s.Vs: the Gram matrix into s.Zs, then
// slarft's forward recurrence by one warp, a row of T per lane.
__device__ void build_t(const Smem& s, int ldv, int mp) {
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
    gemm_vtc(acc, s.Vs, ldv, s.Vs, ldv, (mp + 3) >> 2);
    put_partials(acc, s.Zp);
    __syncthreads();
    sum_partials(s.Zp, s.Zs);
    __syncthreads();
    if (threadIdx.x < 32) {
        const int i = threadIdx.x;
        float t[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float tau = s.taus[j];
            float a = 0.0f;
#pragma unroll
            for (int k = 0; k < j; ++k) a = fmaf(t[k], s.Zs[k * LDZ + j], a);
            t[j] = i < j ? -tau * a : (i == j ? tau : 0.0f);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) s.Ts[i * LDZ + j] = t[j];
    }
    __syncthreads();
}

// The three steps above in one for a panel of at most 256 rows, with a column per lane
// (qr_panel_cols.cuh: the panel in the registers of the block, one barrier and no shuffle
// reduction a step; measured 4 times as fast as factor_panel on 256 rows). In: the panel in s.Vs.
// Out as finish_panel's and build_t's: the factored panel in the scratch matrix, the clean V in
// s.Vs, T in s.Ts. The trailing tile buffer and the partial-sum buffer serve as its scratch.
template <int RW>      // rows a lane: 32 (up to 256 rows) or 64 (up to 512)
__device__ void factor_panel_cols(const Smem& s, int ldv, int mp, int jb, float* W, size_t ldw, int k0, bool pairs) {
    using namespace cols;
    cols::Smem& cs = *reinterpret_cast<cols::Smem*>(s.Cs);
    static_assert(sizeof(cols::Smem) <= 32 * LDC * sizeof(float), "the tile buffer holds the panel scratch");
    float* pub = s.Zp;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nw = (mp + RW - 1) / RW;          // the warps that hold rows
    pair_t x2[RW / 2];
    float my_sc = 0.0f;
    if (warp < nw) {
#pragma unroll
        for (int q = 0; q < RW / 4; ++q) {
            const int row0 = warp * RW + 4 * q;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row0 < mp) v = *reinterpret_cast<const float4*>(s.Vs + lane * ldv + row0);
            x2[2 * q]     = pack(v.x, v.y);
            x2[2 * q + 1] = pack(v.z, v.w);
        }
        if (pairs) factor_cols2<RW>(x2, cs, pub, my_sc, BlockSync{nw});
        else factor_cols<RW, false>(x2, cs, pub, nullptr, my_sc, nw);
    }
    __syncthreads();
    if (warp == 0) build_t_to(cs, s.Ts, LDZ);
    if (warp < nw) {
#pragma unroll
        for (int q = 0; q < RW / 4; ++q) {
            float e[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int r = 4 * q + t, row = warp * RW + r;
                // the block's first 32 rows were retired to cs.rows by warp 0; every other row is still in registers
                const float raw = (warp == 0 && r < 32) ? cs.rows[r & 31][lane] : row_of<RW>(x2, r);
                const float g = row > lane ? raw * my_sc : raw;      // R, beta on the diagonal, the unit-diagonal reflector below
                const bool in = lane < jb && row < mp;
                if (in) W[(size_t)(k0 + row) * ldw + k0 + lane] = g;
                e[t] = in ? (row < lane ? 0.0f : (row == lane ? 1.0f : g)) : 0.0f;
            }
            // (a lane's last rows may lie beyond the column's end in shared memory: ldv follows the matrix's rows)
            if (warp * RW + 4 * q + 3 < ldv) *reinterpret_cast<float4*>(s.Vs + lane * ldv + warp * RW + 4 * q) = make_float4(e[0], e[1], e[2], e[3]);
        }
    }
    __syncthreads();
}

// PRW: the most rows a lane holds in a panel factored with a column per lane. The instantiation for 64 (panels
// of 257 to 512 rows) needs more registers than two blocks a multiprocessor leave and spills; it is launched
// only for matrices of 257 to 512 rows, where it still wins (512 x 512: 13.1 against 14.2 ms for 296 matrices),
// so that every other shape runs the instantiation for 32, which does not.
// MB: the blocks a multiprocessor the registers are held to. Beyond about 330 rows the shared memory leaves room for one
// block only, and holding the instantiation for 64 to two blocks' registers made it spill 2 KB a thread for nothing.
template <int PRW, int MB = 2>
__global__ void __launch_bounds__(NT, MB) qr_mid_kernel(const MidParams p) {
    extern __shared__ __align__(16) float smem_raw[];
    const Smem s = carve(smem_raw, p.ldv);
    const int m = p.m, n = p.n, K = p.K, ldv = p.ldv;
    float* W  = p.ws + (size_t)blockIdx.x * p.slot_floats;
    float* Tg = W + (((size_t)m * n + 3) & ~(size_t)3);

    for (uint32_t mat = blockIdx.x; mat < p.batch; mat += gridDim.x) {
        size_t oa = (size_t)mat * p.a_stride, oq = (size_t)mat * p.q_stride, orr = (size_t)mat * p.r_stride;
        if (p.inner_count) {
            const size_t outer = mat / p.inner_count, inner = mat % p.inner_count;
            oa = outer * p.a_outer + inner * p.a_stride;
            oq = outer * p.q_outer + inner * p.q_stride;
            orr = outer * p.r_outer + inner * p.r_stride;
        }
        const float* A = p.a + oa;
        float*       Q = p.qc ? p.q + oq : nullptr;
        float*       R = p.r + orr;

        // rows of A, the scratch matrix and R on 16-byte boundaries: the copy loops move 16 bytes a lane
        const bool vec4 = (n & 3) == 0 && (p.lda & 3) == 0 && ((reinterpret_cast<size_t>(A) | reinterpret_cast<size_t>(R)) & 15) == 0;
        // 0. scan: largest magnitude, non-finite entries
        int expo = 0;
        if (p.scale) {
            float amax = 0.0f;
            int   bad = 0;
            if (vec4) {      // 16 bytes a lane, sixteen rows in flight (the matrix comes from HBM: few round trips)
                constexpr int kFlight = 16;
                for (int i0 = threadIdx.x / 32; i0 < m; i0 += kFlight * (NT / 32))
                    for (int j = (threadIdx.x & 31) * 4; j < n; j += 128) {
                        float4 v[kFlight];
#pragma unroll
                        for (int u = 0; u < kFlight; ++u) {
                            const int i = i0 + u * (NT / 32);
                            v[u] = i < m ? *reinterpret_cast<const float4*>(A + (size_t)i * p.lda + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int u = 0; u < kFlight; ++u) {
                            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v[u].x), fabsf(v[u].y))), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
                            bad |= nonfinite(v[u].x) | nonfinite(v[u].y) | nonfinite(v[u].z) | nonfinite(v[u].w);
                        }
                    }
            } else {
                for (int i = threadIdx.x / 32; i < m; i += NT / 32)
                    for (int j = threadIdx.x & 31; j < n; j += 32) {
                        const float v = A[(size_t)i * p.lda + j];
                        amax = fmaxf(amax, fabsf(v));
                        bad |= nonfinite(v);
                    }
            }
            amax = warp_max(amax);
            bad = __any_sync(0xffffffffu, bad);
            __syncthreads();   // s.red is free (previous matrix done)
            if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = bad ? -1.0f : amax;
            __syncthreads();
            amax = 0.0f;
            bad = 0;
            for (int w = 0; w < NT / 32; ++w) {
                const float v = s.red[w];
                if (v < 0.0f) bad = 1; else amax = fmaxf(amax, v);
            }
            if (bad) {
                for (size_t i = threadIdx.x; i < (size_t)m * p.qc; i += NT) Q[i] = qnan();
                for (size_t i = threadIdx.x; i < (size_t)p.rr * n; i += NT) R[i] = qnan();
                continue;
            }
            expo = amax_exponent(amax);
        }
        const LoadScaled from_a{Pow2(-expo)};

        // 1. factor, panel by panel
        for (int pi = 0; pi < p.npanels; ++pi) {
            const int k0 = pi * JB, jb = min(JB, K - k0), mp = m - k0;
            __syncthreads();
            if (pi == 0) load_tile(s.Vs, ldv, A, p.lda, 0, mp, 0, jb, from_a);
            else         load_tile(s.Vs, ldv, W, n, k0, mp, k0, jb, LoadPlain{});
            __syncthreads();
            if (mp <= 256 && p.by_columns) {
                factor_panel_cols<32>(s, ldv, mp, jb, W, n, k0, p.pairs != 0);
            } else if (PRW == 64 && mp <= 512 && p.by_columns) {
                factor_panel_cols<PRW>(s, ldv, mp, jb, W, n, k0, p.pairs != 0);
            } else {
                factor_panel(s, ldv, mp, jb);
                finish_panel(s, ldv, mp, jb, W, n, k0);
                build_t(s, ldv, mp);
            }
            for (int i = threadIdx.x; i < 32 * 32; i += NT) Tg[(size_t)pi * 1024 + i] = s.Ts[(i >> 5) * LDZ + (i & 31)];
            if (k0 + jb < n) {
                if (pi == 0) update_columns(s, ldv, A, p.lda, from_a, W, n, 0, mp, jb, n, true);
                else         update_columns(s, ldv, W, n, LoadPlain{}, W, n, k0, mp, k0 + jb, n, true);
            }
        }
        __syncthreads();

        // 2. R, back in the caller's scale
        {
            const Pow2 up(expo);
            if (vec4) {
                for (int i0 = threadIdx.x / 32; i0 < p.rr; i0 += 4 * (NT / 32))
                    for (int j = (threadIdx.x & 31) * 4; j < n; j += 128) {
                        float4 v[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int i = i0 + u * (NT / 32);
                            v[u] = (i < K && j + 3 >= i) ? *reinterpret_cast<const float4*>(W + (size_t)i * n + j)
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int i = i0 + u * (NT / 32);
                            if (i >= p.rr) continue;
                            const bool in = i < K;
                            *reinterpret_cast<float4*>(R + (size_t)i * n + j) =
                                make_float4(in && j >= i ? up(v[u].x) : 0.0f, in && j + 1 >= i ? up(v[u].y) : 0.0f,
                                            in && j + 2 >= i ? up(v[u].z) : 0.0f, in && j + 3 >= i ? up(v[u].w) : 0.0f);
                        }
                    }
            } else {
                for (int i = threadIdx.x / 32; i < p.rr; i += NT / 32)
                    for (int j = threadIdx.x & 31; j < n; j += 32)
                        R[(size_t)i * n + j] = (i < K && j >= i) ? up(W[(size_t)i * n + j]) : 0.0f;
            }
        }
        if (!p.qc) continue;

        // 3. Q = H_0 ... H_{K-1} [I; 0], block reflectors applied backward
        const int qc = p.qc;
        if ((qc & 3) == 0 && (reinterpret_cast<size_t>(Q) & 15) == 0) {
            for (int i = threadIdx.x / 32; i < m; i += NT / 32)
                for (int j = (threadIdx.x & 31) * 4; j < qc; j += 128)
                    *reinterpret_cast<float4*>(Q + (size_t)i * qc + j) =
                        make_float4(i == j ? 1.0f : 0.0f, i == j + 1 ? 1.0f : 0.0f, i == j + 2 ? 1.0f : 0.0f, i == j + 3 ? 1.0f : 0.0f);
        } else {
            for (int i = threadIdx.x / 32; i < m; i += NT / 32)
                for (int j = threadIdx.x & 31; j < qc; j += 32) Q[(size_t)i * qc + j] = i == j ? 1.0f : 0.0f;
        }
        __syncthreads();
        for (int pi = p.npanels - 1; pi >= 0; --pi) {
            const int k0 = pi * JB, jb = min(JB, K - k0), mp = m - k0;
            __syncthreads();
            // the reflectors back from the scratch matrix (rows relative to the panel): unit diagonal, zeros above
            load_tile(s.Vs, ldv, W, n, k0, mp, k0, jb, LoadReflector{});
            for (int i = threadIdx.x; i < 32 * 32; i += NT) s.Ts[(i >> 5) * LDZ + (i & 31)] = Tg[(size_t)pi * 1024 + i];
            __syncthreads();
            update_columns(s, ldv, Q, qc, LoadPlain{}, Q, qc, k0, mp, k0, qc, false);
        }
    }
}

} // namespace

namespace {
// QR_MID_ROWS=1: every panel by factor_panel (a thread per row entry), for comparison and tests
int mid_by_columns() {
    const char* e = std::getenv("QR_MID_ROWS");
    return !(e && e[0] == '1');
}
// QR_PANEL_PAIRS=0: panels a column a reduction instead of two (here and in the blocked QR's cluster panels)
int mid_pairs() {
    const char* e = std::getenv("QR_PANEL_PAIRS");
    return !(e && e[0] == '0');
}
}

bool qr_mid_fits(const DeviceContext& ctx, uint32_t m, uint32_t n) {
    if (m == 0 || n == 0 || m > 1024) return false;
    const int ldv = (int)((m + 31) / 32) * 32 + 4;
    return smem_bytes(ldv) <= ctx.smem_optin && (uint64_t)m * n < ((uint64_t)1 << 31);
}

namespace {
using MidKernel = void (*)(MidParams);
MidKernel mid_kernel_for(uint32_t m) {
    if (!(m > 256 && m <= 512 && mid_by_columns())) return qr_mid_kernel<32>;
    // two blocks a multiprocessor only where their shared memory fits its 228 KB twice (1 KB a block is the system's)
    static const size_t fixed = [] {
        cudaFuncAttributes attr{};
        cuda_check(cudaFuncGetAttributes(&attr, qr_mid_kernel<64, 2>), "qr_mid attributes");
        return attr.sharedSizeBytes + 1024;
    }();
    const bool two = 2 * (smem_bytes((int)((m + 31) / 32) * 32 + 4) + fixed) <= 228 * 1024;
    return two ? qr_mid_kernel<64, 2> : qr_mid_kernel<64, 1>;
}
uint64_t slot_floats_of(uint32_t m, uint32_t n) {
    const uint32_t K = m < n ? m : n;
    return (((uint64_t)m * n + 3) & ~(uint64_t)3) + (uint64_t)((K + JB - 1) / JB) * 1024;
}
uint32_t slots_of(const DeviceContext& ctx, uint32_t m, uint32_t batch) {
    const size_t smem = smem_bytes((int)((m + 31) / 32) * 32 + 4);
    const MidKernel kernel = mid_kernel_for(m);
    cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
               "qr_mid shared memory");
    int per_sm = 0;
    cuda_check(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, NT, smem), "qr_mid occupancy");
    if (per_sm < 1) throw std::runtime_error("qr_mid: the matrix does not fit a thread block");
    return (uint32_t)std::min<uint64_t>(batch, (uint64_t)per_sm * ctx.sm_count);
}
}

size_t qr_mid_workspace_floats(const DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t batch) {
    if (batch == 0) return 0;
    return (size_t)slots_of(ctx, m, batch) * slot_floats_of(m, n);
}

void launch_qr_mid(DeviceContext& ctx, cudaStream_t stream, const QrProblem& pr, const MidOptions& o) {
    if (pr.batch == 0) return;
    MidParams p{};
    p.inner_count = o.inner_count;
    p.a_outer = o.a_outer; p.q_outer = o.q_outer; p.r_outer = o.r_outer;
    p.a = pr.a; p.q = pr.q; p.r = pr.r;
    p.batch = pr.batch;
    p.m = (int)pr.m; p.n = (int)pr.n; p.K = (int)qr_k(pr); p.qc = (int)pr.qc; p.rr = (int)pr.rr;
    p.lda = o.lda ? (int)o.lda : (int)pr.n;
    p.a_stride = o.a_stride ? o.a_stride : (uint64_t)pr.m * p.lda;
    p.q_stride = o.q_stride ? o.q_stride : (uint64_t)pr.m * pr.qc;
    p.r_stride = o.r_stride ? o.r_stride : (uint64_t)pr.rr * pr.n;
    p.scale = o.scale ? 1 : 0;
    p.ldv = (int)((pr.m + 31) / 32) * 32 + 4;
    p.npanels = (p.K + JB - 1) / JB;
    p.by_columns = mid_by_columns();
    p.pairs = mid_pairs();
    p.slot_floats = (((uint64_t)pr.m * pr.n + 3) & ~(uint64_t)3) + (uint64_t)p.npanels * 1024;

    const size_t smem = smem_bytes(p.ldv);
    const MidKernel kernel = mid_kernel_for(pr.m);
    cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
               "qr_mid shared memory");
    int per_sm = 0;
    cuda_check(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, NT, smem), "qr_mid occupancy");
    if (per_sm < 1) throw std::runtime_error("qr_mid: the matrix does not fit a thread block");
    const uint32_t slots = (uint32_t)std::min<uint64_t>(pr.batch, (uint64_t)per_sm * ctx.sm_count);
    p.ws = o.ws ? o.ws : static_cast<float*>(ctx.workspace(stream, (size_t)slots * p.slot_floats * sizeof(float)));
    kernel<<<slots, NT, smem, stream>>>(p);
    cuda_check(cudaGetLastError(), "qr_mid launch");
}

// ---------------------------------------------------------------------------
// The same kernel on scratch memory that is part of the library image
// ---------------------------------------------------------------------------
// launch_qr_mid above takes its per-block scratch slots from a workspace that
// it grows with cudaMalloc (and cudaFree, which stalls the whole GPU) when a
// call needs more than any call before it. Some callers must never trigger
// that: a serving loop with a latency budget, where one implicit device-wide
// synchronisation is a missed deadline, and a process whose framework has
// already claimed the GPU's memory for its own pool (PyTorch's caching
// allocator at its cap, say), where a raw cudaMalloc from a library can simply
// fail. For them the slots can live in the array below instead: it is part of
// the loaded module, so every GPU that loads the library holds these 32 MiB
// from load to exit, and nothing is allocated or freed at call time.
//
// Host code cannot pass `g_static_scratch` to a kernel: in host code that name
// is only a handle for the runtime, not a device address. The address is
// looked up once per GPU with cudaGetSymbolAddress, with that GPU current, on
// the first call that runs there.
constexpr size_t kStaticScratchFloats = (size_t)8 << 20;   // 32 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float*     g_static_address[kMaxDevices] = {};
int        g_static_sms[kMaxDevices] = {};
int        g_static_smem[kMaxDevices] = {};
}

size_t qr_mid_static_capacity_bytes() { return kStaticScratchFloats * sizeof(float); }

void launch_qr_mid_static(int device, cudaStream_t stream, const QrProblem& pr) {
    if (pr.batch == 0 || pr.m == 0 || pr.n == 0) return;
    if (device < 0 || device >= kMaxDevices) throw std::invalid_argument("[qr_no_alloc] no such CUDA device");
    DeviceGuard guard(device);
    float* scratch = nullptr;
    int sms = 0, smem_optin = 0;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static_address[device]) {   // first call on this GPU: the one-time set-up
            float* address = nullptr;
            cuda_check(cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_scratch),
                       "cudaGetSymbolAddress(static scratch)");
            cuda_check(cudaDeviceGetAttribute(&g_static_sms[device], cudaDevAttrMultiProcessorCount, device),
                       "cudaDeviceGetAttribute");
            cuda_check(cudaDeviceGetAttribute(&g_static_smem[device], cudaDevAttrMaxSharedMemoryPerBlockOptin, device),
                       "cudaDeviceGetAttribute");
            g_static_address[device] = address;
        }
        scratch = g_static_address[device];
        sms = g_static_sms[device];
        smem_optin = g_static_smem[device];
    }
    MidParams p{};
    p.a = pr.a; p.q = pr.q; p.r = pr.r;
    p.batch = pr.batch;
    p.m = (int)pr.m; p.n = (int)pr.n; p.K = (int)qr_k(pr); p.qc = (int)pr.qc; p.rr = (int)pr.rr;
    p.lda = (int)pr.n;
    p.a_stride = (uint64_t)pr.m * pr.n;
    p.q_stride = (uint64_t)pr.m * pr.qc;
    p.r_stride = (uint64_t)pr.rr * pr.n;
    p.scale = 1;
    p.ldv = (int)((pr.m + 31) / 32) * 32 + 4;
    p.npanels = (p.K + JB - 1) / JB;
    p.by_columns = mid_by_columns();
    p.pairs = mid_pairs();
    p.slot_floats = (((uint64_t)pr.m * pr.n + 3) & ~(uint64_t)3) + (uint64_t)p.npanels * 1024;
    const size_t smem = smem_bytes(p.ldv);
    if (pr.m > 1024 || smem > (size_t)smem_optin)
        throw std::invalid_argument("[qr_no_alloc] takes matrices of at most 1024 rows, got " + std::to_string(pr.m));
    if (p.slot_floats > kStaticScratchFloats)
        throw std::invalid_argument("[qr_no_alloc] one " + std::to_string(pr.m) + " x " + std::to_string(pr.n) +
                                    " matrix needs " + std::to_string(p.slot_floats * sizeof(float)) +
                                    " bytes of scratch; the built-in scratch holds " +
                                    std::to_string(kStaticScratchFloats * sizeof(float)));
    const MidKernel kernel = mid_kernel_for(pr.m);
    cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
               "qr_mid shared memory");
    int per_sm = 0;
    cuda_check(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, NT, smem), "qr_mid occupancy");
    if (per_sm < 1) throw std::runtime_error("[qr_no_alloc] the matrix does not fit a thread block");
    uint64_t slots = std::min<uint64_t>(pr.batch, (uint64_t)per_sm * sms);
    slots = std::min<uint64_t>(slots, kStaticScratchFloats / p.slot_floats);   // fewer blocks, each looping longer
    p.ws = scratch;
    kernel<<<(unsigned)slots, NT, smem, stream>>>(p);
    cuda_check(cudaGetLastError(), "qr_mid launch");
}

void launch_qr_mid(DeviceContext& ctx, cudaStream_t stream, const QrProblem& p) {
    launch_qr_mid(ctx, stream, p, MidOptions{});
}

} // namespace mlb
