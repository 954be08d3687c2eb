// TSQR: a tall thin matrix (m >> n, n <= 128) as a tree of row blocks, for the
// reduced factorisation and for R alone. This file holds the entry points and
// the scheme with an explicit Q at every block, which takes 65 to 128 columns;
// at most 64 columns go to qr_tsqr_vt.cu (blocks kept as reflectors, Q built
// once on the way down), to which tsqr_core hands over.
//
// It takes the place of the reference's TSQR panel kernels bd_tsqr_leaf /
// bd_tsqr_top / bd_tsqr_rebuild (shaders/Svd_Bidiag.metal:583-869; host side
// src/band_reduce.mm:196-251), which the reference reaches for every matrix
// taller than a threadgroup holds (src/qr_householder.mm:387-391). The
// reference reconstructs Householder vectors from the tree because its caller
// needs them for a trailing update; a tall thin QR has no trailing matrix, so
// here the tree's Q is formed explicitly and no reconstruction is needed:
//
//   level 0   the matrix is cut into blocks of `c` rows; each block is factored
//             by the block-per-matrix kernel (qr_mid.cu), its Q written in place
//             into the output Q and its n x n R onto a stack;
//   level l   the stack of R's (itself a tall matrix, c/n times shorter) is cut
//             and factored the same way, until fewer than two blocks' rows remain, which
//             one block factors: its R is the matrix's R;
//   down      Q's blocks are multiplied from the right by the n x n blocks of
//             the level above, level by level (tsqr_apply_kernel below).
//
// Algorithmic traffic is A read once, Q and R written once; this scheme reads A,
// writes Q, reads and rewrites Q once more on the way down, and the stacks are a
// fraction n/c of that. R's diagonal has the signs of the top-level factorisation,
// which need not be LAPACK's for the whole matrix (the reference's TSQR likewise).
// A block holding a NaN or an infinity gives NaN R for that block, so the stack,
// the top-level Q and with it every entry of the matrix's Q and R are NaN.
#include "common.cuh"
#include "kernels.h"
#include "qr_small_steps.cuh"

#include <algorithm>
#include <cstdlib>
#include <vector>

namespace mlb {

namespace {

constexpr int TR = 64;          // rows of Q per thread block of the apply kernel

struct ApplyParams {
    const float* q;             // blocks of rows (ld n): block i of matrix b at b * q_outer + i * q_stride
    float*       out;           // where the products go: block i of matrix b at b * out_outer + i * out_stride, ld out_ld
    const float* up;            // n x n factors: that block's at (b * blocks + i) * n * n, or one per matrix
    unsigned     shared_up;     // 1: every block of matrix b uses the factor at b * n * n
    unsigned     blocks;        // row blocks per matrix
    unsigned     rows, last_rows;   // rows of a block, and of a matrix's last block
    unsigned     tiles;         // ceil(max(rows, last_rows) / TR)
    int          n, np;         // columns, and columns rounded up to 64
    unsigned long long q_outer, q_stride, out_outer, out_stride, out_ld;
    unsigned long long total;   // matrices * blocks * tiles
};

// Q_block <- Q_block * B in place. A thread block takes a whole row block: B (n x n, row-major) is
// loaded once, then TR rows of Q at a time, kept row-major in shared memory as they come (16-byte
// copies); a thread holds 4 x 4 outputs and reads four k's of its four rows and of B's rows as
// 16-byte words, so that the products run on packed FMAs two columns at a time.
__global__ void __launch_bounds__(256) tsqr_apply_kernel(const ApplyParams p) {
    extern __shared__ __align__(16) float sm[];
    const int n = p.n, np = p.np, kp = (n + 3) & ~3, ldx = kp + 4;
    float* Xs = sm;                       // [TR][ldx]
    float* Bs = sm + (size_t)TR * ldx;    // [kp][np], rows and columns beyond n zero
    const int rg = threadIdx.x >> 4, cg = threadIdx.x & 15;   // 16 row quads x 16 column quads (per 64 columns)
    const unsigned long long blocks_total = p.total / p.tiles;
    for (unsigned long long blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
        const unsigned i = (unsigned)(blk % p.blocks);
        const unsigned long long b = blk / p.blocks;
        const unsigned rows = i + 1 == p.blocks ? p.last_rows : p.rows;
        const float* B = p.up + (p.shared_up ? b : blk) * (unsigned long long)n * n;
        __syncthreads();
        for (int idx = threadIdx.x; idx < kp * np; idx += 256) {
            const int k = idx / np, c = idx % np;
            Bs[idx] = (c < n && k < n) ? B[(size_t)k * n + c] : 0.0f;
        }
        for (unsigned r0 = 0; r0 < rows; r0 += TR) {
            const unsigned nr = min((unsigned)TR, rows - r0);
            const float* Q = p.q + b * p.q_outer + (unsigned long long)i * p.q_stride + (size_t)r0 * n;
            float* O = p.out + b * p.out_outer + (unsigned long long)i * p.out_stride + (size_t)r0 * p.out_ld;
            const size_t ldo = (size_t)p.out_ld;
            const bool vec = (ldo & 3) == 0 && (reinterpret_cast<size_t>(O) & 15) == 0;
            if ((n & 3) == 0 && (reinterpret_cast<size_t>(Q) & 15) == 0) {
                const int nq = n >> 2;
                for (int idx = threadIdx.x; idx < TR * nq; idx += 256) {
                    const int r = idx / nq, kq = idx % nq;
                    const float4 v = (unsigned)r < nr ? *reinterpret_cast<const float4*>(Q + (size_t)r * n + 4 * kq)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4*>(Xs + r * ldx + 4 * kq) = v;
                }
            } else {
                for (int idx = threadIdx.x; idx < TR * kp; idx += 256) {
                    const int r = idx / kp, k = idx % kp;
                    Xs[r * ldx + k] = ((unsigned)r < nr && k < n) ? Q[(size_t)r * n + k] : 0.0f;
                }
            }
            __syncthreads();
            for (int c0 = 0; c0 < np; c0 += 64) {
                using small::pair_t;
                pair_t acc[4][2];
#pragma unroll
                for (int a = 0; a < 4; ++a) acc[a][0] = acc[a][1] = small::pack(0.0f, 0.0f);
#pragma unroll 2
                for (int k0 = 0; k0 < kp; k0 += 4) {
                    float4 x[4];
#pragma unroll
                    for (int a = 0; a < 4; ++a) x[a] = *reinterpret_cast<const float4*>(Xs + (4 * rg + a) * ldx + k0);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(Bs + (k0 + kk) * np + c0 + 4 * cg);
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            const float xv = kk == 0 ? x[a].x : kk == 1 ? x[a].y : kk == 2 ? x[a].z : x[a].w;
                            const pair_t xx = small::pack(xv, xv);
                            acc[a][0] = small::fma2(xx, w.x, acc[a][0]);
                            acc[a][1] = small::fma2(xx, w.y, acc[a][1]);
                        }
                    }
                }
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const unsigned r = 4 * rg + a;
                    if (r < nr) {
                        const int c = c0 + 4 * cg;
                        float o[4];
                        small::unpack(acc[a][0], o[0], o[1]);
                        small::unpack(acc[a][1], o[2], o[3]);
                        if (vec && c + 3 < n) {   // the rows are 16-byte aligned: one word a thread
                            *reinterpret_cast<float4*>(O + (size_t)r * ldo + c) = make_float4(o[0], o[1], o[2], o[3]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (c + e < n) O[(size_t)r * ldo + c + e] = o[e];
                        }
                    }
                }
            }
            __syncthreads();      // the tile has been read: the next one may overwrite it
        }
    }
}

struct Level {
    uint32_t rows;        // rows of this level's matrix (per input matrix)
    uint32_t c;           // rows of a block
    uint32_t blocks;      // blocks per matrix; the last has rows - (blocks - 1) * c
    uint32_t last_rows;
};

// Blocks of 256 rows at every width: the most the block kernel's panels hold with a column per lane. (For 65
// to 128 columns a level then only halves the rows, but blocks of 512 rows, whose panels go a thread per
// entry, measured a quarter to a third slower: 16 x 8192 x 128 in 2.24 against 2.99 ms.)
uint32_t block_rows(uint32_t) {
    const char* e = std::getenv("QR_TSQR_ROWS");      // for measurements: 256 (default) or 512
    return e && std::atoi(e) == 512 ? 512u : 256u;
}

// The levels below the top: each cuts `rows` into blocks of c (the last takes the remainder, < 2c).
std::vector<Level> plan(uint32_t m, uint32_t n) {
    std::vector<Level> levels;
    const uint32_t c = block_rows(n);
    uint32_t rows = m;
    // down to fewer than two blocks' worth of rows: the top is then at most 2c - 1 rows, 256 x n after a level of
    // four blocks (a block of 1024 rows, the most a thread block holds, takes five times as long as one of 256)
    while (rows >= 2 * c) {
        Level L{rows, c, rows / c, 0};
        L.last_rows = rows - (L.blocks - 1) * c;
        levels.push_back(L);
        rows = L.blocks * n;
    }
    return levels;
}

} // namespace

void launch_tsqr_apply(DeviceContext& ctx, cudaStream_t stream, const float* q, uint64_t q_outer, uint64_t q_stride,
                       float* out, uint64_t out_outer, uint64_t out_stride, uint64_t out_ld, const float* up,
                       bool shared_up, uint32_t batch, uint32_t blocks, uint32_t rows, uint32_t last_rows, uint32_t n) {
    if (batch == 0 || blocks == 0 || n == 0 || std::max(rows, last_rows) == 0) return;
    const int np = (int)((n + 63) / 64 * 64);
    const int kp = ((int)n + 3) & ~3;
    const size_t smem = ((size_t)TR * (kp + 4) + (size_t)kp * np) * sizeof(float);
    cuda_check(cudaFuncSetAttribute(tsqr_apply_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
               "tsqr_apply shared memory");
    ApplyParams a{};
    a.q = q; a.out = out; a.up = up;
    a.shared_up = shared_up ? 1 : 0;
    a.blocks = blocks; a.rows = rows; a.last_rows = last_rows;
    a.tiles = (std::max(rows, last_rows) + TR - 1) / TR;
    a.n = (int)n; a.np = np;
    a.q_outer = q_outer; a.q_stride = q_stride;
    a.out_outer = out_outer; a.out_stride = out_stride; a.out_ld = out_ld;
    a.total = (uint64_t)batch * blocks * a.tiles;
    const unsigned grid = (unsigned)std::min<uint64_t>((uint64_t)batch * blocks, (uint64_t)ctx.sm_count * 8);
    tsqr_apply_kernel<<<grid, 256, smem, stream>>>(a);
    cuda_check(cudaGetLastError(), "tsqr_apply launch");
}

namespace {

struct Layout {
    std::vector<Level>  levels;
    std::vector<size_t> s_off, q_off;   // per level l >= 1: its stack of R's and (with Q) its Q, in floats
    size_t              mid_off = 0, total = 0;
    uint32_t            top_rows = 0;
};

Layout layout(const DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t batch, bool want_q) {
    Layout L;
    L.levels = plan(m, n);
    const size_t nl = L.levels.size();
    L.top_rows = nl ? L.levels.back().blocks * n : m;
    auto up64 = [](size_t f) { return (f + 63) & ~(size_t)63; };
    L.s_off.assign(nl + 1, 0);
    L.q_off.assign(nl + 1, 0);
    for (size_t l = 1; l <= nl; ++l) {
        const size_t floats = (size_t)batch * L.levels[l - 1].blocks * n * n;   // one n x n block per block below
        L.s_off[l] = L.total; L.total += up64(floats);
        if (want_q) { L.q_off[l] = L.total; L.total += up64(floats); }
    }
    size_t mid_floats = qr_mid_workspace_floats(ctx, L.top_rows, n, batch);
    for (const Level& lv : L.levels) {
        mid_floats = std::max(mid_floats, qr_mid_workspace_floats(ctx, lv.c, n, batch * lv.blocks));
        mid_floats = std::max(mid_floats, qr_mid_workspace_floats(ctx, lv.last_rows, n, batch));
    }
    L.mid_off = L.total;
    L.total += up64(mid_floats);
    return L;
}

} // namespace

size_t tsqr_workspace_floats(const DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t batch, bool want_q) {
    if (tsqr_vt_takes(m, n)) return tsqr_vt_workspace_floats(m, n, batch, want_q);
    return layout(ctx, m, n, batch, want_q).total;
}

// Thin QR of `batch` matrices of m x n (n <= 128, any m >= n) read with row stride lda and matrix
// stride a_outer: q [batch][m][n] contiguous (null: R alone), r [batch] n x n at stride r_outer.
void tsqr_core(DeviceContext& ctx, cudaStream_t stream, const float* a, uint32_t lda, uint64_t a_outer, uint32_t m,
               uint32_t n, uint32_t batch, float* q, float* r, uint64_t r_outer, float* ws) {
    if (batch == 0) return;
    if (tsqr_vt_takes(m, n)) {      // at most 64 columns: the blocks kept as reflectors, Q built once on the way down
        tsqr_vt_core(stream, a, lda, a_outer, m, n, batch, q, r, r_outer, ws);
        return;
    }
    const bool want_q = q != nullptr;
    const Layout L = layout(ctx, m, n, batch, want_q);
    const size_t nl = L.levels.size();
    const uint32_t qc = want_q ? n : 0;

    // up the tree
    for (size_t l = 0; l < nl; ++l) {
        const Level& lv = L.levels[l];
        const float* in = l == 0 ? a : ws + L.s_off[l];
        const uint32_t in_ld = l == 0 ? lda : n;
        const uint64_t in_outer = l == 0 ? a_outer : (uint64_t)lv.rows * n;
        float* qout = !want_q ? nullptr : (l == 0 ? q : ws + L.q_off[l]);
        float* rout = ws + L.s_off[l + 1];
        MidOptions o;
        o.ws = ws + L.mid_off;
        o.lda = in_ld;
        o.a_stride = (uint64_t)lv.c * in_ld; o.q_stride = (uint64_t)lv.c * n; o.r_stride = (uint64_t)n * n;
        o.a_outer = in_outer; o.q_outer = (uint64_t)lv.rows * n; o.r_outer = (uint64_t)lv.blocks * n * n;
        if (lv.last_rows == lv.c) {   // no remainder: every block of every matrix in one launch
            QrProblem p{in, qout, rout, batch * lv.blocks, lv.c, n, qc, n};
            o.inner_count = lv.blocks;
            launch_qr_mid(ctx, stream, p, o);
            continue;
        }
        if (lv.blocks > 1) {   // the full blocks of every matrix in one launch
            QrProblem p{in, qout, rout, batch * (lv.blocks - 1), lv.c, n, qc, n};
            o.inner_count = lv.blocks - 1;
            launch_qr_mid(ctx, stream, p, o);
        }
        {   // each matrix's last block (c rows plus the remainder)
            const uint64_t skip = (uint64_t)(lv.blocks - 1);
            QrProblem p{in + skip * lv.c * in_ld, qout ? qout + skip * lv.c * n : nullptr, rout + skip * n * n, batch,
                        lv.last_rows, n, qc, n};
            o.inner_count = 1;
            launch_qr_mid(ctx, stream, p, o);
        }
    }
    // the top: one block per matrix; its R is the matrix's R
    {
        MidOptions o;
        o.ws = ws + L.mid_off;
        o.inner_count = 1;
        o.r_outer = r_outer;
        o.r_stride = (uint64_t)n * n;
        if (nl == 0) {
            o.lda = lda; o.a_outer = a_outer; o.a_stride = (uint64_t)m * lda;
            o.q_outer = (uint64_t)m * n; o.q_stride = o.q_outer;
            QrProblem p{a, q, r, batch, m, n, qc, n};
            launch_qr_mid(ctx, stream, p, o);
            return;
        }
        o.a_outer = (uint64_t)L.top_rows * n; o.a_stride = o.a_outer;
        o.q_outer = o.a_outer; o.q_stride = o.a_outer;
        QrProblem p{ws + L.s_off[nl], want_q ? ws + L.q_off[nl] : nullptr, r, batch, L.top_rows, n, qc, n};
        launch_qr_mid(ctx, stream, p, o);
    }
    if (!want_q) return;

    // down the tree: level l's Q blocks times the n x n blocks of level l+1's Q, in place
    for (size_t l = nl; l-- > 0;) {
        const Level& lv = L.levels[l];
        float* ql = l == 0 ? q : ws + L.q_off[l];
        launch_tsqr_apply(ctx, stream, ql, (uint64_t)lv.rows * n, (uint64_t)lv.c * n, ql, (uint64_t)lv.rows * n,
                          (uint64_t)lv.c * n, n, ws + L.q_off[l + 1], false, batch, lv.blocks, lv.c, lv.last_rows, n);
    }
}

bool qr_tsqr_fits(const DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t qc) {
    // reduced or R alone (Q of n columns or none), at most 128 columns, at least two levels' worth of rows
    // reduced or R alone (Q of n columns or none), at most 128 columns, at least two blocks of rows and eight times
    // as tall as wide (640 x 96 is faster in one block; 512 x 64 and 1024 x 128 are faster here)
    // with at most 64 columns the blocks are kept as reflectors (qr_tsqr_vt.cu), and one such block, or two, already beats
    // the general block kernel where a block of 256 rows is filled to three quarters (16384 of 256 x 64: 4.4 against
    // 5.9 ms; 8192 of 500 x 48: 6.3 against 10.6; 16384 of 200 x 40: 4.2 against 5.3; but 16384 of 128 x 64: 4.3 against 3.7)
    if (n >= 1 && n <= 64 && m >= 192 && m >= 3 * n && (qc == 0 || qc == n) && tsqr_vt_takes(m, n)) return true;
    return n >= 1 && n <= 128 && m >= 512 && m >= 8 * n && (qc == 0 || qc == n) && qr_mid_fits(ctx, 1024, n);
}

void launch_qr_tsqr(DeviceContext& ctx, cudaStream_t stream, const QrProblem& pr) {
    if (pr.batch == 0) return;
    const bool want_q = pr.qc != 0;
    const size_t floats = tsqr_workspace_floats(ctx, pr.m, pr.n, pr.batch, want_q);
    float* ws = static_cast<float*>(ctx.workspace(stream, floats * sizeof(float)));
    tsqr_core(ctx, stream, pr.a, pr.n, (uint64_t)pr.m * pr.n, pr.m, pr.n, pr.batch, want_q ? pr.q : nullptr, pr.r,
              (uint64_t)pr.n * pr.n, ws);
}

} // namespace mlb
