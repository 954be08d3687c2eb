// TSQR for at most 64 columns with the row blocks kept as reflectors: every block of the tree is
// factored into (V, T, R) and its explicit Q is never formed; Q is built once, on the way down, as
//
//     Q_block = [B; 0] - V (T (V1^T B)),     B = this block's n x n piece of the Q one level up
//
// so that every entry of Q is computed and written exactly once. The reference's TSQR kernels keep
// V and T in the same way (bd_tsqr_leaf / bd_tsqr_rebuild, shaders/Svd_Bidiag.metal:583-610,
// 808-869; host side src/band_reduce.mm:196-251); qr_tsqr.cu's older scheme (blocks through the
// general block-per-matrix kernel, explicit Q at every block, multiplied again on the way down)
// stays for 65 to 128 columns and behind QR_TSQR_VT=0.
//
// The block kernel: 256 rows x n columns in the registers of one thread block, a COLUMN per lane
// (qr_panel_cols.cuh's layout): warp w holds rows 32 w ..., lane l columns l and 32 + l, two rows
// to a 64-bit register. Two columns a reduction (factor_cols2's arithmetic, with its fallback for
// nearly parallel neighbours): lanes j and j + 1 publish their columns below the pivot pair, every
// lane takes both products with its own two columns, one barrier, and both reflectors are applied
// as one rank-2 update. Columns 0..31 are one panel (pivot rows in warp 0), columns 32..63 the
// next (pivot rows in warp 1); the columns of the other half ride along: right of the panel they
// are updated with it, left of it only their products are taken, which are the Gram entries
// v_k^T v_j that T is built from. The pivot warp's registers rotate as in step_warp0, so no
// register index depends on the step.
//
// Contract of a block: scan + power-of-two scaling, R multiplied back (exact), slarfg's signs; a
// block with a NaN or an infinity gives NaN R, V and T, which makes everything above and below it
// in that matrix's tree NaN.
#include "common.cuh"
#include "kernels.h"
#include "qr_panel_cols.cuh"

#include <algorithm>
#include <cstdlib>
#include <vector>

namespace mlb {

namespace {

using namespace small;
using cols::kPairKeep;
using cols::recip;

constexpr int      kBlockRows = 256;
constexpr int      kThreads   = 256;
constexpr int      kWarps     = 8;

// Block i of a level of `rows` rows cut into `blocks`: 256 rows each, the last the remainder; where the
// remainder is shorter than the matrix is wide the block before it gives up d rows (a block of fewer
// rows than columns would have reflectors that reach into its padding).
__host__ __device__ inline void block_span(unsigned i, unsigned blocks, unsigned rows, unsigned d, unsigned& start,
                                           unsigned& nrows) {
    if (blocks == 1) {
        start = 0;
        nrows = rows;
        return;
    }
    const unsigned rem = rows - (blocks - 1) * kBlockRows;
    start = i * kBlockRows - (i + 1 == blocks ? d : 0);
    nrows = i + 1 == blocks ? rem + d : (i + 2 == blocks ? kBlockRows - d : kBlockRows);
}

template <int SETS>
struct LeafSmem {
    static constexpr int NC = 32 * SETS;
    float red[2][kWarps][32][2 * SETS];     // by pair parity: each warp's partial products per lane (p, q of its set; p, q of the other), one word
    float red1[SETS][kWarps][32];           // the same for a column stepped alone
    float prow[2][2][NC];                   // by pair parity: the two pivot rows of every column
    float prow1[NC];
    float pub[kWarps][2][32];               // each warp's pieces of the two published columns
    float top[NC][NC + 1];                  // the block's first rows as they finish: R, and the reflectors' tails below the diagonal
    float G[NC][NC + 1];                    // G[k][j] = v_k^T v_j, k < j (unit-diagonal reflectors)
    float T[NC][NC + 1];
    float X[32][33];
    float taus[NC], sc[NC];
    float amax[kWarps];
};

struct LeafParams {
    const float* in;            // matrix b at in + b * in_outer, rows of in_ld floats
    float*       v;             // V, rows of n floats: matrix b at v + b * v_outer (null: R alone)
    float*       t;             // T of block i of matrix b at t + (b * blocks + i) * n * n
    float*       r;             // R of that block at r + b * r_outer + i * n * n (n x n, zeros below the diagonal)
    unsigned long long in_outer, v_outer, r_outer;
    unsigned     in_ld;
    unsigned     rows, blocks, d;
    int          n;
};

#define MLB_SEL(u, i) (((i) & 1) ? (u).y : (u).x)

// piv: this warp holds the panel's pivot rows. The pivot warp and the others run separate copies of the loop (fewer
// values live in each, no branches on the warp's role) and meet at a named barrier.
template <int SETS, int P, bool piv>
__device__ __forceinline__ void leaf_steps(pair_t (&xa)[16], pair_t (&xo)[16], LeafSmem<SETS>& s, float& my_sc, float& my_sco,
                                           const int lane, const int warp) {
    constexpr bool kOth = SETS == 2, kRight = SETS == 2 && P == 0, kLeft = SETS == 2 && P == 1;
    constexpr int  cb = 32 * P, co = kOth ? 32 * (1 - P) : 0;
    const bool lead = warp == kWarps - 1;
    ulonglong2* pA = reinterpret_cast<ulonglong2*>(s.pub[warp][0]);
    ulonglong2* pB = reinterpret_cast<ulonglong2*>(s.pub[warp][1]);
    const pair_t zero2 = pack(0.0f, 0.0f);
#pragma unroll 1
    for (int it = 0; it < 16; ++it) {
        const int j = 2 * it, J = cb + j, buf = it & 1;
        // 1. columns j and j + 1 below the pivot pair (the pivot warp's pair 0 holds rows J and J + 1 themselves)
        __syncwarp();
        if (lane == j || lane == j + 1) {
            ulonglong2* dst = lane == j ? pA : pB;
#pragma unroll
            for (int q = 0; q < 8; ++q) dst[q] = make_ulonglong2((piv && q == 0) ? zero2 : xa[2 * q], xa[2 * q + 1]);
        }
        __syncwarp();
        // 2. both products with this lane's columns
        {
            pair_t sa = zero2, sa2 = zero2, sb = zero2, sb2 = zero2;
            pair_t oa = zero2, oa2 = zero2, ob = zero2, ob2 = zero2;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const ulonglong2 ua = pA[q], ub = pB[q];
                sa  = fma2(ua.x, xa[2 * q], sa);
                sa2 = fma2(ua.y, xa[2 * q + 1], sa2);
                sb  = fma2(ub.x, xa[2 * q], sb);
                sb2 = fma2(ub.y, xa[2 * q + 1], sb2);
                if (kOth) {
                    oa  = fma2(ua.x, xo[2 * q], oa);
                    oa2 = fma2(ua.y, xo[2 * q + 1], oa2);
                    ob  = fma2(ub.x, xo[2 * q], ob);
                    ob2 = fma2(ub.y, xo[2 * q + 1], ob2);
                }
            }
            if (kOth) {
                *reinterpret_cast<float4*>(s.red[buf][warp][lane]) =
                    make_float4(hsum2(sa, sa2), hsum2(sb, sb2), hsum2(oa, oa2), hsum2(ob, ob2));
            } else {
                *reinterpret_cast<float2*>(s.red[buf][warp][lane]) = make_float2(hsum2(sa, sa2), hsum2(sb, sb2));
            }
        }
        if (piv) {
            s.prow[buf][0][cb + lane] = lo_of(xa[0]);
            s.prow[buf][1][cb + lane] = hi_of(xa[0]);
            if (kOth) {
                s.prow[buf][0][co + lane] = lo_of(xo[0]);
                s.prow[buf][1][co + lane] = hi_of(xo[0]);
            }
        }
        cols::step_barrier(kThreads);
        float p = 0.0f, q = 0.0f, po = 0.0f, qo = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            if (kOth) {
                const float4 v = *reinterpret_cast<const float4*>(s.red[buf][w][lane]);
                p += v.x; q += v.y; po += v.z; qo += v.w;
            } else {
                const float2 v = *reinterpret_cast<const float2*>(s.red[buf][w][lane]);
                p += v.x; q += v.y;
            }
        }
        // 3. step J, and what step J + 1 will see
        const float r0 = s.prow[buf][0][cb + lane], r1 = s.prow[buf][1][cb + lane];      // rows J and J + 1 of this lane's column
        const float alpha = s.prow[buf][0][J], e = s.prow[buf][1][J];
        const float f0 = s.prow[buf][0][J + 1], f1 = s.prow[buf][1][J + 1];
        const float pj = __shfl_sync(0xffffffffu, p, j), pj1 = __shfl_sync(0xffffffffu, p, j + 1);
        const float qj1 = __shfl_sync(0xffffffffu, q, j + 1);
        float v1, gneg;
        fast_reflector(alpha, fmaf(e, e, pj), v1, gneg);
        const float sv  = fmaf(v1, r0, fmaf(e, r1, p));
        const float tk  = lane > j ? sv * gneg : 0.0f;
        const float tj1 = fmaf(v1, f0, fmaf(e, f1, pj1)) * gneg;
        const float scj = gneg != 0.0f ? recip(v1) : 0.0f;
        float r0o = 0.0f, r1o = 0.0f, svo = 0.0f, tko = 0.0f;
        if (kOth) {
            r0o = s.prow[buf][0][co + lane];
            r1o = s.prow[buf][1][co + lane];
            svo = fmaf(v1, r0o, fmaf(e, r1o, po));
            tko = kRight ? svo * gneg : 0.0f;
        }
        if (lead) {
            if (lane < j) s.G[cb + lane][J] = sv * my_sc * scj;
            if (kLeft) s.G[lane][J] = svo * my_sco * scj;
            if (lane == 0) {
                s.taus[J] = -gneg * v1 * v1;
                s.sc[J]   = scj;
            }
        }
        if (lane == j) my_sc = scj;
        const float m1 = fmaf(tk, e, r1);                                          // row J + 1 of this column after step J
        const float rj = lane > j ? fmaf(tk, v1, r0) : (lane == j ? alpha - v1 : r0);      // row J: final
        const float m1o = fmaf(tko, e, r1o), rjo = fmaf(tko, v1, r0o);
        const float alpha1 = fmaf(tj1, e, f1);
        const float ss1 = fmaf(tj1, fmaf(tj1, pj, 2.0f * pj1), qj1);               // column J + 1's norm below the pair, after step J
        if (!(ss1 < kPairKeep * qj1)) {
            // 4a. step J + 1 from the same sums, and both reflectors in one update
            float v1b, gnegb;
            fast_reflector(alpha1, ss1, v1b, gnegb);
            const float s1  = fmaf(tj1 * tk, pj, fmaf(tj1, p, fmaf(tk, pj1, q)));
            const float sv1 = fmaf(v1b, m1, s1);
            const float t1  = lane > j + 1 ? sv1 * gnegb : 0.0f;
            const float scj1 = gnegb != 0.0f ? recip(v1b) : 0.0f;
            float sv1o = 0.0f, t1o = 0.0f;
            if (kOth) {
                const float s1o = fmaf(tj1 * tko, pj, fmaf(tj1, po, fmaf(tko, pj1, qo)));
                sv1o = fmaf(v1b, m1o, s1o);
                t1o  = kRight ? sv1o * gnegb : 0.0f;
            }
            if (lead) {
                if (lane < j + 1) s.G[cb + lane][J + 1] = sv1 * my_sc * scj1;
                if (kLeft) s.G[lane][J + 1] = sv1o * my_sco * scj1;
                if (lane == 0) {
                    s.taus[J + 1] = -gnegb * v1b * v1b;
                    s.sc[J + 1]   = scj1;
                }
            }
            if (lane == j + 1) my_sc = scj1;
            const float ca = fmaf(t1, tj1, tk), cao = fmaf(t1o, tj1, tko);
            const pair_t a2 = pack(ca, ca), b2 = pack(t1, t1), ao2 = pack(cao, cao), bo2 = pack(t1o, t1o);
            if (piv) {
                const float rj1 = lane > j + 1 ? fmaf(t1, v1b, m1) : (lane == j + 1 ? alpha1 - v1b : m1);
                s.top[J][cb + lane]     = rj;
                s.top[J + 1][cb + lane] = rj1;
                if (kOth) {
                    s.top[J][co + lane]     = rjo;
                    s.top[J + 1][co + lane] = fmaf(t1o, v1b, m1o);
                }
                // the pairs move up one place as the two finished rows leave
#pragma unroll
                for (int i = 1; i < 16; ++i) {
                    const ulonglong2 ua = pA[i / 2], ub = pB[i / 2];
                    xa[i - 1] = fma2(a2, MLB_SEL(ua, i), fma2(b2, MLB_SEL(ub, i), xa[i]));
                    if (kRight) xo[i - 1] = fma2(ao2, MLB_SEL(ua, i), fma2(bo2, MLB_SEL(ub, i), xo[i]));
                    if (kLeft) xo[i - 1] = xo[i];
                }
                xa[15] = zero2;
                if (kOth) xo[15] = zero2;
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const ulonglong2 ua = pA[i / 2], ub = pB[i / 2];
                    xa[i] = fma2(a2, MLB_SEL(ua, i), fma2(b2, MLB_SEL(ub, i), xa[i]));
                    if (kRight) xo[i] = fma2(ao2, MLB_SEL(ua, i), fma2(bo2, MLB_SEL(ub, i), xo[i]));
                }
            }
        } else {
            // 4b. step J alone ...
            const pair_t a2 = pack(tk, tk), ao2 = pack(tko, tko);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const ulonglong2 ua = pA[i / 2];
                xa[i] = fma2(a2, MLB_SEL(ua, i), xa[i]);
                if (kRight) xo[i] = fma2(ao2, MLB_SEL(ua, i), xo[i]);
            }
            if (piv) {      // the published pair 0 was zero: rows J (finished) and J + 1 (the next pivot row) by hand
                xa[0] = pack(rj, m1);
                if (kOth) xo[0] = pack(rjo, m1o);
            }
            // ... then column J + 1 as a step of its own
            __syncwarp();
            if (lane == j + 1) {
#pragma unroll
                for (int q8 = 0; q8 < 8; ++q8) pB[q8] = make_ulonglong2((piv && q8 == 0) ? zero2 : xa[2 * q8], xa[2 * q8 + 1]);
            }
            __syncwarp();
            {
                pair_t sb = zero2, sb2 = zero2, ob = zero2, ob2 = zero2;
#pragma unroll
                for (int q8 = 0; q8 < 8; ++q8) {
                    const ulonglong2 ub = pB[q8];
                    sb  = fma2(ub.x, xa[2 * q8], sb);
                    sb2 = fma2(ub.y, xa[2 * q8 + 1], sb2);
                    if (kOth) {
                        ob  = fma2(ub.x, xo[2 * q8], ob);
                        ob2 = fma2(ub.y, xo[2 * q8 + 1], ob2);
                    }
                }
                s.red1[0][warp][lane] = hsum2(sb, sb2);
                if (kOth) s.red1[SETS - 1][warp][lane] = hsum2(ob, ob2);
            }
            if (piv) {
                s.prow1[cb + lane] = hi_of(xa[0]);
                if (kOth) s.prow1[co + lane] = hi_of(xo[0]);
            }
            cols::step_barrier(kThreads);
            float dd = 0.0f, ddo = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                dd += s.red1[0][w][lane];
                if (kOth) ddo += s.red1[SETS - 1][w][lane];
            }
            const float xj = s.prow1[cb + lane], al = s.prow1[J + 1];
            const float ss = __shfl_sync(0xffffffffu, dd, j + 1);
            float v1c, gnegc;
            fast_reflector(al, ss, v1c, gnegc);
            const float svc  = fmaf(v1c, xj, dd);
            const float tc   = lane > j + 1 ? svc * gnegc : 0.0f;
            const float scj1 = gnegc != 0.0f ? recip(v1c) : 0.0f;
            float xjo = 0.0f, svco = 0.0f, tco = 0.0f;
            if (kOth) {
                xjo  = s.prow1[co + lane];
                svco = fmaf(v1c, xjo, ddo);
                tco  = kRight ? svco * gnegc : 0.0f;
            }
            if (lead) {
                if (lane < j + 1) s.G[cb + lane][J + 1] = svc * my_sc * scj1;
                if (kLeft) s.G[lane][J + 1] = svco * my_sco * scj1;
                if (lane == 0) {
                    s.taus[J + 1] = -gnegc * v1c * v1c;
                    s.sc[J + 1]   = scj1;
                }
            }
            if (lane == j + 1) my_sc = scj1;
            const pair_t c2 = pack(tc, tc), co2 = pack(tco, tco);
            if (piv) {
                const float rj1 = lane > j + 1 ? fmaf(tc, v1c, xj) : (lane == j + 1 ? al - v1c : xj);
                s.top[J][cb + lane]     = lo_of(xa[0]);
                s.top[J + 1][cb + lane] = rj1;
                if (kOth) {
                    s.top[J][co + lane]     = lo_of(xo[0]);
                    s.top[J + 1][co + lane] = fmaf(tco, v1c, xjo);
                }
#pragma unroll
                for (int i = 1; i < 16; ++i) {
                    const ulonglong2 ub = pB[i / 2];
                    xa[i - 1] = fma2(c2, MLB_SEL(ub, i), xa[i]);
                    if (kRight) xo[i - 1] = fma2(co2, MLB_SEL(ub, i), xo[i]);
                    if (kLeft) xo[i - 1] = xo[i];
                }
                xa[15] = zero2;
                if (kOth) xo[15] = zero2;
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const ulonglong2 ub = pB[i / 2];
                    xa[i] = fma2(c2, MLB_SEL(ub, i), xa[i]);
                    if (kRight) xo[i] = fma2(co2, MLB_SEL(ub, i), xo[i]);
                }
            }
        }
    }
}

// The 16 pair steps of panel P (columns 32 P ...): xa its own columns' registers, xo the other half's.
template <int SETS, int P>
__device__ __forceinline__ void leaf_panel(pair_t (&xa)[16], pair_t (&xo)[16], LeafSmem<SETS>& s, float& my_sc, float& my_sco,
                                           const int lane, const int warp) {
    if (warp == P) leaf_steps<SETS, P, true>(xa, xo, s, my_sc, my_sco, lane, warp);
    else leaf_steps<SETS, P, false>(xa, xo, s, my_sc, my_sco, lane, warp);
}

// T of the 32 reflectors from column `off` on (slarft's forward recurrence), by one warp, a row of T per lane.
template <int SETS>
__device__ __forceinline__ void leaf_build_t(LeafSmem<SETS>& s, int off, int lane) {
    float tr[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const float tau = s.taus[off + j];
        float a = 0.0f, a2 = 0.0f;
#pragma unroll
        for (int k = 0; k + 1 < j; k += 2) {
            a  = fmaf(tr[k], s.G[off + k][off + j], a);
            a2 = fmaf(tr[k + 1], s.G[off + k + 1][off + j], a2);
        }
        if (j & 1) a = fmaf(tr[j - 1], s.G[off + j - 1][off + j], a);
        tr[j] = lane < j ? -tau * (a + a2) : (lane == j ? tau : 0.0f);
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) s.T[off + lane][off + j] = tr[j];
}

template <int SETS>
__global__ void __launch_bounds__(kThreads, SETS == 2 ? 2 : 3) tsqr_leaf_kernel(const LeafParams p) {
    extern __shared__ __align__(16) unsigned char leaf_raw[];
    LeafSmem<SETS>& s = *reinterpret_cast<LeafSmem<SETS>*>(leaf_raw);
    constexpr int NC = 32 * SETS;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int n = p.n;
    const unsigned i = blockIdx.x % p.blocks;
    const unsigned long long b = blockIdx.x / p.blocks;
    unsigned start, nrows;
    block_span(i, p.blocks, p.rows, p.d, start, nrows);
    const float* A = p.in + b * p.in_outer + (size_t)start * p.in_ld;
    const unsigned row0 = warp * 32;
    const bool ina = lane < n, inb = SETS == 2 && 32 + lane < n;

    pair_t xa[16], xb[16];
    {
        float va[32], vb[32];
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            const unsigned row = row0 + r;
            va[r] = (ina && row < nrows) ? A[(size_t)row * p.in_ld + lane] : 0.0f;
            vb[r] = (inb && row < nrows) ? A[(size_t)row * p.in_ld + 32 + lane] : 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            amax  = absmax3(va[2 * r], va[2 * r + 1], amax);
            xa[r] = pack(va[2 * r], va[2 * r + 1]);
            if (SETS == 2) {
                amax  = absmax3(vb[2 * r], vb[2 * r + 1], amax);
                xb[r] = pack(vb[2 * r], vb[2 * r + 1]);
            } else {
                xb[r] = pack(0.0f, 0.0f);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) s.amax[warp] = amax;
    }
    __syncthreads();
    float amax = s.amax[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) amax = max_nan(amax, s.amax[w]);
    const bool bad = !(amax < __uint_as_float(0x7F800000u));
    float* R = p.r + b * p.r_outer + (size_t)i * n * n;
    float* V = p.v ? p.v + b * p.v_outer + (size_t)start * n : nullptr;
    float* T = p.v ? p.t + ((size_t)b * p.blocks + i) * n * n : nullptr;
    if (bad) {      // NaN R, V and T: the levels above and the way down carry it to the whole matrix
        for (int idx = t; idx < n * n; idx += kThreads) {
            R[idx] = qnan();
            if (T) T[idx] = qnan();
        }
        if (V)
            for (size_t idx = t; idx < (size_t)nrows * n; idx += kThreads) V[idx] = qnan();
        return;
    }
    const int expo = amax_exponent(amax);
    if (expo != 0) {
        const Scale2 down(-expo);
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            xa[r] = mul2(xa[r], down.s1);
            if (SETS == 2) xb[r] = mul2(xb[r], down.s1);
        }
        if (down.two) {
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                xa[r] = mul2(xa[r], down.s2);
                if (SETS == 2) xb[r] = mul2(xb[r], down.s2);
            }
        }
    }

    float sca = 0.0f, scb = 0.0f;
    leaf_panel<SETS, 0>(xa, xb, s, sca, scb, lane, warp);
    if (SETS == 2) leaf_panel<SETS, 1>(xb, xa, s, scb, sca, lane, warp);

    // V below the pivot rows straight from the registers (unit-diagonal reflectors: the tails times 1 / v1)
    if (V && warp >= SETS) {
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const unsigned row = row0 + 2 * r;
            float a0, a1, b0, b1;
            unpack(xa[r], a0, a1);
            unpack(xb[r], b0, b1);
            if (ina && row < nrows) V[(size_t)row * n + lane] = a0 * sca;
            if (ina && row + 1 < nrows) V[(size_t)(row + 1) * n + lane] = a1 * sca;
            if (inb && row < nrows) V[(size_t)row * n + 32 + lane] = b0 * scb;
            if (inb && row + 1 < nrows) V[(size_t)(row + 1) * n + 32 + lane] = b1 * scb;
        }
    }
    __syncthreads();      // s.top, s.G, s.taus and s.sc are complete

    // T's diagonal blocks by one warp each; meanwhile the other warps write R (scaled back) and the first rows of V from s.top
    if (T && warp < SETS) {
        leaf_build_t<SETS>(s, 32 * warp, lane);
    } else {
        const int t0 = T ? t - 32 * SETS : t, nt = T ? kThreads - 32 * SETS : kThreads;
        const Pow2 up(expo);
        for (int idx = t0; idx < n * n; idx += nt) {
            const int r = idx / n, c = idx % n;
            R[idx] = r <= c ? up(s.top[r][c]) : 0.0f;
        }
        if (V) {
            const int vr = min((unsigned)NC, nrows);
            for (int idx = t0; idx < vr * n; idx += nt) {
                const int r = idx / n, c = idx % n;
                V[idx] = r > c ? s.top[r][c] * s.sc[c] : (r == c ? 1.0f : 0.0f);
            }
        }
    }
    if (!T) return;
    __syncthreads();
    // T12 = -T11 (V1^T V2) T22 by everyone
    if (SETS == 2) {
        const int r = t >> 3, c0 = 4 * (t & 7);
        float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {          // X = G12 T22 (T22 upper triangular)
            const float g = s.G[r][32 + k];
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] = fmaf(g, s.T[32 + k][32 + c0 + e], x[e]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) s.X[r][c0 + e] = x[e];
        __syncthreads();
        float y[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {          // T12 = -T11 X
            const float tv = s.T[r][k];
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = fmaf(tv, s.X[k][c0 + e], y[e]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            s.T[r][32 + c0 + e]      = -y[e];
            s.T[32 + r][c0 + e]      = 0.0f;
        }
        __syncthreads();
    }
    for (int idx = t; idx < n * n; idx += kThreads) {
        const int r = idx / n, c = idx % n;
        T[idx] = s.T[r][c];
    }
}

// ---------------------------------------------------------------------------------------------
// The way down: Q_block = [B; 0] - V (T (V1^T B)), in place over V.

constexpr int LD = 68;          // leading dimension of the blocks in shared memory (16-byte rows, 4 banks apart)

struct DownParams {
    float*       v;             // V in, Q out (rows of n floats): matrix b at v + b * v_outer
    const float* t;             // T of block i of matrix b at t + (b * blocks + i) * n * n
    const float* up;            // B of that block at up + (b * blocks + i) * n * n; null: the identity (the top of the tree)
    unsigned long long v_outer;
    unsigned     rows, blocks, d;
    int          n;
};

// acc (rows 4 rg ..., columns 4 cg ... of a 64 x 64 product, a thread of 256) = op(A) B for A, B in shared memory
// (k_from: op(A)'s rows 4 rg ... are zero left of it: V1^T and T are upper triangular, so a thread starts at its own rows)
template <bool TA>
__device__ __forceinline__ void mm64(const float* A, const float* B, pair_t (&acc)[4][2], int rg, int cg, int k_from = 0) {
#pragma unroll
    for (int a = 0; a < 4; ++a) acc[a][0] = acc[a][1] = pack(0.0f, 0.0f);
#pragma unroll 2
    for (int k0 = k_from; k0 < 64; k0 += 4) {
        float4 x[4];
        if (TA) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) x[kk] = *reinterpret_cast<const float4*>(A + (k0 + kk) * LD + 4 * rg);     // x[kk] = A[k][rows]
        } else {
#pragma unroll
            for (int a = 0; a < 4; ++a) x[a] = *reinterpret_cast<const float4*>(A + (4 * rg + a) * LD + k0);          // x[a] = A[row][ks]
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const ulonglong2 w = *reinterpret_cast<const ulonglong2*>(B + (k0 + kk) * LD + 4 * cg);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                float xv;
                if (TA) xv = a == 0 ? x[kk].x : a == 1 ? x[kk].y : a == 2 ? x[kk].z : x[kk].w;
                else    xv = kk == 0 ? x[a].x : kk == 1 ? x[a].y : kk == 2 ? x[a].z : x[a].w;
                const pair_t xx = pack(xv, xv);
                acc[a][0] = fma2(xx, w.x, acc[a][0]);
                acc[a][1] = fma2(xx, w.y, acc[a][1]);
            }
        }
    }
}

// The large product: 256 rows of A at once, a thread 8 rows (8 rg ...) x 8 columns (4 cg ... and 32 + 4 cg ...): a word
// of B read from shared memory serves eight rows and a word of A eight columns (the path from shared memory into the
// registers, not the FMA pipe, is what bounds these loops: 16 words for 128 packed FMAs here, 8 for 32 in mm64).
__device__ __forceinline__ void mm256(const float* A, const float* B, pair_t (&acc)[8][4], int rg, int cg) {
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int h = 0; h < 4; ++h) acc[a][h] = pack(0.0f, 0.0f);
#pragma unroll 1
    for (int k0 = 0; k0 < 64; k0 += 4) {
        float4 x[8];
#pragma unroll
        for (int a = 0; a < 8; ++a) x[a] = *reinterpret_cast<const float4*>(A + (8 * rg + a) * LD + k0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const ulonglong2 w0 = *reinterpret_cast<const ulonglong2*>(B + (k0 + kk) * LD + 4 * cg);
            const ulonglong2 w1 = *reinterpret_cast<const ulonglong2*>(B + (k0 + kk) * LD + 32 + 4 * cg);
#pragma unroll
            for (int a = 0; a < 8; ++a) {
                const float xv = kk == 0 ? x[a].x : kk == 1 ? x[a].y : kk == 2 ? x[a].z : x[a].w;
                const pair_t xx = pack(xv, xv);
                acc[a][0] = fma2(xx, w0.x, acc[a][0]);
                acc[a][1] = fma2(xx, w0.y, acc[a][1]);
                acc[a][2] = fma2(xx, w1.x, acc[a][2]);
                acc[a][3] = fma2(xx, w1.y, acc[a][3]);
            }
        }
    }
}

__device__ __forceinline__ void store_acc(float* dst, const pair_t (&acc)[4][2], int rg, int cg) {
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        float o[4];
        unpack(acc[a][0], o[0], o[1]);
        unpack(acc[a][1], o[2], o[3]);
        *reinterpret_cast<float4*>(dst + (4 * rg + a) * LD + 4 * cg) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

// Four floats of row-major `src` (rows of n floats) at (r, 4 q), zeros outside rows < nr and columns < n
__device__ __forceinline__ float4 fetch4(const float* src, int n, unsigned nr, unsigned r, int q, bool vec) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < nr) {
        const float* s = src + (size_t)r * n + 4 * q;
        if (vec) {
            if (4 * q < n) v = *reinterpret_cast<const float4*>(s);
        } else {
            if (4 * q < n) v.x = s[0];
            if (4 * q + 1 < n) v.y = s[1];
            if (4 * q + 2 < n) v.z = s[2];
            if (4 * q + 3 < n) v.w = s[3];
        }
    }
    return v;
}

constexpr int kDownSmem = (4 * 64 + 128) * LD * (int)sizeof(float);

__global__ void __launch_bounds__(kThreads, 2) tsqr_down_kernel(const DownParams p) {
    extern __shared__ __align__(16) float down_sm[];
    float* Bs = down_sm;                 // B, zeros beyond n
    float* Ws = Bs + 64 * LD;            // T (V1^T B)
    float* Vs = Ws + 64 * LD;            // V's rows 0 .. 127, and behind them, once T and V1^T B are done with, rows 128 .. 255
    float* Ts = Vs + 128 * LD;
    float* Xs = Ts + 64 * LD;            // V1^T B
    const int t = threadIdx.x, rg = t >> 4, cg = t & 15;
    const int n = p.n;
    const unsigned i = blockIdx.x % p.blocks;
    const unsigned long long b = blockIdx.x / p.blocks;
    unsigned start, nrows;
    block_span(i, p.blocks, p.rows, p.d, start, nrows);
    float* V = p.v + b * p.v_outer + (size_t)start * n;
    const size_t blk = (size_t)b * p.blocks + i;
    const float* Bsrc = p.up ? p.up + blk * n * n : nullptr;
    const float* Tsrc = p.t + blk * n * n;
    const bool n4 = (n & 3) == 0;
    const bool vec = n4 && (reinterpret_cast<size_t>(V) & 15) == 0;
    const bool vecb = n4 && (reinterpret_cast<size_t>(Bsrc) & 15) == 0, vect = n4 && (reinterpret_cast<size_t>(Tsrc) & 15) == 0;

    {   // B, T and the first 128 rows of V: every load in flight before the first store
        float4 fb[4], ft[4], fv[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int idx = t + kThreads * k, r = idx >> 4, q = idx & 15;
            if (Bsrc) {
                fb[k] = fetch4(Bsrc, n, (unsigned)n, (unsigned)r, q, vecb);
            } else {
                const int d = r - 4 * q;
                fb[k] = make_float4(d == 0 && r < n ? 1.f : 0.f, d == 1 && r < n ? 1.f : 0.f, d == 2 && r < n ? 1.f : 0.f,
                                    d == 3 && r < n ? 1.f : 0.f);
            }
            ft[k] = fetch4(Tsrc, n, (unsigned)n, (unsigned)r, q, vect);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int idx = t + kThreads * k, r = idx >> 4, q = idx & 15;
            fv[k] = fetch4(V, n, nrows, (unsigned)r, q, vec);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int idx = t + kThreads * k, r = idx >> 4, q = idx & 15;
            *reinterpret_cast<float4*>(Bs + r * LD + 4 * q) = fb[k];
            *reinterpret_cast<float4*>(Ts + r * LD + 4 * q) = ft[k];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int idx = t + kThreads * k, r = idx >> 4, q = idx & 15;
            *reinterpret_cast<float4*>(Vs + r * LD + 4 * q) = fv[k];
        }
    }
    float4 fn[8];       // rows 128 .. 255 of V, fetched under the two small products
    if (nrows > 128) {
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
            const int idx = t + kThreads * q8, r = idx >> 4, q = idx & 15;
            fn[q8] = fetch4(V, n, nrows, 128u + (unsigned)r, q, vec);
        }
    }
    __syncthreads();
    {
        pair_t acc[4][2];
        mm64<true>(Vs, Bs, acc, rg, cg, 4 * rg);  // rows of B beyond n are zero, so only V1 = V's first n rows count
        store_acc(Xs, acc, rg, cg);
        __syncthreads();
        mm64<false>(Ts, Xs, acc, rg, cg, 4 * rg);
        store_acc(Ws, acc, rg, cg);
    }
    __syncthreads();
    // V's rows 128 .. 255 take T's and X's place (fetched under the two small products)
    if (nrows > 128) {
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
            const int idx = t + kThreads * q8, r = idx >> 4, q = idx & 15;
            *reinterpret_cast<float4*>(Ts + r * LD + 4 * q) = fn[q8];
        }
        __syncthreads();
    }
    {
        const int rg8 = t >> 3, cg8 = t & 7;
        pair_t acc[8][4];
        mm256(Vs, Ws, acc, rg8, cg8);
#pragma unroll
        for (int a = 0; a < 8; ++a) {
            const unsigned r = 8 * rg8 + a;
            if (r >= nrows) continue;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float o[4];
                unpack(acc[a][2 * h], o[0], o[1]);
                unpack(acc[a][2 * h + 1], o[2], o[3]);
                const int c = 32 * h + 4 * cg8;
                if (r < 64) {
                    const float4 bv = *reinterpret_cast<const float4*>(Bs + r * LD + c);
                    o[0] = bv.x - o[0]; o[1] = bv.y - o[1]; o[2] = bv.z - o[2]; o[3] = bv.w - o[3];
                } else {
                    o[0] = -o[0]; o[1] = -o[1]; o[2] = -o[2]; o[3] = -o[3];
                }
                float* dst = V + (size_t)r * n + c;
                if (vec && c + 3 < n) {
                    *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (c + e < n) dst[e] = o[e];
                }
            }
        }
    }
}

struct VtLevel {
    uint32_t rows, blocks, d;
};

struct VtLayout {
    std::vector<VtLevel> levels;        // the last is the top: one block
    std::vector<size_t>  s_off, q_off, t_off;     // per level: its input stack (levels >= 1), its V/Q (levels >= 1), its T
    size_t               total = 0;
};

VtLayout vt_layout(uint32_t m, uint32_t n, uint32_t batch, bool want_q) {
    VtLayout L;
    uint32_t rows = m;
    for (;;) {
        VtLevel lv{rows, (rows + kBlockRows - 1) / kBlockRows, 0};
        if (lv.blocks > 1) {
            const uint32_t rem = rows - (lv.blocks - 1) * kBlockRows;
            lv.d = rem < n ? n - rem : 0;
        }
        L.levels.push_back(lv);
        if (lv.blocks == 1) break;
        rows = lv.blocks * n;
    }
    auto up64 = [](size_t f) { return (f + 63) & ~(size_t)63; };
    const size_t nl = L.levels.size();
    L.s_off.assign(nl, 0);
    L.q_off.assign(nl, 0);
    L.t_off.assign(nl, 0);
    for (size_t l = 0; l < nl; ++l) {
        const size_t in_floats = (size_t)batch * L.levels[l].rows * n;
        if (l >= 1) {
            L.s_off[l] = L.total; L.total += up64(in_floats);
            if (want_q) { L.q_off[l] = L.total; L.total += up64(in_floats); }
        }
        if (want_q) { L.t_off[l] = L.total; L.total += up64((size_t)batch * L.levels[l].blocks * n * n); }
    }
    return L;
}

template <int SETS>
void launch_leaf(cudaStream_t stream, const LeafParams& lp, uint64_t grid) {
    static PerDeviceOnce once;
    if (const int device = current_device(); once.first(device)) {
        cuda_check(cudaFuncSetAttribute(tsqr_leaf_kernel<SETS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)sizeof(LeafSmem<SETS>)), "tsqr_leaf shared memory");
        once.mark(device);
    }
    tsqr_leaf_kernel<SETS><<<(unsigned)grid, kThreads, sizeof(LeafSmem<SETS>), stream>>>(lp);
    cuda_check(cudaGetLastError(), "tsqr_leaf launch");
}

} // namespace

bool tsqr_vt_takes(uint32_t m, uint32_t n) {
    const char* e = std::getenv("QR_TSQR_VT");
    return n >= 1 && n <= 64 && m >= n && !(e && e[0] == '0');      // (at most 256 rows: one block, no tree)
}

size_t tsqr_vt_workspace_floats(uint32_t m, uint32_t n, uint32_t batch, bool want_q) {
    return vt_layout(m, n, batch, want_q).total;
}

// Thin QR of `batch` matrices of m x n (n <= 64, m >= n) read with row stride lda and matrix stride a_outer:
// q [batch][m][n] contiguous (null: R alone), r [batch] n x n at stride r_outer.
void tsqr_vt_core(cudaStream_t stream, const float* a, uint32_t lda, uint64_t a_outer, uint32_t m, uint32_t n,
                  uint32_t batch, float* q, float* r, uint64_t r_outer, float* ws) {
    if (batch == 0) return;
    const bool want_q = q != nullptr;
    const VtLayout L = vt_layout(m, n, batch, want_q);
    const size_t nl = L.levels.size();
    for (size_t l = 0; l < nl; ++l) {
        const VtLevel& lv = L.levels[l];
        const bool top = l + 1 == nl;
        LeafParams lp{};
        lp.in = l == 0 ? a : ws + L.s_off[l];
        lp.in_ld = l == 0 ? lda : n;
        lp.in_outer = l == 0 ? a_outer : (uint64_t)lv.rows * n;
        lp.v = !want_q ? nullptr : (l == 0 ? q : ws + L.q_off[l]);
        lp.v_outer = (uint64_t)lv.rows * n;
        lp.t = want_q ? ws + L.t_off[l] : nullptr;
        lp.r = top ? r : ws + L.s_off[l + 1];
        lp.r_outer = top ? r_outer : (uint64_t)lv.blocks * n * n;
        lp.rows = lv.rows; lp.blocks = lv.blocks; lp.d = lv.d;
        lp.n = (int)n;
        const uint64_t grid = (uint64_t)batch * lv.blocks;
        if (n <= 32) launch_leaf<1>(stream, lp, grid);
        else launch_leaf<2>(stream, lp, grid);
    }
    if (!want_q) return;
    static PerDeviceOnce once;
    if (const int device = current_device(); once.first(device)) {
        cuda_check(cudaFuncSetAttribute(tsqr_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDownSmem),
                   "tsqr_down shared memory");
        once.mark(device);
    }
    for (size_t l = nl; l-- > 0;) {
        const VtLevel& lv = L.levels[l];
        DownParams dp{};
        dp.v = l == 0 ? q : ws + L.q_off[l];
        dp.v_outer = (uint64_t)lv.rows * n;
        dp.t = ws + L.t_off[l];
        dp.up = l + 1 == nl ? nullptr : ws + L.q_off[l + 1];
        dp.rows = lv.rows; dp.blocks = lv.blocks; dp.d = lv.d;
        dp.n = (int)n;
        tsqr_down_kernel<<<(unsigned)((uint64_t)batch * lv.blocks), kThreads, kDownSmem, stream>>>(dp);
        cuda_check(cudaGetLastError(), "tsqr_down launch");
    }
}

} // namespace mlb
