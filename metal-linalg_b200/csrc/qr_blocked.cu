// The blocked compact-WY QR: one matrix spread over the whole grid, any shape.
//
// It takes the place of the reference's qr_blocked (src/qr_blocked.mm:56-302 with
// src/band_reduce.mm:196-507 and the panel kernels of shaders/Svd_Bidiag.metal:
// 428-886,1125-1279) and has its structure: a scaled working copy W of the
// matrix; panels of 32 columns gathered in aggregates of 128; R read off W; Q
// formed backward from [I; 0] by the aggregates' block reflectors.
//
//   panel      rows k0..m, columns k0..k0+32 of W to compact-WY form (Y, T, R) by
//              TSQR over row blocks with Householder reconstruction (Ballard,
//              Demmel, Grigori, Jacquelin, Nguyen, Solomonik 2014; the reference:
//              bd_tsqr_top, shaders/Svd_Bidiag.metal:757-802): the register-resident
//              kernels of qr_panel.cu up to 16384 rows, the general tree
//              (tsqr_core + reconstruct_kernel here) beyond;
//   inside     the panel's reflector applied to the columns left in its aggregate
//              (at most 96) by inner_z_kernel + inner_apply_kernel;
//   aggregate  T of the aggregate's 128 reflectors from its panels' T's and the
//              Gram matrix Y^T Y (merge_t_kernel; the reference: bd_merge_t), then
//              the rank-128 update of everything right of it, C -= Y (T^T (Y^T C)):
//              Zp = Y^T C by row chunks and C -= Y Z on the tcgen05 tensor cores by
//              3xTF32 (tc_gemm.cu), the chunks summed and multiplied by T^T in
//              between (reduce_t_wide_kernel). QR_TENSOR=0 runs both products as
//              FP32 FMA kernels instead (ytc_wide_kernel, yz_wide_kernel): the
//              fallback with plain float32 rounding.
//
// The chain of panels runs on a high-priority stream of its own; after an
// aggregate it updates only the next aggregate's columns itself and leaves the
// columns beyond to the caller's stream, where that update runs beside the next
// panels (look-ahead).
//
// Y is kept apart from W (clean: unit diagonal, zeros above) so that the products
// read it as a plain matrix.
#include "common.cuh"
#include "kernels.h"
#include "tc_split.cuh"

#include <algorithm>
#include <cstdlib>
#include <vector>

namespace mlb {

namespace {

constexpr int NB  = 32;     // panel width

struct MatInfo {            // per matrix, written by the scan
    unsigned amax_bits;     // bit pattern of the largest magnitude (non-negative floats order as integers)
    unsigned bad;           // bit 0: a NaN or an infinity was seen; kStatusTensorWait: a tensor-core product gave
                            // up on a bounded wait. Either way the matrix's outputs are NaN.
};

__global__ void scan_kernel(const float* a, size_t count, MatInfo* info) {
    float amax = 0.0f;
    int   bad = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const float v = a[i];
        amax = fmaxf(amax, fabsf(v));
        bad |= nonfinite(v);
    }
    amax = warp_max(amax);
    bad = __any_sync(0xffffffffu, bad);
    if ((threadIdx.x & 31) == 0) {
        if (bad) atomicOr(&info->bad, 1u);
        else atomicMax(&info->amax_bits, __float_as_uint(amax));
    }
}

__device__ __forceinline__ int info_exponent(const MatInfo* info) {
    return info->bad ? 0 : amax_exponent(__uint_as_float(info->amax_bits));
}

// W (ld ldw) = A * 2^-e
__global__ void scale_copy_kernel(const float* a, float* w, uint32_t m, uint32_t n, uint32_t ldw, const MatInfo* info) {
    const Pow2 down(-info_exponent(info));
    const size_t total = (size_t)m * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / n, c = i % n;
        w[r * ldw + c] = down(a[i]);
    }
}

// R [rr][n] = the upper trapezoid of W's first K rows * 2^e, zeros elsewhere; NaN for a non-finite matrix
// and a wait that ran out during the factorisation is passed on to the context's status word
__global__ void r_out_kernel(const float* w, uint32_t ldw, float* r, uint32_t rr, uint32_t n, uint32_t K,
                             const MatInfo* info, unsigned* status) {
    const Pow2 up(info_exponent(info));
    const bool bad = info->bad != 0;
    if (blockIdx.x == 0 && threadIdx.x == 0 && (info->bad & kStatusTensorWait)) atomicOr(status, (unsigned)kStatusTensorWait);
    const size_t total = (size_t)rr * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / n, c = i % n;
        float v = (row < K && c >= row) ? up(w[row * ldw + c]) : 0.0f;
        r[i] = bad ? qnan() : v;
    }
}

__global__ void nan_fill_kernel(float* q, size_t count, const MatInfo* info) {
    if (!info->bad) return;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        q[i] = qnan();
}

// ---------------------------------------------------------------------------
// Householder reconstruction of one panel (one warp)
// ---------------------------------------------------------------------------
struct ReconParams {
    const float* qp;        // [mp][jb] explicit thin Q of the panel
    const float* rp;        // [jb][jb] its R
    float*       w;         // the working copy: the panel's R (S Rp) goes to rows/cols k0..
    float*       y;         // Y: the unit lower triangular top block goes to rows k0..k0+jb, columns k0..
    float*       t;         // [32][32] T, zero padded
    float*       uinv;      // [jb][jb] U^-1, for the rows below the top block
    uint32_t     ldw, ldy, k0, jb;
};

__global__ void __launch_bounds__(32) reconstruct_kernel(const ReconParams p) {
    __shared__ float M[32][33], Ui[32][33], Tm[32][33];
    __shared__ float sgn[32];
    const int i = threadIdx.x, jb = (int)p.jb;
    for (int c = 0; c < 32; ++c) {
        M[i][c] = (i < jb && c < jb) ? p.qp[(size_t)i * jb + c] : (i == c ? 1.0f : 0.0f);
        Ui[i][c] = 0.0f;
        Tm[i][c] = 0.0f;
    }
    __syncwarp();
    // LU of Q1 - S, S = -sgn(pivot) chosen at each step: every pivot has magnitude >= 1
    for (int j = 0; j < jb; ++j) {
        const float d = M[j][j];
        const float s = d >= 0.0f ? -1.0f : 1.0f;
        const float piv = d - s;
        __syncwarp();
        if (i == j) {
            M[j][j] = piv;
            sgn[j] = s;
        }
        float l = 0.0f;
        if (i > j && i < jb) {
            l = M[i][j] / piv;
            M[i][j] = l;
        }
        __syncwarp();
        if (i > j && i < jb)
            for (int c = j + 1; c < jb; ++c) M[i][c] = fmaf(-l, M[j][c], M[i][c]);
        __syncwarp();
    }
    // U^-1, a column per lane: U x = e_c by back substitution
    if (i < jb) {
        const int c = i;
        float x[32];
#pragma unroll
        for (int r = 31; r >= 0; --r) {
            float v = 0.0f;
            if (r <= c && r < jb) {
                float acc = r == c ? 1.0f : 0.0f;
#pragma unroll
                for (int k = r + 1; k < 32; ++k)
                    if (k <= c) acc = fmaf(-M[r][k], x[k], acc);
                v = acc / M[r][r];
            }
            x[r] = v;
        }
#pragma unroll
        for (int r = 0; r < 32; ++r)
            if (r < jb) Ui[r][c] = x[r];
    }
    __syncwarp();
    // T = -U S L1^-T: row i of T from T L1^T = -U S, forward over the columns
    if (i < jb) {
        float t[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float v = 0.0f;
            if (c >= i && c < jb) {
                float acc = -M[i][c] * sgn[c];
#pragma unroll
                for (int k = 0; k < c; ++k)
                    if (k >= i) acc = fmaf(-t[k], M[c][k], acc);   // L1[c][k], k < c
                v = acc;
            }
            t[c] = v;
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) Tm[i][c] = t[c];
    }
    __syncwarp();
    for (int c = 0; c < 32; ++c) p.t[i * 32 + c] = Tm[i][c];
    if (i < jb) {
        for (int c = 0; c < jb; ++c) {
            p.uinv[(size_t)i * jb + c] = Ui[i][c];
            // Y's top block: unit lower triangular L1
            p.y[(size_t)(p.k0 + i) * p.ldy + p.k0 + c] = c < i ? M[i][c] : (c == i ? 1.0f : 0.0f);
            // the panel's R: S Rp, upper triangular (the part of W below it is never read)
            if (c >= i) p.w[(size_t)(p.k0 + i) * p.ldw + p.k0 + c] = sgn[i] * p.rp[(size_t)i * jb + c];
        }
    }
}

// ---------------------------------------------------------------------------
// Block reflector application for an aggregate of up to 128 reflectors: three kernels
// ---------------------------------------------------------------------------
constexpr int AG  = 128;    // columns per aggregate (four panels)
constexpr int WCH = 512;    // rows per chunk of the wide Y^T C partial sums

// Zp[chunk][i][j] = sum over the chunk's rows r of Y[r][i] C[r][j]; i < 128 (columns of Y from kw on
// read as zero), j < nc. Grid (ceil(nc / 128), chunks); a thread accumulates 8 x 8.
__global__ void __launch_bounds__(256) ytc_wide_kernel(const float* __restrict__ Y, size_t ldy,
                                                       const float* __restrict__ C, size_t ldc, uint32_t mp, uint32_t kw,
                                                       uint32_t nc, float* Zp, uint32_t ncp) {
    dependency_wait_only();
    __shared__ __align__(16) float Ys[32][132];
    __shared__ __align__(16) float Cs[32][132];
    const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
    const uint32_t j0 = blockIdx.x * 128;
    const uint32_t r_begin = blockIdx.y * WCH, r_end = min(mp, r_begin + WCH);
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0.0f;
    for (uint32_t r0 = r_begin; r0 < r_end; r0 += 32) {
        __syncthreads();
#pragma unroll 4
        for (int e = 0; e < 16; ++e) {
            const int idx = threadIdx.x + 256 * e;
            const uint32_t r = r0 + (idx >> 7), c = idx & 127;
            Ys[idx >> 7][c] = (r < r_end && c < kw) ? Y[(size_t)r * ldy + c] : 0.0f;
            Cs[idx >> 7][c] = (r < r_end && j0 + c < nc) ? C[(size_t)r * ldc + j0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int r = 0; r < 32; ++r) {
            const float4 y0 = *reinterpret_cast<const float4*>(&Ys[r][8 * tr]);
            const float4 y1 = *reinterpret_cast<const float4*>(&Ys[r][8 * tr + 4]);
            const float4 c0 = *reinterpret_cast<const float4*>(&Cs[r][8 * tc]);
            const float4 c1 = *reinterpret_cast<const float4*>(&Cs[r][8 * tc + 4]);
            const float yv[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
            const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(yv[a], cv[b], acc[a][b]);
        }
    }
    float* out = Zp + (size_t)blockIdx.y * AG * ncp;
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const uint32_t j = j0 + 8 * tc + b;
            if (j < nc) out[(size_t)(8 * tr + a) * ncp + j] = acc[a][b];
        }
}

// Z[i][j] = sum_k op(T)[i][k] (sum_chunks Zp[chunk][k][j]), T 128 x 128. Grid ceil(nc / 32).
// Dynamic shared memory: op(T) transposed [128][132] and the summed chunks [128][36].
// zsp non-null: the result goes out split into its tf32 parts, in the layout the second product's bulk copies fetch
// (the stages of its kw rows), instead of as Z: a thread holds four consecutive rows of four columns, a word each.
__global__ void __launch_bounds__(256) reduce_t_wide_kernel(const float* __restrict__ Zp, uint32_t chunks, uint32_t nc,
                                                            uint32_t ncp, const float* __restrict__ T, int transposed,
                                                            float* Z, float* zsp, uint32_t kw) {
    dependency_wait_only();
    extern __shared__ __align__(16) float dsm[];
    float (*Tt)[132] = reinterpret_cast<float (*)[132]>(dsm);                // Tt[k][i] = op(T)[i][k]
    float (*Zs)[36]  = reinterpret_cast<float (*)[36]>(dsm + 128 * 132);
    const uint32_t j0 = blockIdx.x * 32;
    // Both operands are fetched many loads at a time (sixteen of T; a thread's sixteen entries of four chunks): read
    // one by one in a loop, every load waited for L2 (37 us a launch at 4096 x 4096, most of it those waits).
    for (int base = 0; base < 128 * 128; base += 16 * 256) {
        float tv[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) tv[u] = T[base + threadIdx.x + 256 * u];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int idx = base + threadIdx.x + 256 * u, a = idx >> 7, c = idx & 127;      // T[a][c]
            if (transposed) Tt[a][c] = tv[u];      // Tt[k][i] = op(T)[i][k] = T[k][i]
            else Tt[c][a] = tv[u];                 // Tt[k][i] = T[i][k]
        }
    }
    {
        float sum[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) sum[e] = 0.0f;
        const uint32_t j = j0 + (threadIdx.x & 31);
        if (j < nc) {
            const float* src = Zp + (size_t)(threadIdx.x >> 5) * ncp + j;      // entry e: row k = (threadIdx.x >> 5) + 8 e
            const size_t step = (size_t)AG * ncp;
            uint32_t ch = 0;
            for (; ch + 4 <= chunks; ch += 4) {      // the chunks are added in order, four at a time in flight
                float v[4][16];
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[c][e] = src[(size_t)(ch + c) * step + (size_t)8 * e * ncp];
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int e = 0; e < 16; ++e) sum[e] += v[c][e];
            }
            for (; ch < chunks; ++ch) {
                float v[16];
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = src[(size_t)ch * step + (size_t)8 * e * ncp];
#pragma unroll
                for (int e = 0; e < 16; ++e) sum[e] += v[e];
            }
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) Zs[(threadIdx.x >> 5) + 8 * e][threadIdx.x & 31] = sum[e];
    }
    __syncthreads();
    const int ig = threadIdx.x >> 3, jg = threadIdx.x & 7;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
#pragma unroll 4
    for (int k = 0; k < 128; ++k) {
        const float4 t4 = *reinterpret_cast<const float4*>(&Tt[k][4 * ig]);
        const float4 z0 = *reinterpret_cast<const float4*>(&Zs[k][4 * jg]);
        const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
        const float zv[4] = {z0.x, z0.y, z0.z, z0.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(tv[a], zv[b], acc[a][b]);
    }
    if (zsp) {
        const uint32_t stages = (kw + tcsplit::kStageK - 1) / tcsplit::kStageK, k0 = 4 * ig;
        if (k0 < tcsplit::kStageK * stages) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t j = j0 + 4 * jg + b;
                const float v[4] = {k0 < kw ? acc[0][b] : 0.0f, k0 + 1 < kw ? acc[1][b] : 0.0f, k0 + 2 < kw ? acc[2][b] : 0.0f,
                                    k0 + 3 < kw ? acc[3][b] : 0.0f};      // rows from kw on are zero
                if (j < nc) tcsplit::store_word(zsp, stages, j, (uint32_t)ig, v);
            }
        }
        return;
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t j = j0 + 4 * jg + b;
            if (j < nc) Z[(size_t)(4 * ig + a) * ncp + j] = acc[a][b];
        }
}

// The same for a narrow update (the look-ahead's 128 columns): eight columns a block, so that a
// narrow Z still spreads over many blocks; T is read from global memory (L2) as it is.
// Grid ceil(nc / 8); thread (i, half) computes Z[i][4 half .. + 3] of the block's eight columns.
__global__ void __launch_bounds__(1024) reduce_t_narrow_kernel(const float* __restrict__ Zp, uint32_t chunks, uint32_t nc,
                                                              uint32_t ncp, const float* __restrict__ T, int transposed,
                                                              float* Z) {
    dependency_wait();
    __shared__ __align__(16) float Zs[128][8];
    extern __shared__ __align__(16) float dsm_narrow[];
    float (*Tt)[129] = reinterpret_cast<float (*)[129]>(dsm_narrow);       // Tt[k][i] = op(T)[i][k]
    const uint32_t j0 = blockIdx.x * 8;
    {   // T into shared memory, sixteen entries a thread, all in flight together (read from global memory entry by
        // entry inside the product below, every step of its 128 waited for L2)
        float tv[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) tv[u] = T[threadIdx.x + 1024 * u];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int idx = threadIdx.x + 1024 * u, a = idx >> 7, b = idx & 127;      // T[a][b]
            if (transposed) Tt[a][b] = tv[u];      // op(T)[i][k] = T[k][i]: Tt[k][i] = T[k][i]
            else Tt[b][a] = tv[u];                 // op(T)[i][k] = T[i][k]: Tt[k][i] = T[i][k]
        }
    }
    {   // 1024 threads, an entry each, eight loads in flight; the chunks are added in order
        const int idx = threadIdx.x;
        const uint32_t k = idx >> 3, j = j0 + (idx & 7);
        float sum = 0.0f;
        if (j < nc) {
            const float* src = Zp + (size_t)k * ncp + j;
            const size_t step = (size_t)AG * ncp;
            uint32_t ch = 0;
            for (; ch + 8 <= chunks; ch += 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = src[(size_t)(ch + u) * step];
#pragma unroll
                for (int u = 0; u < 8; ++u) sum += v[u];
            }
            for (; ch < chunks; ++ch) sum += src[(size_t)ch * step];
        }
        Zs[k][idx & 7] = sum;
    }
    __syncthreads();
    if (threadIdx.x >= 256) return;
    const int i = threadIdx.x & 127, h = threadIdx.x >> 7;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int k = 0; k < 128; ++k) {
        const float t = Tt[k][i];
        const float4 z = *reinterpret_cast<const float4*>(&Zs[k][4 * h]);
        acc[0] = fmaf(t, z.x, acc[0]); acc[1] = fmaf(t, z.y, acc[1]);
        acc[2] = fmaf(t, z.z, acc[2]); acc[3] = fmaf(t, z.w, acc[3]);
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint32_t j = j0 + 4 * h + b;
        if (j < nc) Z[(size_t)i * ncp + j] = acc[b];
    }
}

// C[r][j] -= sum_k Y[r][k] Z[k][j], k < kw <= 128. Grid (ceil(nc / 128), ceil(mp / 128)); a thread owns 8 x 8.
__global__ void __launch_bounds__(256) yz_wide_kernel(const float* __restrict__ Y, size_t ldy,
                                                      const float* __restrict__ Z, uint32_t ncp, float* C, size_t ldc,
                                                      uint32_t mp, uint32_t kw, uint32_t nc) {
    dependency_wait_only();
    __shared__ __align__(16) float Ys[32][132];   // [k][row]
    __shared__ __align__(16) float Zs[32][128];   // [k][col]
    const uint32_t j0 = blockIdx.x * 128, r0 = blockIdx.y * 128;
    const int tr = threadIdx.x >> 4, tc = threadIdx.x & 15;
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0.0f;
    for (uint32_t k0 = 0; k0 < kw; k0 += 32) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < 128 * 32; idx += 256) {
            const uint32_t r = idx >> 5, k = idx & 31;
            Ys[k][r] = (r0 + r < mp && k0 + k < kw) ? Y[(size_t)(r0 + r) * ldy + k0 + k] : 0.0f;
        }
        for (int idx = threadIdx.x; idx < 32 * 128; idx += 256) {
            const uint32_t k = idx >> 7, j = idx & 127;
            Zs[k][j] = (j0 + j < nc && k0 + k < kw) ? Z[(size_t)(k0 + k) * ncp + j0 + j] : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int k = 0; k < 32; ++k) {
            const float4 y0 = *reinterpret_cast<const float4*>(&Ys[k][8 * tr]);
            const float4 y1 = *reinterpret_cast<const float4*>(&Ys[k][8 * tr + 4]);
            const float4 z0 = *reinterpret_cast<const float4*>(&Zs[k][8 * tc]);
            const float4 z1 = *reinterpret_cast<const float4*>(&Zs[k][8 * tc + 4]);
            const float yv[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
            const float zv[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(yv[a], zv[b], acc[a][b]);
        }
    }
    const bool vec = (ldc & 3) == 0 && (reinterpret_cast<size_t>(C) & 15) == 0 && j0 + 8 * tc + 8 <= nc;
#pragma unroll
    for (int a = 0; a < 8; ++a) {
        const uint32_t r = r0 + 8 * tr + a;
        if (r >= mp) continue;
        float* row = C + (size_t)r * ldc + j0 + 8 * tc;
        if (vec) {
            float4 c0 = *reinterpret_cast<float4*>(row), c1 = *reinterpret_cast<float4*>(row + 4);
            c0.x -= acc[a][0]; c0.y -= acc[a][1]; c0.z -= acc[a][2]; c0.w -= acc[a][3];
            c1.x -= acc[a][4]; c1.y -= acc[a][5]; c1.z -= acc[a][6]; c1.w -= acc[a][7];
            *reinterpret_cast<float4*>(row) = c0;
            *reinterpret_cast<float4*>(row + 4) = c1;
        } else {
#pragma unroll
            for (int b = 0; b < 8; ++b)
                if (j0 + 8 * tc + b < nc) row[b] -= acc[a][b];
        }
    }
}

// T of an aggregate (128 x 128, zero padded) from its panels' T's and the Gram matrix of its Y:
// T(0:c, c:c+32) = -T(0:c, 0:c) (Y(:, 0:c)^T Y_q) T_q for each panel q after the first
// (the reference: bd_merge_t, shaders/Svd_Bidiag.metal:1131-1164). One block; dynamic shared memory.
// The chunks' partial Gram matrices added up into the first one, an entry per thread.
__global__ void gram_sum_kernel(float* zp, uint32_t chunks, uint32_t count) {
    dependency_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float g0 = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f;
    uint32_t ch = 0;
    for (; ch + 4 <= chunks; ch += 4) {
        g0 += zp[(size_t)ch * count + i];
        g1 += zp[(size_t)(ch + 1) * count + i];
        g2 += zp[(size_t)(ch + 2) * count + i];
        g3 += zp[(size_t)(ch + 3) * count + i];
    }
    for (; ch < chunks; ++ch) g0 += zp[(size_t)ch * count + i];
    zp[i] = (g0 + g1) + (g2 + g3);
}

struct MergeParams {
    const float* gram;      // the Gram matrix [128][gld] (null when there is one panel)
    uint32_t     chunks, gld;
    const float* tp;        // the panels' T's, [panels][32][32]
    uint32_t     panels;
    float*       tagg;      // [128][128]
};

// One block: its time is the latency of its loads and stores, so it is given every thread a block may have.
constexpr int kMergeThreads = 1024;

__global__ void __launch_bounds__(kMergeThreads) merge_t_kernel(const MergeParams p) {
    dependency_wait();
    extern __shared__ __align__(16) float dsm[];
    float (*Ta)[129] = reinterpret_cast<float (*)[129]>(dsm);
    float (*G)[129]  = reinterpret_cast<float (*)[129]>(dsm + 128 * 129);
    float (*X)[33]   = reinterpret_cast<float (*)[33]>(dsm + 2 * 128 * 129);
    const int t = threadIdx.x;
    const int width = 32 * (int)p.panels;
    {   // a thread's sixteen entries of each matrix are fetched before the first is stored: one trip to L2, not sixteen
        constexpr int kPer = 128 * 128 / kMergeThreads;
        float tv[kPer], gv[kPer];
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int idx = t + u * kMergeThreads, i = idx >> 7, j = idx & 127;
            tv[u] = 0.0f;
            if ((i >> 5) == (j >> 5) && (uint32_t)(i >> 5) < p.panels) tv[u] = p.tp[(size_t)(i >> 5) * 1024 + (i & 31) * 32 + (j & 31)];
            // the Gram matrix, already summed over the chunks (gram_sum_kernel)
            gv[u] = (p.gram && i < width && j < width && (uint32_t)j < p.gld) ? p.gram[(size_t)i * p.gld + j] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int idx = t + u * kMergeThreads, i = idx >> 7, j = idx & 127;
            Ta[i][j] = tv[u];
            G[i][j] = gv[u];
        }
    }
    __syncthreads();
    for (uint32_t q = 1; q < p.panels; ++q) {
        const int c0 = 32 * (int)q;
        for (int idx = t; idx < c0 * 32; idx += kMergeThreads) {      // X = G(0:c0, c0:c0+32) T_q
            const int i = idx >> 5, c = idx & 31;
            float a = 0.0f;
#pragma unroll 8
            for (int k = 0; k < 32; ++k) a = fmaf(G[i][c0 + k], Ta[c0 + k][c0 + c], a);
            X[i][c] = a;
        }
        __syncthreads();
        for (int idx = t; idx < c0 * 32; idx += kMergeThreads) {
            const int i = idx >> 5, c = idx & 31;
            float a = 0.0f;
            for (int k = i; k < c0; ++k) a = fmaf(Ta[i][k], X[k][c], a);   // T is upper triangular
            Ta[i][c0 + c] = -a;
        }
        __syncthreads();
    }
    for (int idx = t; idx < 128 * 128; idx += kMergeThreads) p.tagg[idx] = Ta[idx >> 7][idx & 127];
}

// The two large products run on the tensor cores (3xTF32, tc_gemm.cu) unless QR_TENSOR=0 asks for
// the FP32 FMA kernels above, which stay as the fallback.
bool use_tensor_cores() {
    const char* e = std::getenv("QR_TENSOR");
    return !(e && e[0] == '0');
}

constexpr size_t kReduceWideSmem = (128 * 132 + 128 * 36) * sizeof(float);
constexpr size_t kReduceNarrowSmem = 128 * 129 * sizeof(float);
constexpr size_t kMergeSmem = (2 * 128 * 129 + 96 * 33) * sizeof(float);

// C (mp rows, nc columns) <- (I - Y op(T) Y^T) C for an aggregate: Y mp x kw (kw <= 128), T 128 x 128.
// ysp, zsp: scratch for the split operands of a wide update's second product (null: the product splits
// its operands as it goes; QR_TC_SPLIT=0 asks for that everywhere).
void apply_aggregate(cudaStream_t stream, const float* Y, size_t ldy, const float* T, bool transposed, float* C,
                     size_t ldc, uint32_t mp, uint32_t kw, uint32_t nc, float* zp, float* z, unsigned* error,
                     float* ysp = nullptr, float* zsp = nullptr, float* ytsp = nullptr) {
    if (nc == 0 || mp == 0) return;
    const uint32_t ncp = (nc + 3) & ~3u;
    const bool tc = use_tensor_cores();
    // a narrow update (the look-ahead's) in short row chunks, so that it still fills the GPU
    const bool narrow = tc && nc <= 256;
    // QR_TC_SPLIT=0: the products whose blocks split their operands as they load them
    const char* split_env = std::getenv("QR_TC_SPLIT");
    const bool split = tc && !narrow && ysp && zsp && ytsp && !(split_env && split_env[0] == '0');
    // rows a tensor-core accumulator sums over (the accumulation truncates: chains are kept short); the split-operand
    // product's blocks take two such runs of rows each, in two accumulators (QR_TC_PAIR=0: one)
    const char* chunk_env = std::getenv("QR_TC_CHUNK");
    const uint32_t sub_rows = chunk_env && std::atoi(chunk_env) >= 256 ? (uint32_t)std::atoi(chunk_env) / 256 * 256 : 256u;
    // ... where that still leaves two waves of blocks (two a multiprocessor): at 4096 x 4096 the halved grid is a single
    // wave of longer blocks and the product takes 37 instead of 29 us
    const char* pair_env = std::getenv("QR_TC_PAIR");
    const bool pair = split && (pair_env ? pair_env[0] != '0'
                                         : (uint64_t)((mp + 2 * sub_rows - 1) / (2 * sub_rows)) * ((nc + 127) / 128) >= 4 * 148);
    const uint32_t wide_rows = pair ? 2 * sub_rows : sub_rows;
    const uint32_t rows = narrow ? 128u : tc ? wide_rows : (uint32_t)WCH;
    const uint32_t chunks = (mp + rows - 1) / rows;
    if (split) launch_tc_ytc_split(stream, Y, ldy, C, ldc, mp, kw, nc, zp, ncp, rows, sub_rows, ytsp, error, ysp);      // both splits of Y
    else if (tc) launch_tc_ytc(stream, Y, ldy, C, ldc, mp, kw, nc, zp, ncp, rows, error);
    else launch_dependent(ytc_wide_kernel, dim3((nc + 127) / 128, chunks), 256, 0, stream, Y, ldy, C, ldc, mp, kw, nc, zp, ncp);
    if (narrow) launch_dependent(reduce_t_narrow_kernel, (nc + 7) / 8, 1024, kReduceNarrowSmem, stream, zp, chunks, nc, ncp, T, transposed ? 1 : 0, z);
    else launch_dependent(reduce_t_wide_kernel, (nc + 31) / 32, 256, kReduceWideSmem, stream, zp, chunks, nc, ncp, T, transposed ? 1 : 0, z,
                          split ? zsp : (float*)nullptr, kw);
    if (split) launch_tc_yz_split(stream, (const float*)nullptr, ldy, (const float*)nullptr, ncp, C, ldc, mp, kw, nc, ysp, zsp, error);
    else if (tc) launch_tc_yz(stream, Y, ldy, z, ncp, C, ldc, mp, kw, nc, error);
    else launch_dependent(yz_wide_kernel, dim3((nc + 127) / 128, (mp + 127) / 128), 256, 0, stream, Y, ldy, z, ncp, C, ldc, mp, kw, nc);
    cuda_check(cudaGetLastError(), "aggregate reflector launch");
}

// T of the aggregate whose Y starts at `Y` (ma rows, wa columns, `panels` panels with T's at tp).
void build_aggregate_t(cudaStream_t stream, const float* Y, size_t ldy, uint32_t ma, uint32_t wa, uint32_t panels,
                       const float* tp, float* tagg, float* zp, unsigned* error) {
    MergeParams mp{nullptr, 0, 0, tp, panels, tagg};
    if (panels > 1) {
        // the Gram matrix Y^T Y by chunks of rows (short chunks on the tensor cores: the product is
        // small and tall, and many blocks hide its latency)
        const uint32_t rows = use_tensor_cores() ? 128u : (uint32_t)WCH;
        const uint32_t chunks = (ma + rows - 1) / rows, gld = (wa + 3) & ~3u;
        if (use_tensor_cores()) launch_tc_ytc(stream, Y, ldy, Y, ldy, ma, wa, wa, zp, gld, rows, error);
        else launch_dependent(ytc_wide_kernel, dim3(1, chunks), 256, 0, stream, Y, ldy, Y, ldy, ma, wa, wa, zp, gld);
        launch_dependent(gram_sum_kernel, (AG * gld + 255) / 256, 256, 0, stream, zp, chunks, AG * gld);
        mp.gram = zp; mp.chunks = chunks; mp.gld = gld;
    }
    launch_dependent(merge_t_kernel, 1, kMergeThreads, kMergeSmem, stream, mp);
    cuda_check(cudaGetLastError(), "aggregate T launch");
}

// ---------------------------------------------------------------------------
// A panel's own update: its reflector applied to the few columns left in its aggregate
// ---------------------------------------------------------------------------
// C (mp x nc, nc <= 96) <- (I - Y T^T Y^T) C in two launches over a grid of (4 columns) x (1024
// rows). inner_z_kernel: a block's part of Z = Y^T C (32 x 4), a thread taking four rows in
// registers, summed over the block (shuffles, then shared memory), to zpart[row chunk].
// inner_apply_kernel: every block sums the row chunks' parts for its columns (a fixed order, so
// the result does not depend on scheduling), W = T^T Z, and C -= Y W on its rows.
constexpr int ICS = 4;          // columns per block
constexpr int IRB = 1024;       // rows per block

__device__ __forceinline__ void inner_load_y(float (&y)[32], const float* yr, bool yvec, uint32_t jb) {
    if (yvec) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 f = *reinterpret_cast<const float4*>(yr + 4 * q);
            y[4 * q] = f.x; y[4 * q + 1] = f.y; y[4 * q + 2] = f.z; y[4 * q + 3] = f.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) y[k] = (uint32_t)k < jb ? yr[k] : 0.0f;
    }
}

// zpart [row chunks][32][ncp]
__global__ void __launch_bounds__(256) inner_z_kernel(const float* __restrict__ Y, size_t ldy, const float* __restrict__ C,
                                                      size_t ldc, uint32_t mp, uint32_t jb, uint32_t nc, float* zpart,
                                                      uint32_t ncp) {
    dependency_wait();
    __shared__ float red[8][32 * ICS];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t c0 = blockIdx.x * ICS, ncb = min((uint32_t)ICS, nc - c0);
    const uint32_t r_begin = blockIdx.y * IRB, r_end = min(mp, r_begin + IRB);
    const bool yvec = (ldy & 3) == 0 && jb == 32 && (reinterpret_cast<size_t>(Y) & 15) == 0;
    float z[32][ICS];
#pragma unroll
    for (int k = 0; k < 32; ++k)
#pragma unroll
        for (int j = 0; j < ICS; ++j) z[k][j] = 0.0f;
    for (uint32_t r = r_begin + t; r < r_end; r += 256) {
        float y[32], c[ICS];
        inner_load_y(y, Y + (size_t)r * ldy, yvec, jb);
#pragma unroll
        for (int j = 0; j < ICS; ++j) c[j] = (uint32_t)j < ncb ? C[(size_t)r * ldc + c0 + j] : 0.0f;
#pragma unroll
        for (int k = 0; k < 32; ++k)
#pragma unroll
            for (int j = 0; j < ICS; ++j) z[k][j] = fmaf(y[k], c[j], z[k][j]);
    }
    // block sum of the 128 numbers: per column j a 32-value butterfly (lane k ends with the warp's z[k][j])
#pragma unroll
    for (int j = 0; j < ICS; ++j) {
        float pcol[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) pcol[k] = z[k][j];
#pragma unroll
        for (int half = 16; half >= 1; half >>= 1) {
            const bool upper = (lane & half) != 0;
#pragma unroll
            for (int i = 0; i < half; ++i) {
                const float send = upper ? pcol[i] : pcol[i + half];
                const float keep = upper ? pcol[i + half] : pcol[i];
                pcol[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
            }
        }
        red[warp][lane * ICS + j] = pcol[0];
    }
    __syncthreads();
    if (t < 32 * ICS) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][t];
        const uint32_t k = t / ICS, j = t % ICS;
        if (j < ncb) zpart[((size_t)blockIdx.y * 32 + k) * ncp + c0 + j] = v;
    }
}

__global__ void __launch_bounds__(256) inner_apply_kernel(const float* __restrict__ Y, size_t ldy,
                                                          const float* __restrict__ T, float* C, size_t ldc, uint32_t mp,
                                                          uint32_t jb, uint32_t nc, const float* __restrict__ zpart,
                                                          uint32_t ncp, uint32_t chunks) {
    dependency_wait();
    __shared__ float Zs[32][ICS], Ws[32][ICS];
    __shared__ float Ts[32][33];
    const int t = threadIdx.x;
    const uint32_t c0 = blockIdx.x * ICS, ncb = min((uint32_t)ICS, nc - c0);
    const uint32_t r_begin = blockIdx.y * IRB, r_end = min(mp, r_begin + IRB);
    const bool yvec = (ldy & 3) == 0 && jb == 32 && (reinterpret_cast<size_t>(Y) & 15) == 0;
    for (int idx = t; idx < 1024; idx += 256) Ts[idx >> 5][idx & 31] = T[idx];
    if (t < 32 * ICS) {
        const uint32_t k = t / ICS, j = t % ICS;
        float v = 0.0f;
        if (j < ncb)
            for (uint32_t ch = 0; ch < chunks; ++ch) v += zpart[((size_t)ch * 32 + k) * ncp + c0 + j];
        Zs[k][j] = v;
    }
    __syncthreads();
    if (t < 32 * ICS) {     // W = T^T Z
        const int i = t / ICS, j = t % ICS;
        float v = 0.0f;
#pragma unroll 8
        for (int k = 0; k < 32; ++k) v = fmaf(Ts[k][i], Zs[k][j], v);
        Ws[i][j] = v;
    }
    __syncthreads();
    float w[32][ICS];
#pragma unroll
    for (int k = 0; k < 32; ++k)
#pragma unroll
        for (int j = 0; j < ICS; ++j) w[k][j] = Ws[k][j];
    for (uint32_t r = r_begin + t; r < r_end; r += 256) {
        float y[32];
        inner_load_y(y, Y + (size_t)r * ldy, yvec, jb);
        float d[ICS];
#pragma unroll
        for (int j = 0; j < ICS; ++j) d[j] = 0.0f;
#pragma unroll
        for (int k = 0; k < 32; ++k)
#pragma unroll
            for (int j = 0; j < ICS; ++j) d[j] = fmaf(y[k], w[k][j], d[j]);
#pragma unroll
        for (int j = 0; j < ICS; ++j)
            if ((uint32_t)j < ncb) C[(size_t)r * ldc + c0 + j] -= d[j];
    }
}

// The two kernels above in one launch, for panels of at most 8 x 1024 rows: the blocks of a column group (one per
// 1024 rows) form a thread-block cluster, every block stores its part of Z = Y^T C into the shared memory of all of
// them (distributed shared memory), and after one cluster barrier each sums the parts in the same fixed order and
// applies W = T^T Z to its own rows. One launch and no round trip through global memory between the halves.
constexpr int kInnerCluster = 8;
constexpr int kInnerYld = 36;           // floats between a thread's rows of Y in shared memory and the next thread's: 16-byte words, conflict-free
constexpr size_t kInnerSmem = (size_t)IRB * kInnerYld * sizeof(float);

__device__ __forceinline__ uint32_t inner_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t inner_cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}

__global__ void __launch_bounds__(256) inner_fused_kernel(const float* __restrict__ Y, size_t ldy, const float* __restrict__ T,
                                                          float* C, size_t ldc, uint32_t mp, uint32_t jb, uint32_t nc) {
    dependency_wait();
    // every block of the cluster has started once this barrier's wait (below, before the remote stores) returns
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    __shared__ float red[8][32 * ICS];
    __shared__ float parts[kInnerCluster][32 * ICS];      // parts[r]: the part of the cluster's block r, stored by that block
    __shared__ float Zs[32][ICS], Ws[32][ICS];
    __shared__ float Ts[32][33];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t rank = inner_cluster_rank(), nblk = inner_cluster_size();
    const uint32_t c0 = blockIdx.x * ICS, ncb = min((uint32_t)ICS, nc - c0);
    const uint32_t r_begin = blockIdx.y * IRB, r_end = min(mp, r_begin + IRB);
    const bool yvec = (ldy & 3) == 0 && jb == 32 && (reinterpret_cast<size_t>(Y) & 15) == 0;
    // Y's rows of this block go to shared memory once, by 16-byte asynchronous copies that are all in flight together
    // (eight consecutive lanes a row: whole 128-byte lines; a lane a row asked for every line eight times over), and
    // serve both passes; C's entries stay in registers from the first pass to the second. (Read row by row from global
    // memory, in both passes, the block waited for L2 eight times over.)
    extern __shared__ __align__(16) float inner_ys[];       // [IRB][kInnerYld]: row r_begin + i at i * kInnerYld
    float cv[IRB / 256][ICS];
    if (yvec) {
#pragma unroll 8
        for (int i = 0; i < IRB * 8 / 256; ++i) {
            const uint32_t idx = t + 256 * i, rl = idx >> 3, q = idx & 7, r = r_begin + rl;
            if (r < r_end) {
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(inner_ys + (size_t)rl * kInnerYld + 4 * q);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(Y + (size_t)r * ldy + 4 * q) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const bool cvec = (ldc & 3) == 0 && ncb == (uint32_t)ICS && ICS == 4 && (reinterpret_cast<size_t>(C + c0) & 15) == 0;
#pragma unroll
    for (int i = 0; i < IRB / 256; ++i) {
        const uint32_t r = r_begin + t + 256 * i;
        if (cvec) {
            const float4 f = r < r_end ? *reinterpret_cast<const float4*>(C + (size_t)r * ldc + c0) : make_float4(0.f, 0.f, 0.f, 0.f);
            cv[i][0] = f.x; cv[i][1] = f.y; cv[i][2] = f.z; cv[i][3] = f.w;
        } else {
#pragma unroll
            for (int j = 0; j < ICS; ++j) cv[i][j] = (r < r_end && (uint32_t)j < ncb) ? C[(size_t)r * ldc + c0 + j] : 0.0f;
        }
    }
    float tv[4];                                            // T on its way to shared memory while Z is formed
#pragma unroll
    for (int u = 0; u < 4; ++u) tv[u] = T[t + 256 * u];
    float z[32][ICS];
#pragma unroll
    for (int k = 0; k < 32; ++k)
#pragma unroll
        for (int j = 0; j < ICS; ++j) z[k][j] = 0.0f;
    if (yvec) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();      // a row's eight words came from eight threads
    }
#pragma unroll
    for (int i = 0; i < IRB / 256; ++i) {
        const uint32_t r = r_begin + t + 256 * i;
        if (r < r_end) {
            float y[32];
            if (yvec) inner_load_y(y, inner_ys + (size_t)(i * 256 + t) * kInnerYld, true, jb);
            else inner_load_y(y, Y + (size_t)r * ldy, false, jb);
#pragma unroll
            for (int k = 0; k < 32; ++k)
#pragma unroll
                for (int j = 0; j < ICS; ++j) z[k][j] = fmaf(y[k], cv[i][j], z[k][j]);
        }
    }
#pragma unroll
    for (int j = 0; j < ICS; ++j) {
        float pcol[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) pcol[k] = z[k][j];
#pragma unroll
        for (int half = 16; half >= 1; half >>= 1) {
            const bool upper = (lane & half) != 0;
#pragma unroll
            for (int i = 0; i < half; ++i) {
                const float send = upper ? pcol[i] : pcol[i + half];
                const float keep = upper ? pcol[i + half] : pcol[i];
                pcol[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
            }
        }
        red[warp][lane * ICS + j] = pcol[0];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) Ts[(t + 256 * u) >> 5][(t + 256 * u) & 31] = tv[u];
    __syncthreads();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (t < 32 * ICS) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][t];
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(&parts[rank][t]);
        for (uint32_t r = 0; r < nblk; ++r) {
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(r));
            asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(remote), "f"(v) : "memory");
        }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (t < 32 * ICS) {
        float v = 0.0f;
        for (uint32_t r = 0; r < nblk; ++r) v += parts[r][t];      // the same order in every block
        Zs[t / ICS][t % ICS] = (uint32_t)(t % ICS) < ncb ? v : 0.0f;
    }
    __syncthreads();
    if (t < 32 * ICS) {     // W = T^T Z
        const int i = t / ICS, j = t % ICS;
        float v = 0.0f;
#pragma unroll 8
        for (int k = 0; k < 32; ++k) v = fmaf(Ts[k][i], Zs[k][j], v);
        Ws[i][j] = v;
    }
    __syncthreads();
    float w[32][ICS];
#pragma unroll
    for (int k = 0; k < 32; ++k)
#pragma unroll
        for (int j = 0; j < ICS; ++j) w[k][j] = Ws[k][j];
#pragma unroll
    for (int i = 0; i < IRB / 256; ++i) {
        const uint32_t r = r_begin + t + 256 * i;
        if (r < r_end) {
            float y[32];
            if (yvec) inner_load_y(y, inner_ys + (size_t)(i * 256 + t) * kInnerYld, true, jb);
            else inner_load_y(y, Y + (size_t)r * ldy, false, jb);
            float d[ICS];
#pragma unroll
            for (int j = 0; j < ICS; ++j) d[j] = 0.0f;
#pragma unroll
            for (int k = 0; k < 32; ++k)
#pragma unroll
                for (int j = 0; j < ICS; ++j) d[j] = fmaf(y[k], w[k][j], d[j]);
            if (cvec) {
                *reinterpret_cast<float4*>(C + (size_t)r * ldc + c0) =
                    make_float4(cv[i][0] - d[0], cv[i][1] - d[1], cv[i][2] - d[2], cv[i][3] - d[3]);
            } else {
#pragma unroll
                for (int j = 0; j < ICS; ++j)
                    if ((uint32_t)j < ncb) C[(size_t)r * ldc + c0 + j] = cv[i][j] - d[j];
            }
        }
    }
}

// zpart: scratch of at least ceil(mp / 1024) * 32 * ((nc + 3) & ~3) floats
void apply_inner(cudaStream_t stream, const float* Y, size_t ldy, const float* T, float* C, size_t ldc, uint32_t mp,
                 uint32_t jb, uint32_t nc, float* zpart) {
    if (nc == 0 || mp == 0) return;
    const uint32_t chunks = (mp + IRB - 1) / IRB, ncp = (nc + 3) & ~3u;
    const dim3 grid((nc + ICS - 1) / ICS, chunks);
    const char* fused_env = std::getenv("QR_INNER_FUSED");      // QR_INNER_FUSED=0: the two kernels
    const bool fused = !(fused_env && fused_env[0] == '0');
    if (fused && chunks <= (uint32_t)kInnerCluster) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = kInnerSmem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = chunks;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = dependent_launches_enabled() ? 2 : 1;
        cuda_check(cudaLaunchKernelEx(&cfg, inner_fused_kernel, Y, ldy, T, C, ldc, mp, jb, nc), "inner update launch");
        return;
    }
    launch_dependent(inner_z_kernel, grid, 256, 0, stream, Y, ldy, C, ldc, mp, jb, nc, zpart, ncp);
    launch_dependent(inner_apply_kernel, grid, 256, 0, stream, Y, ldy, T, C, ldc, mp, jb, nc, zpart, ncp, chunks);
    cuda_check(cudaGetLastError(), "inner update launch");
}

// A square n x n row-major matrix transposed in place: a block swaps the 32 x 32 tile (bx, by) with
// the tile (by, bx), through shared memory (by <= bx; the others leave at once).
__global__ void __launch_bounds__(256) transpose_inplace_kernel(float* a, uint32_t n) {
    __shared__ float t0[32][33], t1[32][33];
    const uint32_t bx = blockIdx.x, by = blockIdx.y;
    if (by > bx) return;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (uint32_t r = ty; r < 32; r += 8) {
        const uint32_t i0 = by * 32 + r, j0 = bx * 32 + tx;      // tile (by, bx)
        t0[r][tx] = (i0 < n && j0 < n) ? a[(size_t)i0 * n + j0] : 0.0f;
        const uint32_t i1 = bx * 32 + r, j1 = by * 32 + tx;      // tile (bx, by)
        t1[r][tx] = (i1 < n && j1 < n) ? a[(size_t)i1 * n + j1] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (uint32_t r = ty; r < 32; r += 8) {
        const uint32_t i0 = by * 32 + r, j0 = bx * 32 + tx;
        if (i0 < n && j0 < n) a[(size_t)i0 * n + j0] = t1[tx][r];
        const uint32_t i1 = bx * 32 + r, j1 = by * 32 + tx;
        if (bx != by && i1 < n && j1 < n) a[(size_t)i1 * n + j1] = t0[tx][r];
    }
}

unsigned grid_for(size_t count) { return (unsigned)std::min<size_t>((count + 255) / 256, 148 * 8); }

} // namespace

bool qr_blocked_fits(uint32_t m, uint32_t n) {
    return m > 0 && n > 0 && (uint64_t)m * n < ((uint64_t)1 << 31) && (uint64_t)m * std::min(m, n) < ((uint64_t)1 << 31);
}

void launch_qr_blocked(DeviceContext& ctx, cudaStream_t stream, const QrProblem& pr) {
    if (pr.batch == 0) return;
    const uint32_t m = pr.m, n = pr.n, K = qr_k(pr), qc = pr.qc, rr = pr.rr;
    const uint32_t ldw = (n + 3) & ~3u, ldy = (K + 3) & ~3u;
    const uint32_t npanels = (K + NB - 1) / NB;
    const uint32_t wide = std::max(n, qc);                       // the widest matrix a reflector is applied to
    const uint32_t ncp = (wide + 3) & ~3u;

    // workspace (floats), shared by the matrices of the batch, which are factored one after another
    const uint32_t naggs = (K + AG - 1) / AG;
    auto up64 = [](size_t f) { return (f + 63) & ~(size_t)63; };
    size_t off = 0;
    auto take = [&](size_t floats) { const size_t o = off; off += up64(floats); return o; };
    const size_t o_w = take((size_t)m * ldw), o_y = take((size_t)m * ldy), o_t = take((size_t)npanels * 1024);
    const size_t o_ta = take((size_t)naggs * AG * AG);
    const size_t o_qp = take((size_t)m * NB), o_rp = take(NB * NB), o_ui = take(NB * NB);
    const size_t gram_floats = (size_t)((m + 127) / 128) * AG * AG;   // the Gram partials of an aggregate, 128 rows a chunk
    // partial sums Y^T C: 512-row chunks of the full width, or 128-row chunks of a narrow (<= 256 columns) update
    const size_t zp_floats = std::max({(size_t)((m + 255) / 256) * AG * ncp, gram_floats,
                                       (size_t)((m + 127) / 128) * AG * std::min<size_t>(ncp, 256)});
    const size_t o_zp = take(zp_floats);
    const size_t o_z = take((size_t)AG * ncp);
    const size_t o_zp2 = take(zp_floats), o_z2 = take((size_t)AG * ncp);   // the second stream's
    const size_t o_ysp = take(tc_split_floats(m)), o_zsp = take(tc_split_floats(ncp)), o_ytsp = take(tc_split_t_floats(m));   // split operands of the wide updates
    // the inner updates' partial sums where they take two kernels (more than eight chunks of rows, or QR_INNER_FUSED=0): the
    // chain's own and the look-ahead stream's, which run side by side
    const size_t inner_floats = (size_t)((m + 1023) / 1024) * 32 * 2 * AG;
    const size_t o_zi = take(inner_floats), o_zi2 = take(inner_floats);
    const size_t o_info = take(64);
    size_t tsqr_floats = 0;
    for (uint32_t k0 = 0; k0 < K; k0 += NB)
        if (!panel_fast_fits(m - k0, std::min<uint32_t>(NB, K - k0)))
            tsqr_floats = std::max(tsqr_floats, tsqr_workspace_floats(ctx, m - k0, std::min<uint32_t>(NB, K - k0), 1, true));
    const size_t o_ts = take(tsqr_floats);
    const size_t o_pf = take(panel_fast_workspace_floats(std::min<uint32_t>(m, 16384)));
    const bool slow_panels = std::getenv("QR_PANEL_TREE") != nullptr;   // the general tree for every panel, for comparison
    const bool look_ahead = std::getenv("QR_NO_LOOKAHEAD") == nullptr;
    // A batch of large matrices is factored several at a time, each on its own pair of streams and
    // its own slice of the workspace: one matrix's chain of panel kernels keeps a handful of
    // multiprocessors busy, and the others' updates fill the rest.
    uint32_t nlanes = 1;
    if (pr.batch > 1 && naggs > 1) {
        const char* e = std::getenv("QR_BLOCKED_LANES");
        const size_t budget = (size_t)6 << 30;   // bytes of workspace
        const size_t fit = std::max<size_t>(1, budget / (off * sizeof(float)));
        nlanes = (uint32_t)std::min<size_t>({(size_t)pr.batch, (size_t)DeviceContext::kExtraLanes + 1, fit});
        if (e && std::atoi(e) >= 1) nlanes = std::min<uint32_t>(nlanes, (uint32_t)std::atoi(e));
    }
    float* ws_all = static_cast<float*>(ctx.workspace(stream, (size_t)nlanes * off * sizeof(float)));
    static PerDeviceOnce once;      // the opt-in is recorded per GPU
    if (once.first(ctx.device)) {
        cuda_check(cudaFuncSetAttribute(reduce_t_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kReduceWideSmem), "reduce_t_wide shared memory");
        cuda_check(cudaFuncSetAttribute(merge_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMergeSmem),
                   "merge_t shared memory");
        cuda_check(cudaFuncSetAttribute(reduce_t_narrow_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)kReduceNarrowSmem), "reduce_t_narrow shared memory");
        cuda_check(cudaFuncSetAttribute(inner_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kInnerSmem),
                   "inner_fused shared memory");
        once.mark(ctx.device);
    }
    const cudaStream_t caller = stream;
    if (nlanes > 1) {      // the extra lanes start after what the caller's stream holds
        for (uint32_t l = 1; l < nlanes; ++l) ctx.lane(l - 1);
        cuda_check(cudaEventRecord(ctx.ev_fork, caller), "cudaEventRecord");
        for (uint32_t l = 1; l < nlanes; ++l)
            cuda_check(cudaStreamWaitEvent(ctx.lane(l - 1).update, ctx.ev_fork, 0), "cudaStreamWaitEvent");
    }

    for (uint32_t b = 0; b < pr.batch; ++b) {
        const float* A = pr.a + (size_t)b * m * n;
        float* Q = qc ? pr.q + (size_t)b * m * qc : nullptr;
        float* R = pr.r + (size_t)b * rr * n;
        // this matrix's lane: streams, events, workspace
        const uint32_t ln = b % nlanes;
        const cudaStream_t stream = ln ? ctx.lane(ln - 1).update : caller;
        const cudaStream_t panel_stream = ln ? ctx.lane(ln - 1).panel : ctx.aux;
        const cudaStream_t look_stream = ln ? ctx.lane(ln - 1).look : ctx.look;
        cudaEvent_t* const ev_look = ln ? ctx.lane(ln - 1).ev_look : ctx.ev_look;
        cudaEvent_t* const ev_panel  = ln ? ctx.lane(ln - 1).ev_panel : ctx.ev_panel;
        cudaEvent_t* const ev_update = ln ? ctx.lane(ln - 1).ev_update : ctx.ev_update;
        float* ws = ws_all + (size_t)ln * off;
        float *W = ws + o_w, *Y = ws + o_y, *T = ws + o_t, *Ta = ws + o_ta, *Qp = ws + o_qp, *Rp = ws + o_rp, *Ui = ws + o_ui;
        float *Zp = ws + o_zp, *Z = ws + o_z, *Zp2 = ws + o_zp2, *Z2 = ws + o_z2, *ts = ws + o_ts, *pf = ws + o_pf;
        float *Ysp = ws + o_ysp, *Zsp = ws + o_zsp, *Ytsp = ws + o_ytsp, *Zi = ws + o_zi, *Zi2 = ws + o_zi2;
        MatInfo* info = reinterpret_cast<MatInfo*>(ws + o_info);

        cuda_check(cudaMemsetAsync(info, 0, sizeof(MatInfo), stream), "cudaMemsetAsync");
        if (take_injected_wait_failure())      // a test's stand-in for a wait that ran out: every byte of `bad` = the bit
            cuda_check(cudaMemsetAsync(&info->bad, (int)kStatusTensorWait, sizeof(unsigned), stream), "cudaMemsetAsync");
        scan_kernel<<<grid_for((size_t)m * n), 256, 0, stream>>>(A, (size_t)m * n, info);
        scale_copy_kernel<<<grid_for((size_t)m * n), 256, 0, stream>>>(A, W, m, n, ldw, info);

        // forward. Panels of 32 columns in aggregates of 128: a panel's reflector is applied at once
        // only to the columns left in its aggregate; the columns right of the aggregate get all of
        // its (up to) 128 reflectors in one rank-128 update.
        //
        // Look-ahead: the chain of panels runs on the context's high-priority stream `ps`, the large
        // updates on the caller's stream `us`. After an aggregate's panels, `ps` itself updates only
        // the next aggregate's columns, so that its panels can start; the columns beyond go to `us`
        // and run beside those panels. Updates of one column range stay in order: before its own
        // update `ps` waits for the previous update on `us`, which covered the same columns.
        cudaStream_t ps = look_ahead && naggs > 1 ? panel_stream : stream, us = stream;
        const bool two = ps != us;
        if (two) {
            cuda_check(cudaEventRecord(ev_update[1], us), "cudaEventRecord");        // the working copy is ready
            cuda_check(cudaStreamWaitEvent(ps, ev_update[1], 0), "cudaStreamWaitEvent");
        }
        // A square Q is accumulated FORWARD, beside the panels: P = Q^T = H_{K-1}^T ... H_0^T I takes each
        // aggregate's reflectors from the left as soon as they are formed (the same product as the
        // trailing update's, on all m columns), on the update stream, which the chain of panels leaves
        // idle most of the time; Q is P transposed in place at the end. It costs 2 m^3 flops where the
        // backward accumulation below costs 4/3 m^3, but those ran after the last panel with nothing
        // beside them (3 of 17 ms at 4096 x 4096; 15.2 ms with the forward accumulation). Not for a batch
        // of matrices beyond 4096 rows, whose lanes keep the update streams full already (four 8192 x
        // 8192: 34 ms a matrix backward, 38 ms forward). Orthogonality at 4096 x 4096 by 3xTF32: 8e-4
        // against 4e-4 backward (bound 4.9e-3): every entry of P takes every aggregate's update.
        // QR_BACKWARD_Q=1 keeps the backward accumulation.
        const bool forward_q = two && qc == m && (nlanes == 1 || m <= 4096) && std::getenv("QR_BACKWARD_Q") == nullptr;
        if (forward_q) launch_fill_identity(us, Q, 1, m, m);
        // Look-ahead by panels (QR_LOOK_PANELS=0: by aggregates, below): a third stream `ls` keeps the NEXT aggregate's
        // columns up to date panel by panel (the same inner update, on those 128 columns, as soon as a panel is
        // factored), builds the aggregate's T and applies the aggregate to the columns of the aggregate after the
        // next; the wide update on `us` starts beyond those. The chain on `ps` is then panels and their updates
        // inside the aggregate only: the next aggregate's first panel waits for the last of the third stream's inner
        // updates, not for the Gram matrix, the merge of the T's and a rank-128 update behind them.
        // It costs more work in all (four inner updates of 128 columns an aggregate beside the rank-128 update), so it
        // is for a matrix whose chain of panels is what bounds it: one matrix of at most 6144 rows, or whose wide
        // updates are light (no Q to accumulate, or at most 4096 columns of A and Q). One B200, ms, by panels / by
        // aggregates: 1024^2 1.19 / 1.55, 2048^2 2.53 / 3.23, 4096^2 6.61 / 7.64, 5120^2 10.5 / 11.2, 6144^2 15.5 / 15.6,
        // 8192^2 30.2 / 28.7 but R alone 17.9 / 19.3 and 8192 x 2048 5.63 / 6.01; eight 4096^2 42.0 / 35.1.
        // QR_LOOK_PANELS=1 asks for it everywhere, =0 nowhere.
        const char* deep_env = std::getenv("QR_LOOK_PANELS");
        const bool deep = two && (deep_env ? deep_env[0] != '0' : (nlanes == 1 && (m <= 6144 || qc == 0 || std::max(n, qc) <= 4096)));
        const cudaStream_t ls = look_stream;
        if (deep) cuda_check(cudaStreamWaitEvent(ls, ev_update[1], 0), "cudaStreamWaitEvent");       // the working copy is ready
        for (uint32_t ag = 0; ag < naggs; ++ag) {
            const uint32_t j0 = ag * AG, wa = std::min<uint32_t>(AG, K - j0), ma = m - j0, pans = (wa + NB - 1) / NB;
            const uint32_t right = n - (j0 + wa);
            const uint32_t s1 = deep ? std::min<uint32_t>(AG, right) : 0;            // the next aggregate's columns
            const uint32_t s2 = deep ? std::min<uint32_t>(AG, right - s1) : 0;       // and those of the one after
            if (deep && ag > 0) cuda_check(cudaStreamWaitEvent(ps, ev_look[1], 0), "cudaStreamWaitEvent");   // this aggregate's columns are complete
            for (uint32_t pp = 0; pp < pans; ++pp) {
                const uint32_t pi = ag * (AG / NB) + pp, k0 = pi * NB, jb = std::min<uint32_t>(NB, K - k0), mp = m - k0;
                if (!slow_panels && panel_fast_fits(mp, jb)) {
                    panel_factor_fast(ps, W + (size_t)k0 * ldw + k0, ldw, mp, jb, Y + (size_t)k0 * ldy + k0, ldy,
                                      T + (size_t)pi * 1024, pf, &info->bad);
                } else {   // taller than the register-resident panel kernels take: the general tree
                    tsqr_core(ctx, ps, W + (size_t)k0 * ldw + k0, ldw, 0, mp, jb, 1, Qp, Rp, 0, ts);
                    ReconParams rp{Qp, Rp, W, Y, T + (size_t)pi * 1024, Ui, ldw, ldy, k0, jb};
                    reconstruct_kernel<<<1, 32, 0, ps>>>(rp);
                    if (mp > jb)   // the rows below the top block: Qp U^-1
                        launch_tsqr_apply(ctx, ps, Qp + (size_t)jb * jb, 0, 0, Y + (size_t)(k0 + jb) * ldy + k0, 0, 0,
                                          ldy, Ui, true, 1, 1, mp - jb, mp - jb, jb);
                }
                if (pp)   // Y is read as one mp x wa matrix by the aggregate's products: zeros above the panel's top
                    cuda_check(cudaMemset2DAsync(Y + (size_t)j0 * ldy + k0, (size_t)ldy * sizeof(float), 0,
                                                 jb * sizeof(float), k0 - j0, ps), "cudaMemset2DAsync");
                if (deep) {      // the panel's reflector to the next aggregate's columns, beside the chain
                    cuda_check(cudaEventRecord(ev_look[0], ps), "cudaEventRecord");
                    cuda_check(cudaStreamWaitEvent(ls, ev_look[0], 0), "cudaStreamWaitEvent");
                    if (s1)
                        apply_inner(ls, Y + (size_t)k0 * ldy + k0, ldy, T + (size_t)pi * 1024,
                                    W + (size_t)k0 * ldw + j0 + wa, ldw, mp, jb, s1, Zi2);
                }
                const uint32_t inside = j0 + wa - (k0 + jb);   // columns of the aggregate right of the panel
                if (inside)
                    apply_inner(ps, Y + (size_t)k0 * ldy + k0, ldy, T + (size_t)pi * 1024,
                                W + (size_t)k0 * ldw + k0 + jb, ldw, mp, jb, inside, Zi);
            }
            if (deep) {
                cuda_check(cudaEventRecord(ev_look[1], ls), "cudaEventRecord");      // the next aggregate's columns are complete
                if (right || qc) {
                    build_aggregate_t(ls, Y + (size_t)j0 * ldy + j0, ldy, ma, wa, pans, T + (size_t)ag * (AG / NB) * 1024,
                                      Ta + (size_t)ag * AG * AG, Zp, &info->bad);
                    cuda_check(cudaEventRecord(ev_look[2], ls), "cudaEventRecord");
                    cuda_check(cudaStreamWaitEvent(us, ev_look[2], 0), "cudaStreamWaitEvent");
                }
                if (s2) {      // the aggregate to the columns of the aggregate after the next, which the previous wide update covered
                    if (ag > 0) cuda_check(cudaStreamWaitEvent(ls, ev_update[(ag - 1) & 1], 0), "cudaStreamWaitEvent");
                    apply_aggregate(ls, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                    W + (size_t)j0 * ldw + j0 + wa + s1, ldw, ma, wa, s2, Zp, Z, &info->bad);
                }
                if (right > s1 + s2)
                    apply_aggregate(us, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                    W + (size_t)j0 * ldw + j0 + wa + s1 + s2, ldw, ma, wa, right - s1 - s2, Zp2, Z2, &info->bad,
                                    Ysp, Zsp, Ytsp);
                cuda_check(cudaEventRecord(ev_update[ag & 1], us), "cudaEventRecord");
                if (forward_q)
                    apply_aggregate(us, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                    Q + (size_t)j0 * m, m, ma, wa, m, Zp2, Z2, &info->bad, Ysp, Zsp, Ytsp);
                continue;
            }
            if (right || qc)
                build_aggregate_t(ps, Y + (size_t)j0 * ldy + j0, ldy, ma, wa, pans, T + (size_t)ag * (AG / NB) * 1024,
                                  Ta + (size_t)ag * AG * AG, Zp, &info->bad);
            if (right && !two) {
                apply_aggregate(us, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                W + (size_t)j0 * ldw + j0 + wa, ldw, ma, wa, right, Zp, Z, &info->bad, Ysp, Zsp, Ytsp);
            } else if (right) {
                const uint32_t next = std::min<uint32_t>(AG, right);
                if (ag > 0) cuda_check(cudaStreamWaitEvent(ps, ev_update[(ag - 1) & 1], 0), "cudaStreamWaitEvent");
                apply_aggregate(ps, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                W + (size_t)j0 * ldw + j0 + wa, ldw, ma, wa, next, Zp, Z, &info->bad);
                cuda_check(cudaEventRecord(ev_panel[ag & 1], ps), "cudaEventRecord");
                cuda_check(cudaStreamWaitEvent(us, ev_panel[ag & 1], 0), "cudaStreamWaitEvent");
                if (right > next)
                    apply_aggregate(us, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                    W + (size_t)j0 * ldw + j0 + wa + next, ldw, ma, wa, right - next, Zp2, Z2, &info->bad,
                                    Ysp, Zsp, Ytsp);
                cuda_check(cudaEventRecord(ev_update[ag & 1], us), "cudaEventRecord");
                if (forward_q)
                    apply_aggregate(us, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                    Q + (size_t)j0 * m, m, ma, wa, m, Zp2, Z2, &info->bad, Ysp, Zsp, Ytsp);
            } else if (forward_q) {      // the last aggregate: nothing right of it, but P takes it too
                cuda_check(cudaEventRecord(ev_panel[ag & 1], ps), "cudaEventRecord");
                cuda_check(cudaStreamWaitEvent(us, ev_panel[ag & 1], 0), "cudaStreamWaitEvent");
                apply_aggregate(us, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, true,
                                Q + (size_t)j0 * m, m, ma, wa, m, Zp2, Z2, &info->bad, Ysp, Zsp, Ytsp);
            }
        }
        if (deep) {   // the caller's stream joins the look-ahead stream too
            cuda_check(cudaEventRecord(ev_look[2], ls), "cudaEventRecord");
            cuda_check(cudaStreamWaitEvent(us, ev_look[2], 0), "cudaStreamWaitEvent");
        }
        if (two) {   // the caller's stream joins the panel stream
            cuda_check(cudaEventRecord(ev_panel[0], ps), "cudaEventRecord");
            cuda_check(cudaStreamWaitEvent(us, ev_panel[0], 0), "cudaStreamWaitEvent");
        }
        r_out_kernel<<<grid_for((size_t)rr * n), 256, 0, stream>>>(W, ldw, R, rr, n, K, info, ctx.status);
        if (!qc) continue;

        if (forward_q) {
            const uint32_t tiles = (m + 31) / 32;
            transpose_inplace_kernel<<<dim3(tiles, tiles), 256, 0, stream>>>(Q, m);
        } else {
            // backward: Q = H_0 ... H_{K-1} [I; 0], an aggregate at a time
            launch_fill_identity(stream, Q, 1, m, qc);
            for (uint32_t ag = naggs; ag-- > 0;) {
                const uint32_t j0 = ag * AG, wa = std::min<uint32_t>(AG, K - j0), ma = m - j0;
                apply_aggregate(stream, Y + (size_t)j0 * ldy + j0, ldy, Ta + (size_t)ag * AG * AG, false,
                                Q + (size_t)j0 * qc + j0, qc, ma, wa, qc - j0, Zp, Z, &info->bad, Ysp, Zsp, Ytsp);
            }
        }
        nan_fill_kernel<<<grid_for((size_t)m * qc), 256, 0, stream>>>(Q, (size_t)m * qc, info);
    }
    for (uint32_t l = 1; l < nlanes; ++l) {      // the caller's stream waits for the extra lanes
        cuda_check(cudaEventRecord(ctx.lane(l - 1).ev_done, ctx.lane(l - 1).update), "cudaEventRecord");
        cuda_check(cudaStreamWaitEvent(caller, ctx.lane(l - 1).ev_done, 0), "cudaStreamWaitEvent");
    }
    cuda_check(cudaGetLastError(), "qr_blocked launch");
}

} // namespace mlb
