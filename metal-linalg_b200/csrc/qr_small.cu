// The small-matrix kernel: a matrix of at most 32 x 32 in the registers of one
// warp, or of a half or a quarter of one (two or four matrices a warp).
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
// product is a reduction across lanes. Here a lane holds a COLUMN (R rows of it
// in registers), so a reflector's dot products with the columns right of it are
// each lane's own FMAs with no reduction at all. What crosses lanes is the
// reflector: the lane that owns column j writes it to shared memory once (16
// bytes an instruction) and every lane reads it back as broadcast 16-byte words,
// four rows an instruction; it stays there for the Q pass, which therefore only
// reads. The arithmetic on rows is packed two to an instruction (fma.rn.f32x2,
// the Blackwell packed FP32 FMA). The reflector is kept unnormalised, H = I - g v
// v^T with v = (alpha - beta; tail): one reciprocal a column, no pass to scale the
// tail, and the pivot row is updated by the same packed instructions as the rest.
//
// The kernel is bound by instruction issue, not by memory (its DRAM traffic is
// the algorithmic 12 KB per 32 x 32 matrix), so the design minimises warp
// instructions per matrix: about 2 per row and step while factoring (one packed
// FMA each for the dot product, the reflector's norm and the update, a quarter
// load, a quarter store) and 1.25 while forming Q.
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

// Two floats in one 64-bit register, the operand form of the packed FP32 FMA. Keeping rows
// packed from load to store (and moving them through shared memory packed) is what makes a packed
// FMA cost one issue slot: built from separate 32-bit registers it needs a move per operand.
typedef unsigned long long pair_t;
__device__ __forceinline__ pair_t pack(float lo, float hi) {
    pair_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack(pair_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ float lo_of(pair_t v) { float a, b; unpack(v, a, b); return a; }
__device__ __forceinline__ float hi_of(pair_t v) { float a, b; unpack(v, a, b); return b; }
__device__ __forceinline__ float hsum(pair_t v) { float a, b; unpack(v, a, b); return a + b; }
__device__ __forceinline__ pair_t fma2(pair_t a, pair_t b, pair_t c) {
    pair_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// a / b to within an ulp or so from the reciprocal and one Newton step (b normal, not tiny)
__device__ __forceinline__ float fast_div(float a, float b) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(b));
    const float q = a * r;
    return fmaf(fmaf(-b, q, a), r, q);
}

// The reflector of a column (alpha; tail) whose tail has sum of squares ss, unnormalised:
// H = I - g v v^T with v = (v1; tail), v1 = alpha - beta, g = 1 / (beta (beta - alpha)) and
// beta = -sign(alpha) ||(alpha; tail)||, LAPACK's slarfg with v not divided by v1 (the same
// reflector, one reciprocal instead of two). g = 0 (H = I, beta = alpha) for a tail taken as zero.
__device__ __forceinline__ void fast_reflector(float alpha, float ss, float& beta, float& v1, float& g) {
    beta = alpha;
    v1   = 0.0f;
    g    = 0.0f;
    if (ss >= kTinySumsq) {
        const float n2 = fmaf(alpha, alpha, ss);
        const float y = rsqrtf(n2);
        float nrm = n2 * y;
        nrm = fmaf(fmaf(-nrm, nrm, n2), 0.5f * y, nrm);
        beta = -copysignf(nrm, alpha);
        v1   = alpha - beta;
        g    = fast_div(-1.0f, beta * v1);
    }
}

// R: rows held per lane (row capacity, a multiple of 4). G: lanes per matrix (column capacity).
// Shared memory per matrix: for each of min(R, G) reflectors its vector v over the R rows (zeros
// above the diagonal), then one float per reflector (g).
template <int R, int G>
__global__ void __launch_bounds__(256, 3) qr_small_kernel(const SmallParams p) {
    constexpr int kSteps = R < G ? R : G;
    constexpr int NQ = R / 4;              // 16-byte words per column
    constexpr int kSlot = kSteps * R + kSteps + (4 - kSteps % 4) % 4;   // floats per matrix, a multiple of 4
    extern __shared__ __align__(16) float smem[];
    const int lane  = threadIdx.x & 31;
    const int l     = lane % G;          // this lane's column
    const uint32_t group = threadIdx.x / G;                       // matrix slot within the block
    uint32_t mat = blockIdx.x * (blockDim.x / G) + group;
    const bool live = mat < p.batch;
    if (!live) mat = p.batch - 1;        // keeps the group in step with the warp; stores are masked
    const int m = p.m, n = p.n, K = p.K;
    ulonglong2* V = reinterpret_cast<ulonglong2*>(smem + (size_t)group * kSlot);   // [kSteps][NQ] words
    float* Vg = smem + (size_t)group * kSlot + kSteps * R;

    const float* src = p.a + (size_t)mat * m * n;

    // 1. load, scan, scale; rows 2p and 2p+1 packed in x2[p]
    pair_t x2[R / 2];
    float amax = 0.0f;
    bool  bad  = false;
    {
        float x[R];
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
        // a non-finite matrix is replaced by zeros, which keeps the arithmetic quiet; its outputs are NaN
        const Pow2 down(bad ? 0 : -amax_exponent(amax));
#pragma unroll
        for (int i = 0; i < R / 2; ++i)
            x2[i] = bad ? pack(0.0f, 0.0f) : pack(down(x[2 * i]), down(x[2 * i + 1]));
    }
    const int expo = bad ? 0 : amax_exponent(amax);

    // 2. factor. Step j: the owner of column j (lane j) takes the norm of its tail, forms the
    // reflector and publishes v = (v1; tail) (zeros above row j) and g; every lane then applies
    // H = I - g v v^T to rows >= j of its own column. No lane is masked: in the owner's column the
    // update leaves beta in row j (up to rounding), and the lanes left of j hold nothing live in
    // rows >= j (their R entries are above, their reflectors already published).
#pragma unroll
    for (int j = 0; j < kSteps; ++j) {
        if (j < K) {
            const int q0 = j / 4;          // first word that holds a row >= j
            {
                pair_t n2 = pack(0.0f, 0.0f), n2b = pack(0.0f, 0.0f);   // two chains, half the latency
                float alo, ahi;
                unpack(x2[j / 2], alo, ahi);
                const float alpha = (j & 1) ? ahi : alo;
                if (!(j & 1)) n2 = pack(0.0f, ahi * ahi);          // row j + 1 shares row j's pair
#pragma unroll
                for (int pi = j / 2 + 1; pi < R / 2; ++pi) {
                    if (pi & 1) n2b = fma2(x2[pi], x2[pi], n2b);
                    else n2 = fma2(x2[pi], x2[pi], n2);
                }
                float beta, v1, g;
                fast_reflector(alpha, hsum(n2) + hsum(n2b), beta, v1, g);
                if (l == j) {
#pragma unroll
                    for (int q = q0; q < NQ; ++q) {
                        pair_t a = x2[2 * q], b = x2[2 * q + 1];
                        if (q == q0) {         // v1 in row j, zeros above it
                            const int e = j & 3;
                            if (e == 0) a = pack(v1, hi_of(a));
                            else if (e == 1) a = pack(0.0f, v1);
                            else if (e == 2) { a = pack(0.0f, 0.0f); b = pack(v1, hi_of(b)); }
                            else { a = pack(0.0f, 0.0f); b = pack(0.0f, v1); }
                        }
                        V[j * NQ + q] = make_ulonglong2(a, b);
                    }
                    Vg[j] = g;
                }
            }
            __syncwarp();
            ulonglong2 u[NQ];
            pair_t s2 = pack(0.0f, 0.0f), s2b = pack(0.0f, 0.0f);
#pragma unroll
            for (int q = q0; q < NQ; ++q) {
                u[q] = V[j * NQ + q];
                s2  = fma2(u[q].x, x2[2 * q], s2);
                s2b = fma2(u[q].y, x2[2 * q + 1], s2b);
            }
            const float  c  = -(hsum(s2) + hsum(s2b)) * Vg[j];
            const pair_t c2 = pack(c, c);
#pragma unroll
            for (int q = q0; q < NQ; ++q) {
                x2[2 * q]     = fma2(c2, u[q].x, x2[2 * q]);
                x2[2 * q + 1] = fma2(c2, u[q].y, x2[2 * q + 1]);
            }
        }
    }

    // 3. R: row i across the lanes
    const Pow2 up(expo);
    if (live && l < n) {
        float* dst = p.r + (size_t)mat * p.rr * n;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            if (i < p.rr) {
                const float xi = (i & 1) ? hi_of(x2[i / 2]) : lo_of(x2[i / 2]);
                float v = (i < K && l >= i) ? up(xi) : 0.0f;
                if (bad) v = qnan();
                dst[i * n + l] = v;
            }
        }
    }
    if (p.qc == 0) return;

    // 4. Q's columns, backward: lane l holds column l of Q; the reflectors are read back from V
    pair_t q2[R / 2];
#pragma unroll
    for (int i = 0; i < R / 2; ++i) q2[i] = pack(2 * i == l ? 1.0f : 0.0f, 2 * i + 1 == l ? 1.0f : 0.0f);
#pragma unroll
    for (int j = kSteps - 1; j >= 0; --j) {
        if (j < K) {
            const int q0 = j / 4;
            ulonglong2 u[NQ];
            pair_t s2 = pack(0.0f, 0.0f), s2b = pack(0.0f, 0.0f);
#pragma unroll
            for (int q = q0; q < NQ; ++q) {
                u[q] = V[j * NQ + q];
                s2  = fma2(u[q].x, q2[2 * q], s2);
                s2b = fma2(u[q].y, q2[2 * q + 1], s2b);
            }
            const float  c  = -(hsum(s2) + hsum(s2b)) * Vg[j];
            const pair_t c2 = pack(c, c);
#pragma unroll
            for (int q = q0; q < NQ; ++q) {
                q2[2 * q]     = fma2(c2, u[q].x, q2[2 * q]);
                q2[2 * q + 1] = fma2(c2, u[q].y, q2[2 * q + 1]);
            }
        }
    }

    // 5. Q
    if (live && l < p.qc) {
        float* dst = p.q + (size_t)mat * m * p.qc;
#pragma unroll
        for (int i = 0; i < R / 2; ++i) {
            float a, b;
            unpack(q2[i], a, b);
            if (2 * i < m) dst[(2 * i) * p.qc + l] = bad ? qnan() : a;
            if (2 * i + 1 < m) dst[(2 * i + 1) * p.qc + l] = bad ? qnan() : b;
        }
    }
}

template <int R, int G>
void launch(cudaStream_t stream, const SmallParams& p) {
    constexpr int per_warp = 32 / G;
    constexpr int steps = R < G ? R : G;
    static const int warps_per_block = [] {
        const char* e = std::getenv("QR_SMALL_WARPS");
        const int w = e ? std::atoi(e) : 8;
        return w >= 1 && w <= 8 ? w : 8;
    }();
    const uint32_t per_block = per_warp * warps_per_block;
    const uint32_t blocks = (p.batch + per_block - 1) / per_block;
    const size_t smem = (size_t)per_block * (steps * R + steps + (4 - steps % 4) % 4) * sizeof(float);
    cuda_check(cudaFuncSetAttribute(qr_small_kernel<R, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024),
               "qr_small shared memory");
    qr_small_kernel<R, G><<<blocks, 32 * warps_per_block, smem, stream>>>(p);
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
