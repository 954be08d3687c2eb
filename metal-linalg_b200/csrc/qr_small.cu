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

__device__ __forceinline__ pair_t add2(pair_t a, pair_t b) {
    pair_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ pair_t mul2(pair_t a, pair_t b) {
    pair_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// the sum of the four halves of two packed accumulators: one packed add, one scalar add
__device__ __forceinline__ float hsum2(pair_t a, pair_t b) { return hsum(add2(a, b)); }

// max(|a|, |b|, c), NaN if any of them is (the three-input form is one instruction)
__device__ __forceinline__ float absmax3(float a, float b, float c) {
    float d;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(fabsf(a)), "f"(fabsf(b)), "f"(c));
    return d;
}
__device__ __forceinline__ float max_nan(float a, float b) {
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

// The reflector of a column (alpha; tail) whose tail has sum of squares ss, unnormalised:
// H = I - g v v^T with v = (v1; tail), v1 = alpha - beta, beta = -sign(alpha) ||(alpha; tail)||
// (LAPACK's slarfg with v not divided by v1: the same reflector) and g = 2 / (v^T v), taken from
// v itself so that H is orthogonal to rounding whatever the last bit of beta. Returns -g.
// g = 0 (H = I, beta = alpha, v1 = 0) for a tail taken as zero.
__device__ __forceinline__ void fast_reflector(float alpha, float ss, float& v1, float& gneg) {
    const float n2 = fmaf(alpha, alpha, ss);
    float y, r;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(n2));
    const float nrm = n2 * y;      // to two ulps: H stays orthogonal to rounding (g is taken from v), R's
                                   // diagonal and the entries dropped below it are off by as much
    const bool  ok   = ss >= kTinySumsq;
    const float beta = ok ? -copysignf(nrm, alpha) : alpha;
    v1 = alpha - beta;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(fmaf(v1, v1, ss)));
    gneg = ok ? -2.0f * r : 0.0f;
}

// x * 2^e for every entry, exact wherever the result is representable: one multiplication by
// 2^e where that is a normal number, else two by 2^(e/2) and 2^(e - e/2) (|e| <= 160).
struct Scale2 {
    pair_t s1, s2;
    bool   two;
    __device__ __forceinline__ explicit Scale2(int e) {
        two = e < -126 || e > 127;
        const int e1 = two ? e / 2 : e;
        const float a = pow2f(e1), b = pow2f(e - e1);
        s1 = pack(a, a);
        s2 = pack(b, b);
    }
};

// floats of shared memory per matrix: the reflectors (kSteps vectors of R rows), -g of each, and
// padding to 4 floats more than a multiple of 32, so that the matrices of a warp sit 16 bytes apart
// in the banks and their broadcast loads do not collide
__host__ __device__ constexpr int slot_floats(int R, int steps) {
    int f = steps * R + steps;
    f += (4 - f % 4) % 4;
    f += (4 + 32 - f % 32) % 32;
    return f;
}

// Blocks of up to kMaxWarps warps; how many of them a multiprocessor is to hold, by the registers
// a lane needs for its R * C matrix entries.
constexpr int kMaxWarps = 8;
__host__ __device__ constexpr int min_blocks(int R, int C) { return R * C > 64 ? 1 : R * C > 32 ? 2 : 3; }

// R: rows held per lane (row capacity, a multiple of 4). G: lanes per matrix. C: columns per lane
// (column capacity G * C; lane l holds columns l, l + G, ...).
// Square: the matrix is exactly R x R with R = G * C (and Q, where asked for, R x R), so every bound
// is known when the kernel is compiled and no load, store or step is guarded.
template <int R, int G, int C, bool Square>
__global__ void __launch_bounds__(kMaxWarps * 32, min_blocks(R, C)) qr_small_kernel(const SmallParams p) {
    constexpr int kCols  = G * C;
    constexpr int kSteps = R < kCols ? R : kCols;
    constexpr int NQ = R / 4;              // 16-byte words per column
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
    ulonglong2* V = reinterpret_cast<ulonglong2*>(smem + (size_t)group * kSlot);   // [kSteps][NQ] words
    float* Vg = smem + (size_t)group * kSlot + kSteps * R;

    const float* src = p.a + (size_t)mat * m * n;

    // 1. load, scan, scale; rows 2p and 2p+1 of column l + c G packed in x2[c][p]. A NaN or an
    // Inf anywhere makes amax non-finite; such a matrix is computed on as it is (nothing traps)
    // and its outputs are made NaN by the scale of R and the start value of Q.
    pair_t x2[C][R / 2];
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int col = l + c * G;
#pragma unroll
        for (int i = 0; i < R / 2; ++i) {
            float a = 0.0f, b = 0.0f;
            if (2 * i < m && col < n) a = src[(2 * i) * n + col];
            if (2 * i + 1 < m && col < n) b = src[(2 * i + 1) * n + col];
            amax = absmax3(a, b, amax);
            x2[c][i] = pack(a, b);
        }
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const bool bad  = !(amax < __uint_as_float(0x7F800000u));
    const int  expo = bad ? 0 : amax_exponent(amax);
    {
        const Scale2 down(-expo);
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < R / 2; ++i) x2[c][i] = mul2(x2[c][i], down.s1);
        if (down.two) {
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < R / 2; ++i) x2[c][i] = mul2(x2[c][i], down.s2);
        }
    }

    // 2. factor. Step j: the owner of column j (lane j % G, its column j / G) publishes the tail
    // of that column (rows > j; zeros in the rows <= j of its first word), and every lane takes the
    // tail's dot product with its own columns from j / G on (the earlier ones are finished in every
    // lane). In the owner's lane that dot product is the tail's sum of squares, so the norm costs
    // nothing extra: the owner forms the reflector from it, v = (v1; tail) and -g go round by
    // shuffle, and every lane applies H = I - g v v^T to rows >= j of its columns. No lane is masked:
    // in the owner's column the update leaves beta in row j (up to rounding), and the lanes left of
    // the owner hold nothing live in rows >= j of that column (their R entries are above). The owner
    // also leaves v1 and -g in shared memory for the Q pass.
#pragma unroll
    for (int j = 0; j < kSteps; ++j) {
        if (j < K) {
            const int cj = j / G;          // the owner's column among its lane's
            const int q0 = j / 4;          // the word that holds row j
            const int qt = (j + 1) / 4;    // first word that holds a row > j
            const int e  = j & 3;
            const bool owner = l == j % G;
            if (owner) {
#pragma unroll
                for (int q = q0; q < NQ; ++q) {
                    pair_t a = x2[cj][2 * q], b = x2[cj][2 * q + 1];
                    if (q == q0) {         // zeros in rows <= j
                        if (e == 0) a = pack(0.0f, hi_of(a));
                        else if (e == 1) a = pack(0.0f, 0.0f);
                        else if (e == 2) { a = pack(0.0f, 0.0f); b = pack(0.0f, hi_of(b)); }
                        else { a = pack(0.0f, 0.0f); b = pack(0.0f, 0.0f); }
                    }
                    V[j * NQ + q] = make_ulonglong2(a, b);
                }
            }
            __syncwarp();
            ulonglong2 u[NQ];
#pragma unroll
            for (int q = qt; q < NQ; ++q) u[q] = V[j * NQ + q];
            float d[C], xj[C];
#pragma unroll
            for (int c = cj; c < C; ++c) {
                d[c] = 0.0f;
                if (qt < NQ) {
                    pair_t s2 = mul2(u[qt].x, x2[c][2 * qt]), s2b = mul2(u[qt].y, x2[c][2 * qt + 1]);
#pragma unroll
                    for (int q = qt + 1; q < NQ; ++q) {
                        s2  = fma2(u[q].x, x2[c][2 * q], s2);
                        s2b = fma2(u[q].y, x2[c][2 * q + 1], s2b);
                    }
                    d[c] = hsum2(s2, s2b);
                }
                xj[c] = (j & 1) ? hi_of(x2[c][j / 2]) : lo_of(x2[c][j / 2]);
            }
            float v1, gneg;
            fast_reflector(xj[cj], d[cj], v1, gneg);       // meaningful in the owner's lane
            v1   = __shfl_sync(0xffffffffu, v1, j % G, G);
            gneg = __shfl_sync(0xffffffffu, gneg, j % G, G);
            if (owner) {
                (smem + (size_t)group * kSlot)[j * R + j] = v1;
                Vg[j] = gneg;
            }
            // the reflector's first word with v1 in row j
            ulonglong2 w0;
            if (qt == q0) w0 = u[q0];
            else w0 = make_ulonglong2(pack(0.0f, 0.0f), pack(0.0f, 0.0f));
            if (e == 0) w0.x = pack(v1, hi_of(w0.x));
            else if (e == 1) w0.x = pack(0.0f, v1);
            else if (e == 2) w0.y = pack(v1, hi_of(w0.y));
            else w0.y = pack(0.0f, v1);
#pragma unroll
            for (int c = cj; c < C; ++c) {
                const float  t  = fmaf(v1, xj[c], d[c]) * gneg;
                const pair_t t2 = pack(t, t);
                if (e < 2) x2[c][2 * q0] = fma2(t2, w0.x, x2[c][2 * q0]);
                x2[c][2 * q0 + 1] = fma2(t2, w0.y, x2[c][2 * q0 + 1]);
#pragma unroll
                for (int q = q0 + 1; q < NQ; ++q) {
                    x2[c][2 * q]     = fma2(t2, u[q].x, x2[c][2 * q]);
                    x2[c][2 * q + 1] = fma2(t2, u[q].y, x2[c][2 * q + 1]);
                }
            }
        }
    }
    __syncwarp();      // the last v1 and -g are in shared memory before the Q pass reads them

    // 3. R: row i across the lanes, scaled back (by NaN for a matrix with a NaN or an Inf)
    {
        Scale2 up(expo);
        if (bad) up.s1 = pack(qnan(), qnan());
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < R / 2; ++i) x2[c][i] = mul2(x2[c][i], up.s1);
        if (up.two) {
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < R / 2; ++i) x2[c][i] = mul2(x2[c][i], up.s2);
        }
        const float zero = bad ? qnan() : 0.0f;
        float* dst = p.r + (size_t)mat * rr * n;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int col = l + c * G;
            if (live && col < n) {
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const float v = (i & 1) ? hi_of(x2[c][i / 2]) : lo_of(x2[c][i / 2]);
                    if (i < rr) dst[i * n + col] = (i < K && col >= i) ? v : zero;
                }
            }
        }
    }
    if (qc == 0) return;

    // 4. Q's columns, backward: lane l holds columns l + c G of Q; the reflectors are read back
    // from V. Step j leaves the columns left of j untouched, so a lane's columns below j / G are
    // skipped. A matrix with a NaN or an Inf starts from NaN instead of the identity.
    pair_t q2[C][R / 2];
    {
        const float one = bad ? qnan() : 1.0f, zero = bad ? qnan() : 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int i = 0; i < R / 2; ++i)
                q2[c][i] = pack(2 * i == l + c * G ? one : zero, 2 * i + 1 == l + c * G ? one : zero);
    }
#pragma unroll
    for (int j = kSteps - 1; j >= 0; --j) {
        if (j < K) {
            const int cj = j / G;
            const int q0 = j / 4;
            ulonglong2 u[NQ];
#pragma unroll
            for (int q = q0; q < NQ; ++q) u[q] = V[j * NQ + q];
            const float gneg = Vg[j];
#pragma unroll
            for (int c = cj; c < C; ++c) {
                pair_t s2 = mul2(u[q0].x, q2[c][2 * q0]), s2b = mul2(u[q0].y, q2[c][2 * q0 + 1]);
#pragma unroll
                for (int q = q0 + 1; q < NQ; ++q) {
                    s2  = fma2(u[q].x, q2[c][2 * q], s2);
                    s2b = fma2(u[q].y, q2[c][2 * q + 1], s2b);
                }
                const float  t  = hsum2(s2, s2b) * gneg;
                const pair_t t2 = pack(t, t);
#pragma unroll
                for (int q = q0; q < NQ; ++q) {
                    q2[c][2 * q]     = fma2(t2, u[q].x, q2[c][2 * q]);
                    q2[c][2 * q + 1] = fma2(t2, u[q].y, q2[c][2 * q + 1]);
                }
            }
        }
    }

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
                    if (2 * i < m) dst[(2 * i) * qc + col] = a;
                    if (2 * i + 1 < m) dst[(2 * i + 1) * qc + col] = b;
                }
            }
        }
    }
}

template <int R, int G, int C, bool Square>
void launch(cudaStream_t stream, const SmallParams& p) {
    constexpr int per_warp = 32 / G;
    constexpr int steps = R < G * C ? R : G * C;
    static const int warps_per_block = [] {
        const char* e = std::getenv("QR_SMALL_WARPS");
        const int w = e ? std::atoi(e) : kMaxWarps;
        return w >= 1 && w <= kMaxWarps ? w : kMaxWarps;
    }();
    const uint32_t per_block = per_warp * warps_per_block;
    const uint32_t blocks = (p.batch + per_block - 1) / per_block;
    const size_t smem = (size_t)per_block * slot_floats(R, steps) * sizeof(float);
    static const bool configured = [] {
        cuda_check(cudaFuncSetAttribute(qr_small_kernel<R, G, C, Square>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (32 / G) * kMaxWarps * slot_floats(R, steps) * (int)sizeof(float)),
                   "qr_small shared memory");
        cuda_check(cudaFuncSetAttribute(qr_small_kernel<R, G, C, Square>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared),
                   "qr_small shared memory carveout");
        return true;
    }();
    (void)configured;
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

void launch_qr_small(DeviceContext&, cudaStream_t stream, const QrProblem& pr) {
    if (pr.batch == 0) return;
    SmallParams p{pr.a, pr.q, pr.r, pr.batch, (int)pr.m, (int)pr.n, (int)qr_k(pr), (int)pr.qc, (int)pr.rr};
    const int R   = pow2_at_least(pr.m, 8);
    const int cap = pow2_at_least(pr.n > pr.qc ? pr.n : pr.qc, 8);      // column capacity
    int C = forced_columns_a_lane() ? forced_columns_a_lane() : 2;
    while (C > 1 && cap / C < 4) C /= 2;
    if (cap == 8 && !forced_columns_a_lane()) C = 1;
    const int G = cap / C;
    const bool square = pr.m == pr.n && (int)pr.m == R && cap == R && pr.rr == pr.m && (pr.qc == 0 || pr.qc == pr.m);
#define MLB_SMALL(RR, GG, CC)                                                    \
    if (R == RR && G == GG && C == CC) {                                         \
        if constexpr (RR == GG * CC) {                                           \
            if (square) launch<RR, GG, CC, true>(stream, p);                     \
            else launch<RR, GG, CC, false>(stream, p);                           \
        } else launch<RR, GG, CC, false>(stream, p);                             \
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
