#pragma once
// The arithmetic of the small-matrix kernels, shared by the kernel that reads and
// writes global memory itself (qr_small.cu) and the one that streams matrices
// through shared memory with bulk asynchronous copies (qr_small_stream.cu): a
// matrix of at most 32 x 32 in the registers of G lanes, C columns a lane.
//
// Contract (the reference's register kernel, shaders/QR_Householder.metal:189-300):
// scan for the largest magnitude and for NaN/Inf, scale by a power of two into
// [0.5, 1), LAPACK's sgeqr2 with slarfg's signs, R multiplied back by the power of
// two, Q formed backward as sorg2r does. A matrix with a NaN or an Inf gives
// all-NaN Q and R.
//
// Mapping: lane l of a group of G holds columns l, l + G, ... (C of them, R rows
// each, two rows to a 64-bit register), so a reflector's dot products with the
// columns right of it are each lane's own FMAs with no reduction. What crosses
// lanes is the reflector: the owner of column j writes its tail to shared memory
// (16 bytes an instruction), every lane reads it back as broadcast 16-byte words,
// and it stays there for the Q pass. The arithmetic on rows is packed two to an
// instruction (fma.rn.f32x2, the Blackwell packed FP32 FMA). The reflector is
// kept unnormalised, H = I - g v v^T with v = (alpha - beta; tail).
#include "common.cuh"

#include <type_traits>

namespace mlb {
namespace small {

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

// floats of shared memory per matrix: the reflectors (`steps` vectors of R rows), -g of each, and
// padding to 4 floats more than a multiple of 32, so that the matrices of a warp sit 16 bytes apart
// in the banks and their broadcast loads do not collide
__host__ __device__ constexpr int slot_floats(int R, int steps) {
    int f = steps * R + steps;
    f += (4 - f % 4) % 4;
    f += (4 + 32 - f % 32) % 32;
    return f;
}
__host__ __device__ constexpr int steps_of(int R, int G, int C) { return R < G * C ? R : G * C; }

// f(integral_constant<int, 0>) ... f(integral_constant<int, N - 1>): a loop whose index is a constant
// in the body (for the steps, whose register indices must be)
template <int N, int I = 0, typename F>
__device__ __forceinline__ void static_for(F&& f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<N, I + 1>(f);
    }
}

// 1. The largest magnitude of the group's matrix (a NaN or an Inf anywhere makes it non-finite),
// and the matrix scaled into [0.5, 1). A non-finite matrix is computed on as it is (nothing
// traps); its outputs are made NaN by the scale of R and the start value of Q.
template <int R, int G, int C>
__device__ __forceinline__ void scan_scale(pair_t (&x2)[C][R / 2], bool& bad, int& expo) {
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
        for (int i = 0; i < R / 2; ++i) {
            float a, b;
            unpack(x2[c][i], a, b);
            amax = absmax3(a, b, amax);
        }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bad  = !(amax < __uint_as_float(0x7F800000u));
    expo = bad ? 0 : amax_exponent(amax);
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

// 2. Factor. Step j: the owner of column j (lane j % G, its column j / G) publishes the tail of
// that column (rows > j; zeros in the rows <= j of its first word), and every lane takes the
// tail's dot product with its own columns from j / G on (the earlier ones are finished in every
// lane). In the owner's lane that dot product is the tail's sum of squares, so the norm costs
// nothing extra: the owner forms the reflector from it, v1 and -g go round by shuffle, and every
// lane applies H = I - g v v^T to rows >= j of its columns. No lane is masked: in the owner's
// column the update leaves beta in row j (up to rounding), and the lanes left of the owner hold
// nothing live in rows >= j of that column (their R entries are above). The owner also leaves v1
// and -g in shared memory for the Q pass. `slot`: the matrix's slot_floats() floats; l: the lane
// within the group; K: the number of reflectors.
// (Measured alternative: every lane forming the reflector for itself from the broadcast column,
// which saves the shuffles and takes the square root off the critical path, costs a sum of
// squares per lane and step and is 10 % slower: the kernel is bound by throughput, not latency.)
template <int R, int G, int C>
__device__ __forceinline__ void factor(pair_t (&x2)[C][R / 2], float* slot, int l, int K) {
    constexpr int kSteps = steps_of(R, G, C);
    constexpr int NQ = R / 4;              // 16-byte words per column
    ulonglong2* V = reinterpret_cast<ulonglong2*>(slot);   // [kSteps][NQ] words
    float* Vg = slot + kSteps * R;
    // the owner of column jn writes its tail (rows > jn; zeros in the rows <= jn of the first word)
    auto publish = [&](auto jn_c) {
        constexpr int jn = decltype(jn_c)::value;
        constexpr int cn = jn / G, q0n = jn / 4, en = jn & 3;
        if (l == jn % G) {
#pragma unroll
            for (int q = q0n; q < NQ; ++q) {
                pair_t a = x2[cn][2 * q], b = x2[cn][2 * q + 1];
                if (q == q0n) {
                    if (en == 0) a = pack(0.0f, hi_of(a));
                    else if (en == 1) a = pack(0.0f, 0.0f);
                    else if (en == 2) { a = pack(0.0f, 0.0f); b = pack(0.0f, hi_of(b)); }
                    else { a = pack(0.0f, 0.0f); b = pack(0.0f, 0.0f); }
                }
                V[jn * NQ + q] = make_ulonglong2(a, b);
            }
        }
    };
    if (0 < K) publish(std::integral_constant<int, 0>{});
    __syncwarp();
    static_for<kSteps>([&](auto j_c) {
        constexpr int j = decltype(j_c)::value;
        if (j < K) {
            constexpr int cj = j / G;          // the owner's column among its lane's
            constexpr int q0 = j / 4;          // the word that holds row j
            constexpr int qt = (j + 1) / 4;    // first word that holds a row > j
            constexpr int e  = j & 3;
            const bool owner = l == j % G;
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
                slot[j * R + j] = v1;
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
            auto update = [&](int c) {
                const float  t  = fmaf(v1, xj[c], d[c]) * gneg;
                const pair_t t2 = pack(t, t);
                if (e < 2) x2[c][2 * q0] = fma2(t2, w0.x, x2[c][2 * q0]);
                x2[c][2 * q0 + 1] = fma2(t2, w0.y, x2[c][2 * q0 + 1]);
#pragma unroll
                for (int q = q0 + 1; q < NQ; ++q) {
                    x2[c][2 * q]     = fma2(t2, u[q].x, x2[c][2 * q]);
                    x2[c][2 * q + 1] = fma2(t2, u[q].y, x2[c][2 * q + 1]);
                }
            };
            // the next owner's column first, so that its tail is on its way to shared memory while
            // the other columns are updated
            constexpr int jn = j + 1, cn = jn < kSteps ? jn / G : C;
            if (cn < C) update(cn);
            if (jn < kSteps) {
                if (jn < K) publish(std::integral_constant<int, (jn < kSteps ? jn : 0)>{});
            }
#pragma unroll
            for (int c = cj; c < C; ++c)
                if (c != cn) update(c);
            __syncwarp();
        }
    });
    __syncwarp();      // the last v1 and -g are in shared memory before the Q pass reads them
}

// 3. R scaled back (by NaN for a matrix with a NaN or an Inf). The entries below the diagonal
// are not touched here: whoever stores R writes zeros (NaN for such a matrix) there.
template <int R, int G, int C>
__device__ __forceinline__ void scale_up(pair_t (&x2)[C][R / 2], int expo, bool bad) {
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
}

// 4. Q's columns, backward: lane l holds columns l + c G of Q; the reflectors are read back from
// the slot. Step j leaves the columns left of j untouched, so a lane's columns below j / G are
// skipped. A matrix with a NaN or an Inf starts from NaN instead of the identity. `between`
// is called once, half way (the streaming kernel starts its next load there).
template <int R, int G, int C, typename Between>
__device__ __forceinline__ void form_q(pair_t (&q2)[C][R / 2], const float* slot, int l, int K, bool bad,
                                       Between between) {
    constexpr int kSteps = steps_of(R, G, C);
    constexpr int NQ = R / 4;
    const ulonglong2* V = reinterpret_cast<const ulonglong2*>(slot);
    const float* Vg = slot + kSteps * R;
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
        if (j == kSteps / 2 - 1) between();
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
}

} // namespace small
} // namespace mlb
