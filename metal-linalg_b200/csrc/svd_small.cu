// The small SVD on the far side of the QR: Hestenes' one-sided Jacobi on the K x K triangular factor
// of a QR-preconditioned SVD (reference: svd_qr_jacobi, src/svd.mm:614-661, whose inner kernel is
// shaders/Svd_Jacobi.metal), K <= 128, and the product U = Q U_R that follows it.
//
// Layout for K <= 32 (for 32 < K <= 128 see svd_block_kernel): a matrix belongs to a group of R lanes (R = 4, 8, 16 or 32 >= K; 32 / R matrices a warp),
// lane c holding column c of G (= the factor R, scaled by a power of two so that its largest entry
// lies in [0.5, 1)) and column c of V in registers. A round pairs every column with one partner
// (the circle method: R - 1 rounds visit every pair once); the partner's column comes by R
// shuffles, both lanes of a pair form the same three inner products in the same order (rows packed two
// to a 64-bit register: fma.rn.f32x2), hence the same rotation, and each applies its own half. No
// shared memory, no barrier.
//
// The rules of the reference's kernel are kept: a pair is rotated iff |gamma| > tol sqrt(alpha beta)
// with tol = sqrt(max(rows, 64)) eps; two numerically null columns (below 32 eps of the largest
// column) are never rotated against each other, and a null column against another keeps the sweeps
// going only while the angle is gross and the column not negligible; a sweep that rotates nothing
// ends the solve; singular values descending (ties by column index); left vectors of null columns
// are replaced by an orthonormal completion; a matrix with a NaN or an infinity gives NaN outputs;
// info = sweeps | converged << 16 | non-finite << 17 | rank-deficient << 18.
#include "common.cuh"
#include "kernels.h"
#include "qr_small_steps.cuh"
#include "runtime.h"

#include <cfloat>

namespace mlb {
namespace {

constexpr float kNullTol        = 32.0f * FLT_EPSILON;   // src/svd.mm:65
constexpr float kNegligible     = 1.2e-7f;               // shaders/Svd_Jacobi.metal:82
constexpr float kCleanCos       = 0.05f;                 // shaders/Svd_Jacobi.metal:78
constexpr float kZetaAsymptotic = 1e15f;                 // shaders/Svd_Jacobi.metal:75

struct SvdSmallParams {
    const float* r;        // [batch, k, k] row-major
    float*       s;        // [batch, k]
    float*       ur;       // [batch, k, k] left vectors of the factor as columns, or null
    float*       v;        // [batch, k, k]: V^T (row t = right vector t), or V itself when v_as_columns
    uint32_t*    info;     // [batch] or null
    uint32_t     batch, k;
    uint32_t     max_sweeps;
    float        tol;
    int          v_as_columns;
};

template <int R>
__device__ __forceinline__ float group_max(float v, unsigned mask) {
#pragma unroll
    for (int o = R / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(mask, v, o, R));
    return v;
}
template <int R>
__device__ __forceinline__ float group_sum(float v, unsigned mask) {
#pragma unroll
    for (int o = R / 2; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o, R);
    return v;
}

__device__ __forceinline__ small::pair_t shuffle_pair(unsigned mask, small::pair_t v, int src, int width) {
    float lo, hi;
    small::unpack(v, lo, hi);
    return small::pack(__shfl_sync(mask, lo, src, width), __shfl_sync(mask, hi, src, width));
}

// A fixed pseudo-random number in [-0.5, 0.5) for entry i of candidate `seed`.
__device__ __forceinline__ float candidate_entry(uint32_t seed, uint32_t i) {
    uint32_t x = seed * 0x9E3779B9u + i * 0x85EBCA6Bu + 0x27D4EB2Fu;
    x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
    return (float)(x >> 8) * (1.0f / 16777216.0f) - 0.5f;
}

template <int R, bool Vectors>
__global__ void __launch_bounds__(128) svd_small_kernel(const SvdSmallParams p) {
    dependency_wait_only();
    const int lane = threadIdx.x & 31, col = lane & (R - 1);
    constexpr int kPerWarp = 32 / R;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t mat = warp * kPerWarp + (lane / R);
    if (mat >= p.batch) return;      // a whole group leaves together
    const unsigned mask = R == 32 ? 0xffffffffu : (((1u << (R & 31)) - 1u) << (lane & ~(R - 1)));
    const uint32_t k = p.k;

    float g[R], v[Vectors ? R : 1];
    const float* src = p.r + (size_t)mat * k * k;
    float amax = 0.0f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        g[i] = ((uint32_t)i < k && (uint32_t)col < k) ? src[i * k + col] : 0.0f;
        bad |= nonfinite(g[i]);
        amax = fmaxf(amax, fabsf(g[i]));
    }
    const bool nonfin = __ballot_sync(mask, bad) != 0;
    amax = group_max<R>(amax, mask);
    const int expo = nonfin ? 0 : amax_exponent(amax);
    {
        const Pow2 down(-expo);
#pragma unroll
        for (int i = 0; i < R; ++i) g[i] = down(g[i]);
    }
    if (Vectors) {
#pragma unroll
        for (int i = 0; i < R; ++i) v[i] = i == col ? 1.0f : 0.0f;
    }

    // The sweeps work on rows packed two to a 64-bit register (fma.rn.f32x2: half the arithmetic
    // instructions); the partner's column comes by shuffles. (The same exchange through shared memory as
    // 16-byte words takes a quarter of the instructions but measured slower with vectors, 45 against 36 ms
    // for 262 144 matrices of 32 x 32: the round is a latency chain, and the registers it costs leave three
    // warps a scheduler.)
    using small::pair_t;
    constexpr int H = R / 2;
    pair_t gp[H], vp[Vectors ? H : 1];
#pragma unroll
    for (int i = 0; i < H; ++i) gp[i] = small::pack(g[2 * i], g[2 * i + 1]);
    if (Vectors) {
#pragma unroll
        for (int i = 0; i < H; ++i) vp[i] = small::pack(v[2 * i], v[2 * i + 1]);
    }

    uint32_t sweeps = 0;
    bool converged = false;
    while (!nonfin && sweeps < p.max_sweeps) {
        float own;
        {
            pair_t acc = small::mul2(gp[0], gp[0]);
#pragma unroll
            for (int i = 1; i < H; ++i) acc = small::fma2(gp[i], gp[i], acc);
            own = small::hsum(acc);
        }
        const float cmax2 = group_max<R>(own, mask);
        const float null2 = kNullTol * kNullTol * cmax2, negl2 = kNegligible * kNegligible * cmax2;
        bool rotated = false;
#pragma unroll 1
        for (int round = 0; round < R - 1; ++round) {
            // the circle method: columns i, j < R - 1 meet when i + j = round (mod R - 1); the one
            // that would meet itself meets column R - 1
            int partner;
            if (col == R - 1) {
                partner = (round * (R / 2)) % (R - 1);
            } else {
                partner = (round + (R - 1) - col) % (R - 1);
                if (partner == col) partner = R - 1;
            }
            const bool lower = col < partner;
            pair_t pg[H];
#pragma unroll
            for (int i = 0; i < H; ++i) pg[i] = shuffle_pair(mask, gp[i], partner, R);
            pair_t am = small::mul2(gp[0], gp[0]), at = small::mul2(pg[0], pg[0]), ag = small::mul2(gp[0], pg[0]);
#pragma unroll
            for (int i = 1; i < H; ++i) {
                am = small::fma2(gp[i], gp[i], am);
                at = small::fma2(pg[i], pg[i], at);
                ag = small::fma2(gp[i], pg[i], ag);
            }
            const float mine = small::hsum(am), theirs = small::hsum(at), gamma = small::hsum(ag);
            const float alpha = lower ? mine : theirs, beta = lower ? theirs : mine;   // of columns p < q
            const float ab = alpha * beta;
            // both lanes of a pair decide alike: they saw the same numbers, summed in the same order. The
            // updates below run for every pair, with the identity where nothing is rotated.
            const bool rotate = !(alpha <= null2 && beta <= null2) && fabsf(gamma) > p.tol * sqrtf(ab);
            float c = 1.0f, cs = 0.0f;
            if (rotate) {
                const float zeta = (beta - alpha) / (2.0f * gamma);
                float t;
                if (fabsf(zeta) > kZetaAsymptotic) {
                    t = 0.5f / zeta;
                } else {
                    t = 1.0f / (fabsf(zeta) + sqrtf(fmaf(zeta, zeta, 1.0f)));
                    if (zeta < 0.0f) t = -t;
                }
                c = 1.0f / sqrtf(fmaf(t, t, 1.0f));
                const float sn = c * t;
                cs = lower ? -sn : sn;       // p: x' = c x - s y;   q: y' = s x + c y
                const bool one_null = alpha <= null2 || beta <= null2;
                if (!one_null) rotated = true;
                else if (fminf(alpha, beta) > negl2 && gamma * gamma > kCleanCos * kCleanCos * ab) rotated = true;
            }
            const pair_t c2 = small::pack(c, c), cs2 = small::pack(cs, cs);
#pragma unroll
            for (int i = 0; i < H; ++i) gp[i] = small::fma2(cs2, pg[i], small::mul2(c2, gp[i]));
            if (Vectors) {
#pragma unroll
                for (int i = 0; i < H; ++i)
                    vp[i] = small::fma2(cs2, shuffle_pair(mask, vp[i], partner, R), small::mul2(c2, vp[i]));
            }
        }
        ++sweeps;
        if (__ballot_sync(mask, rotated) == 0) { converged = true; break; }
    }
#pragma unroll
    for (int i = 0; i < H; ++i) small::unpack(gp[i], g[2 * i], g[2 * i + 1]);
    if (Vectors) {
#pragma unroll
        for (int i = 0; i < H; ++i) small::unpack(vp[i], v[2 * i], v[2 * i + 1]);
    }

    // singular values, their order, the null threshold
    float sig = 0.0f;
#pragma unroll
    for (int i = 0; i < R; ++i) sig = fmaf(g[i], g[i], sig);
    sig = sqrtf(sig);
    uint32_t rank = 0;
#pragma unroll
    for (int c = 0; c < R; ++c) {
        const float sc = __shfl_sync(mask, sig, c, R);
        rank += (sc > sig || (sc == sig && c < col)) ? 1u : 0u;
    }
    if (nonfin) rank = col;      // NaN compares false with everything
    const float smax = group_max<R>(sig, mask);
    const float thr = kNullTol * smax;
    const bool real = (uint32_t)col < k;
    const bool deficient = (__ballot_sync(mask, real && !(sig > thr)) != 0) && !nonfin;

    const size_t kk = (size_t)k * k;
    if (real) p.s[(size_t)mat * k + rank] = nonfin ? qnan() : Pow2(expo)(sig);
    if (col == 0 && p.info)
        p.info[mat] = sweeps | (converged ? 1u << 16 : 0u) | (nonfin ? 1u << 17 : 0u) | (deficient ? 1u << 18 : 0u);
    if (!Vectors) return;

    float* out_v = p.v + (size_t)mat * kk;
    float* out_u = p.ur + (size_t)mat * kk;
    if (nonfin) {
        if (real)
            for (uint32_t i = 0; i < k; ++i) { out_v[i * k + col] = qnan(); out_u[i * k + col] = qnan(); }
        return;
    }
    if (real) {
#pragma unroll
        for (int i = 0; i < R; ++i)
            if ((uint32_t)i < k) out_v[p.v_as_columns ? (size_t)i * k + rank : (size_t)rank * k + i] = v[i];
    }
    // left vectors: the normalised columns; a null column is completed below
    bool valid = real && sig > thr;
    {
        const float inv = valid ? 1.0f / sig : 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) g[i] *= inv;
    }
    if (deficient) {
        // Every null column in turn takes a fixed pseudo-random vector made orthogonal (three
        // passes) to the columns in place: any unit vector orthogonal to the others is a valid
        // left vector there (reference: complete_columns_impl, src/svd.mm:148-186).
        uint32_t seed = 1;
        for (uint32_t c = 0; c < k; ++c) {
            const bool needs = __shfl_sync(mask, valid ? 0 : 1, c, R) != 0;
            if (!needs) continue;
            for (int attempt = 0; attempt < 8; ++attempt, ++seed) {
                float w[R];
                float start = 0.0f;
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    w[i] = (uint32_t)i < k ? candidate_entry(seed, i) : 0.0f;
                    start = fmaf(w[i], w[i], start);
                }
                for (int pass = 0; pass < 3; ++pass) {
                    float dot = 0.0f;
#pragma unroll
                    for (int i = 0; i < R; ++i) dot = fmaf(g[i], w[i], dot);
                    if (!valid) dot = 0.0f;
#pragma unroll
                    for (int i = 0; i < R; ++i) w[i] -= group_sum<R>(dot * g[i], mask);
                }
                float nrm = 0.0f;
#pragma unroll
                for (int i = 0; i < R; ++i) nrm = fmaf(w[i], w[i], nrm);
                if (nrm > 1e-6f * start) {        // squares: a residual above 1e-3 of the start
                    if (col == c) {
                        const float inv = rsqrtf(nrm);
#pragma unroll
                        for (int i = 0; i < R; ++i) g[i] = w[i] * inv;
                        valid = true;
                    }
                    break;
                }
            }
        }
    }
    if (real) {
#pragma unroll
        for (int i = 0; i < R; ++i)
            if ((uint32_t)i < k) out_u[(size_t)i * k + rank] = g[i];
    }
}

// out = Q U_R for every matrix: Q [batch, l, k] row-major, U_R [batch, k, k]; a thread a row of Q.
// `transposed`: out is [batch, k, l] (the right vectors of a wide matrix), else [batch, l, k].
template <int KP>
__global__ void __launch_bounds__(256) svd_left_vectors_kernel(const float* __restrict__ q, const float* __restrict__ ur,
                                                               float* __restrict__ out, uint32_t batch, uint32_t l, uint32_t k,
                                                               int transposed) {
    dependency_wait_only();
    const size_t row = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= (size_t)batch * l) return;
    const uint32_t b = (uint32_t)(row / l), i = (uint32_t)(row % l);
    const float* qr = q + row * k;
    const float* u = ur + (size_t)b * k * k;
    float acc[KP];
#pragma unroll
    for (int j = 0; j < KP; ++j) acc[j] = 0.0f;
    for (uint32_t t = 0; t < k; ++t) {
        const float x = qr[t];
#pragma unroll
        for (int j = 0; j < KP; ++j)
            if ((uint32_t)j < k) acc[j] = fmaf(x, u[t * k + j], acc[j]);
    }
    if (transposed) {
        float* o = out + (size_t)b * k * l + i;
#pragma unroll
        for (int j = 0; j < KP; ++j)
            if ((uint32_t)j < k) o[(size_t)j * l] = acc[j];
    } else {
        float* o = out + row * k;
#pragma unroll
        for (int j = 0; j < KP; ++j)
            if ((uint32_t)j < k) o[j] = acc[j];
    }
}

// out[b][j][i] = in[b][i][j]: in [batch, rows, cols].
__global__ void __launch_bounds__(256) transpose_batched_kernel(const float* __restrict__ in, float* __restrict__ out,
                                                                uint32_t rows, uint32_t cols) {
    dependency_wait_only();
    __shared__ float tile[32][33];
    const size_t base = (size_t)blockIdx.z * rows * cols;
    const uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (uint32_t r = ty; r < 32; r += 8)
        if (r0 + r < rows && c0 + tx < cols) tile[r][tx] = in[base + (size_t)(r0 + r) * cols + c0 + tx];
    __syncthreads();
    for (uint32_t c = ty; c < 32; c += 8)
        if (c0 + c < cols && r0 + tx < rows) out[base + (size_t)(c0 + c) * rows + r0 + tx] = tile[tx][c];
}

// ---------------------------------------------------------------------------
// 32 < k <= 128: a matrix to a thread block, G and V by column in shared memory, a warp to a pair
// (lanes along the rows; the three inner products by a warp sum), one barrier a round -- the
// arrangement of the reference's kernel (shaders/Svd_Jacobi.metal:20-33) -- with the same rules.
// ---------------------------------------------------------------------------
constexpr int kBlockWarps = 32;

struct BlockShared {
    float red[kBlockWarps];
    float sig[128];
    uint32_t rank[128];
    unsigned char valid[128];
    float w[128];
    int flag;
};

__device__ __forceinline__ float block_max(float v, float* red, int warp, int lane, int nw) {
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < nw; ++i) r = fmaxf(r, red[i]);
    return r;
}

template <bool Vectors>
__global__ void __launch_bounds__(32 * kBlockWarps) svd_block_kernel(const SvdSmallParams p) {
    dependency_wait_only();
    extern __shared__ __align__(16) float dyn[];
    __shared__ BlockShared sh;
    const uint32_t k = p.k, ld = k | 1u;          // odd: the transposing load and the stores by row spread over the banks
    float* G = dyn;
    float* V = dyn + (size_t)k * ld;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nt = blockDim.x, nw = nt >> 5;
    const uint32_t mat = blockIdx.x;
    const size_t kk = (size_t)k * k;
    const float* src = p.r + mat * kk;

    float amax = 0.0f;
    int bad = 0;
    for (uint32_t idx = tid; idx < kk; idx += nt) {
        const uint32_t i = idx / k, c = idx - i * k;
        const float x = src[idx];
        bad |= nonfinite(x) ? 1 : 0;
        amax = fmaxf(amax, fabsf(x));
        G[c * ld + i] = x;
        if (Vectors) V[c * ld + i] = i == c ? 1.0f : 0.0f;
    }
    const bool nonfin = __syncthreads_or(bad) != 0;
    amax = block_max(amax, sh.red, warp, lane, nw);
    const int expo = nonfin ? 0 : amax_exponent(amax);
    {
        const Pow2 down(-expo);
        for (uint32_t idx = tid; idx < kk; idx += nt) {
            const uint32_t c = idx / k, i = idx - c * k;
            G[c * ld + i] = down(G[c * ld + i]);
        }
    }
    __syncthreads();

    const uint32_t n_even = (k + 1) & ~1u, np = n_even / 2, m1 = n_even - 1;
    uint32_t sweeps = 0;
    bool converged = false;
    while (!nonfin && sweeps < p.max_sweeps) {
        float cmax2 = 0.0f;
        for (uint32_t c = warp; c < k; c += nw) {
            float acc = 0.0f;
            for (uint32_t i = lane; i < k; i += 32) acc = fmaf(G[c * ld + i], G[c * ld + i], acc);
            cmax2 = fmaxf(cmax2, warp_sum(acc));
        }
        cmax2 = block_max(cmax2, sh.red, warp, lane, nw);
        const float null2 = kNullTol * kNullTol * cmax2, negl2 = kNegligible * kNegligible * cmax2;
        int rotated = 0;
        for (uint32_t round = 0; round < m1; ++round) {
            // the circle method: x0 with 2 x0 = round (mod n_even - 1) meets the last column, and
            // x0 + j meets x0 - j
            const uint32_t x0 = (round * np) % m1;
            for (uint32_t j = warp; j < np; j += nw) {
                const uint32_t a = j == 0 ? x0 : (x0 + j) % m1, b = j == 0 ? m1 : (x0 + m1 - j) % m1;
                const uint32_t cp = min(a, b), cq = max(a, b);
                if (cq >= k) continue;          // the dummy column of an odd k
                float* gp = G + cp * ld;
                float* gq = G + cq * ld;
                float alpha = 0.0f, beta = 0.0f, gamma = 0.0f;
                for (uint32_t i = lane; i < k; i += 32) {
                    const float x = gp[i], y = gq[i];
                    alpha = fmaf(x, x, alpha);
                    beta = fmaf(y, y, beta);
                    gamma = fmaf(x, y, gamma);
                }
                alpha = warp_sum(alpha);
                beta = warp_sum(beta);
                gamma = warp_sum(gamma);
                if (alpha <= null2 && beta <= null2) continue;
                const float ab = alpha * beta;
                if (!(fabsf(gamma) > p.tol * sqrtf(ab))) continue;
                const float zeta = (beta - alpha) / (2.0f * gamma);
                float t;
                if (fabsf(zeta) > kZetaAsymptotic) {
                    t = 0.5f / zeta;
                } else {
                    t = 1.0f / (fabsf(zeta) + sqrtf(fmaf(zeta, zeta, 1.0f)));
                    if (zeta < 0.0f) t = -t;
                }
                const float c = 1.0f / sqrtf(fmaf(t, t, 1.0f)), sn = c * t;
                for (uint32_t i = lane; i < k; i += 32) {
                    const float x = gp[i], y = gq[i];
                    gp[i] = fmaf(-sn, y, c * x);
                    gq[i] = fmaf(sn, x, c * y);
                }
                if (Vectors) {
                    float* vp = V + cp * ld;
                    float* vq = V + cq * ld;
                    for (uint32_t i = lane; i < k; i += 32) {
                        const float x = vp[i], y = vq[i];
                        vp[i] = fmaf(-sn, y, c * x);
                        vq[i] = fmaf(sn, x, c * y);
                    }
                }
                const bool one_null = alpha <= null2 || beta <= null2;
                if (!one_null) rotated = 1;
                else if (fminf(alpha, beta) > negl2 && gamma * gamma > kCleanCos * kCleanCos * ab) rotated = 1;
            }
            __syncthreads();      // the next round pairs columns other warps have just written
        }
        ++sweeps;
        if (__syncthreads_or(rotated) == 0) { converged = true; break; }
    }

    // singular values, their order, the null threshold
    for (uint32_t c = warp; c < k; c += nw) {
        float acc = 0.0f;
        for (uint32_t i = lane; i < k; i += 32) acc = fmaf(G[c * ld + i], G[c * ld + i], acc);
        acc = warp_sum(acc);
        if (lane == 0) sh.sig[c] = sqrtf(acc);
    }
    __syncthreads();
    float smax = 0.0f;
    for (uint32_t c = tid; c < k; c += nt) smax = fmaxf(smax, sh.sig[c]);
    smax = block_max(smax, sh.red, warp, lane, nw);
    const float thr = kNullTol * smax;
    int low = 0;
    for (uint32_t c = tid; c < k; c += nt) {
        const float sc = sh.sig[c];
        uint32_t before = 0;
        for (uint32_t d = 0; d < k; ++d) {
            const float sd = sh.sig[d];
            before += (sd > sc || (sd == sc && d < c)) ? 1u : 0u;
        }
        sh.rank[c] = nonfin ? c : before;
        sh.valid[c] = sc > thr ? 1 : 0;
        low |= sc > thr ? 0 : 1;
        p.s[(size_t)mat * k + sh.rank[c]] = nonfin ? qnan() : Pow2(expo)(sc);
    }
    const bool deficient = (__syncthreads_or(low) != 0) && !nonfin;      // also orders rank and valid before their readers
    if (tid == 0 && p.info)
        p.info[mat] = sweeps | (converged ? 1u << 16 : 0u) | (nonfin ? 1u << 17 : 0u) | (deficient ? 1u << 18 : 0u);
    if (!Vectors) return;

    float* out_v = p.v + mat * kk;
    float* out_u = p.ur + mat * kk;
    if (nonfin) {
        for (uint32_t idx = tid; idx < kk; idx += nt) { out_v[idx] = qnan(); out_u[idx] = qnan(); }
        return;
    }
    // left vectors: the normalised columns, zero for a null one
    for (uint32_t c = warp; c < k; c += nw) {
        const float inv = sh.valid[c] ? 1.0f / sh.sig[c] : 0.0f;
        for (uint32_t i = lane; i < k; i += 32) G[c * ld + i] *= inv;
    }
    __syncthreads();
    if (deficient && warp == 0) {
        // Every null column in turn takes a fixed pseudo-random vector made orthogonal (three passes) to the
        // columns in place (reference: complete_columns_impl, src/svd.mm:148-186); one warp does it.
        uint32_t seed = 1;
        for (uint32_t c = 0; c < k; ++c) {
            if (sh.valid[c]) continue;
            for (int attempt = 0; attempt < 8; ++attempt, ++seed) {
                float start = 0.0f;
                for (uint32_t i = lane; i < k; i += 32) {
                    const float x = candidate_entry(seed, i);
                    sh.w[i] = x;
                    start = fmaf(x, x, start);
                }
                start = warp_sum(start);
                __syncwarp();
                for (int pass = 0; pass < 3; ++pass)
                    for (uint32_t d = 0; d < k; ++d) {
                        if (!sh.valid[d]) continue;
                        float dot = 0.0f;
                        for (uint32_t i = lane; i < k; i += 32) dot = fmaf(G[d * ld + i], sh.w[i], dot);
                        dot = warp_sum(dot);
                        for (uint32_t i = lane; i < k; i += 32) sh.w[i] = fmaf(-dot, G[d * ld + i], sh.w[i]);
                        __syncwarp();
                    }
                float nrm = 0.0f;
                for (uint32_t i = lane; i < k; i += 32) nrm = fmaf(sh.w[i], sh.w[i], nrm);
                nrm = warp_sum(nrm);
                if (nrm > 1e-6f * start) {
                    const float inv = rsqrtf(nrm);
                    for (uint32_t i = lane; i < k; i += 32) G[c * ld + i] = sh.w[i] * inv;
                    if (lane == 0) sh.valid[c] = 1;
                    __syncwarp();
                    break;
                }
            }
        }
    }
    __syncthreads();
    for (uint32_t idx = tid; idx < kk; idx += nt) {
        const uint32_t i = idx / k, c = idx - i * k;
        const uint32_t rk = sh.rank[c];
        out_u[(size_t)i * k + rk] = G[c * ld + i];
        out_v[p.v_as_columns ? (size_t)i * k + rk : (size_t)rk * k + i] = V[c * ld + i];
    }
}

size_t block_smem(uint32_t k, bool vectors) { return (size_t)k * (k | 1u) * sizeof(float) * (vectors ? 2 : 1); }

void launch_block_jacobi(cudaStream_t stream, const SvdSmallParams& p, bool vectors) {
    static PerDeviceOnce once;      // the opt-in is recorded per GPU
    if (const int device = current_device(); once.first(device)) {
        cuda_check(cudaFuncSetAttribute(svd_block_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)block_smem(128, true)), "svd_block shared memory");
        cuda_check(cudaFuncSetAttribute(svd_block_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)block_smem(128, false)), "svd_block shared memory");
        once.mark(device);
    }
    const uint32_t pairs = (p.k + 1) / 2;
    // with vectors a block fills a multiprocessor's shared memory and takes every warp it may have; the values
    // alone leave room for three blocks, which 16 warps each use better (1024 x 128 x 128: 22 against 25 ms)
    const uint32_t cap = vectors ? (uint32_t)kBlockWarps : 16u;
    const uint32_t warps = pairs < cap ? pairs : cap;
    if (vectors) launch_dependent(svd_block_kernel<true>, p.batch, 32 * warps, block_smem(p.k, true), stream, p);
    else launch_dependent(svd_block_kernel<false>, p.batch, 32 * warps, block_smem(p.k, false), stream, p);
}

// out = Q U_R for k > 32: a block takes 64 rows of Q, U_R in shared memory, a thread 1 row x k / 4 columns.
__global__ void __launch_bounds__(256) svd_left_vectors_wide_kernel(const float* __restrict__ q, const float* __restrict__ ur,
                                                                    float* __restrict__ out, uint32_t l, uint32_t k, int transposed) {
    dependency_wait_only();
    extern __shared__ __align__(16) float dyn[];
    float* U = dyn;                        // [k][k]
    float* Qs = dyn + (size_t)k * k;       // [64][k + 1]
    const uint32_t b = blockIdx.y, r0 = blockIdx.x * 64, tid = threadIdx.x;
    const float* ub = ur + (size_t)b * k * k;
    const float* qb = q + ((size_t)b * l + r0) * k;
    const uint32_t rows = min(64u, l - r0);
    for (uint32_t idx = tid; idx < k * k; idx += 256) U[idx] = ub[idx];
    for (uint32_t idx = tid; idx < rows * k; idx += 256) Qs[(idx / k) * (k + 1) + idx % k] = qb[idx];
    __syncthreads();
    const uint32_t row = tid >> 2, quarter = tid & 3;
    if (row >= rows) return;
    float acc[32];
#pragma unroll
    for (int jj = 0; jj < 32; ++jj) acc[jj] = 0.0f;
    for (uint32_t t = 0; t < k; ++t) {
        const float x = Qs[row * (k + 1) + t];
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
            const uint32_t j = quarter + 4 * jj;
            if (j < k) acc[jj] = fmaf(x, U[t * k + j], acc[jj]);
        }
    }
#pragma unroll
    for (int jj = 0; jj < 32; ++jj) {
        const uint32_t j = quarter + 4 * jj;
        if (j >= k) continue;
        if (transposed) out[((size_t)b * k + j) * l + r0 + row] = acc[jj];
        else out[((size_t)b * l + r0 + row) * k + j] = acc[jj];
    }
}

template <int R>
void launch_jacobi(cudaStream_t stream, const SvdSmallParams& p, bool vectors) {
    const uint32_t per_block = 4 * (32 / R);
    const uint32_t blocks = (p.batch + per_block - 1) / per_block;
    if (vectors) launch_dependent(svd_small_kernel<R, true>, blocks, 128, 0, stream, p);
    else launch_dependent(svd_small_kernel<R, false>, blocks, 128, 0, stream, p);
}

} // namespace

bool svd_small_fits(uint32_t k) { return k >= 1 && k <= 128; }

void launch_svd_small(cudaStream_t stream, const float* r, uint32_t batch, uint32_t k, uint32_t effective_rows,
                      float* s, float* ur, float* v, bool v_as_columns, uint32_t* info) {
    SvdSmallParams p{};
    p.r = r; p.s = s; p.ur = ur; p.v = v; p.info = info;
    p.batch = batch; p.k = k;
    p.max_sweeps = 30;                                           // SvdOptions::max_sweeps, core.h:705
    const float rows = (float)(effective_rows > 64u ? effective_rows : 64u);   // kMinEffectiveRows, src/svd.mm:60
    p.tol = sqrtf(rows) * FLT_EPSILON;
    p.v_as_columns = v_as_columns ? 1 : 0;
    const bool vectors = ur != nullptr;
    if (k <= 4) launch_jacobi<4>(stream, p, vectors);
    else if (k <= 8) launch_jacobi<8>(stream, p, vectors);
    else if (k <= 16) launch_jacobi<16>(stream, p, vectors);
    else if (k <= 32) launch_jacobi<32>(stream, p, vectors);
    else launch_block_jacobi(stream, p, vectors);
    cuda_check(cudaGetLastError(), "svd_small launch");
}

void launch_svd_left_vectors(cudaStream_t stream, const float* q, const float* ur, float* out, uint32_t batch, uint32_t l,
                             uint32_t k, bool transposed) {
    if (k > 32) {
        static PerDeviceOnce once;
        if (const int device = current_device(); once.first(device)) {
            cuda_check(cudaFuncSetAttribute(svd_left_vectors_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)((128 * 128 + 64 * 129) * sizeof(float))), "svd_left_vectors shared memory");
            once.mark(device);
        }
        const size_t smem = ((size_t)k * k + 64 * (k + 1)) * sizeof(float);
        for (uint32_t b0 = 0; b0 < batch; b0 += 65535) {      // the batch along y in slices
            const uint32_t nb = batch - b0 < 65535 ? batch - b0 : 65535;
            launch_dependent(svd_left_vectors_wide_kernel, dim3((l + 63) / 64, nb), 256, smem, stream, q + (size_t)b0 * l * k,
                             ur + (size_t)b0 * k * k, out + (size_t)b0 * l * k, l, k, transposed ? 1 : 0);
        }
        cuda_check(cudaGetLastError(), "svd_left_vectors launch");
        return;
    }
    const size_t rows = (size_t)batch * l;
    const uint32_t blocks = (uint32_t)((rows + 255) / 256);
    const int t = transposed ? 1 : 0;
    if (k <= 4) launch_dependent(svd_left_vectors_kernel<4>, blocks, 256, 0, stream, q, ur, out, batch, l, k, t);
    else if (k <= 8) launch_dependent(svd_left_vectors_kernel<8>, blocks, 256, 0, stream, q, ur, out, batch, l, k, t);
    else if (k <= 16) launch_dependent(svd_left_vectors_kernel<16>, blocks, 256, 0, stream, q, ur, out, batch, l, k, t);
    else launch_dependent(svd_left_vectors_kernel<32>, blocks, 256, 0, stream, q, ur, out, batch, l, k, t);
    cuda_check(cudaGetLastError(), "svd_left_vectors launch");
}

void launch_transpose_batched(cudaStream_t stream, const float* in, float* out, uint32_t batch, uint32_t rows, uint32_t cols) {
    // the batch along z in slices of at most 65535
    for (uint32_t b0 = 0; b0 < batch; b0 += 65535) {
        const uint32_t nb = batch - b0 < 65535 ? batch - b0 : 65535;
        const size_t off = (size_t)b0 * rows * cols;
        launch_dependent(transpose_batched_kernel, dim3((cols + 31) / 32, (rows + 31) / 32, nb), 256, 0, stream, in + off,
                         out + off, rows, cols);
    }
    cuda_check(cudaGetLastError(), "transpose launch");
}

} // namespace mlb
