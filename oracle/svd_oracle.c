/* TEST INFRASTRUCTURE ONLY: nothing the library ships may call this.
 *
 * A CPU restatement, in plain C and float32, of the reference's QR-preconditioned SVD for
 * min(M, N) small: svd_qr_jacobi (src/svd.mm:614-661), i.e. A = Q R by the Householder QR of
 * qr_oracle.c, then Hestenes' one-sided Jacobi on R as the reference's kernel does it
 * (shaders/Svd_Jacobi.metal:159-372): power-of-two scaling, the round-robin order of
 * tournament_pair (shaders/eigh_jacobi_common.h:54-67), a pair rotated iff |gamma| > tol
 * sqrt(alpha beta) with tol = sqrt(max(rows, 64)) eps (src/svd.mm:511-513), the rules for null
 * columns (Svd_Jacobi.metal:171-209,236-271), the descending order with ties by index
 * (:322-331), zero left vectors for null columns completed to an orthonormal basis
 * (src/svd.mm:148-186; the completing vectors are not unique, so only their orthonormality is
 * comparable), NaN outputs and the info word (c_api.h:96-102).
 *
 * Pinned by: the reference's own known-answer case (tests/test_c_api.c:97-111: the 2 x 3
 * matrix with rows of norms 3 and 2) and float64 LAPACK singular values (numpy) on seeded
 * inputs and LAPACK sgesdd fixtures (tests/golden/svd_golden.npz), in tests/test_svd.py. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int oracle_qr(const float* a, uint32_t batch, uint32_t m, uint32_t n, int mode, float* q, float* r);

#define EPS32 1.1920929e-7f
static const float kNullTol = 32.0f * EPS32, kNegligible = 1.2e-7f, kCleanCos = 0.05f, kZetaAsymptotic = 1e15f;

static void pair_of(uint32_t round, uint32_t j, uint32_t n_even, uint32_t* p, uint32_t* q) {
    const uint32_t m = n_even - 1;
    uint32_t a, b;
    if (j == 0) { a = 0; b = 1 + (m - 1 + round) % m; }
    else { a = 1 + (j - 1 + round) % m; b = 1 + (m - 1 - j + round) % m; }
    *p = a < b ? a : b;
    *q = a < b ? b : a;
}

/* One k x k factor r (row-major) -> s, ur (k x k, columns), v (k x k, columns); returns info. */
static uint32_t jacobi(const float* r, uint32_t k, uint32_t rows, float* s, float* ur, float* v) {
    float* g = malloc(sizeof(float) * k * k);          /* column-major */
    int nonfinite = 0;
    float amax = 0.0f;
    for (uint32_t i = 0; i < k; ++i)
        for (uint32_t c = 0; c < k; ++c) {
            const float x = r[i * k + c];
            if (!isfinite(x)) nonfinite = 1;
            if (fabsf(x) > amax) amax = fabsf(x);
            g[c * k + i] = x;
        }
    int expo = 0;
    if (!nonfinite && amax > 0.0f) (void)frexpf(amax, &expo);
    for (uint32_t i = 0; i < k * k; ++i) g[i] = ldexpf(g[i], -expo);
    for (uint32_t i = 0; i < k * k; ++i) v[i] = 0.0f;
    for (uint32_t i = 0; i < k; ++i) v[i * k + i] = 1.0f;

    const float tol = sqrtf((float)(rows > 64 ? rows : 64)) * EPS32;
    const uint32_t n_even = (k + 1) & ~1u, np = n_even / 2;
    uint32_t sweeps = 0;
    int converged = 0;
    while (!nonfinite && sweeps < 30) {
        float cmax2 = 0.0f;
        for (uint32_t c = 0; c < k; ++c) {
            float acc = 0.0f;
            for (uint32_t i = 0; i < k; ++i) acc += g[c * k + i] * g[c * k + i];
            if (acc > cmax2) cmax2 = acc;
        }
        const float null2 = kNullTol * kNullTol * cmax2, negl2 = kNegligible * kNegligible * cmax2;
        int rotated = 0;
        for (uint32_t round = 0; round + 1 < n_even; ++round)
            for (uint32_t j = 0; j < np; ++j) {
                uint32_t p, q;
                pair_of(round, j, n_even, &p, &q);
                if (q >= k) continue;
                float *gp = g + p * k, *gq = g + q * k;
                float alpha = 0.0f, beta = 0.0f, gamma = 0.0f;
                for (uint32_t i = 0; i < k; ++i) { alpha += gp[i] * gp[i]; beta += gq[i] * gq[i]; gamma += gp[i] * gq[i]; }
                if (alpha <= null2 && beta <= null2) continue;
                const float ab = alpha * beta;
                if (fabsf(gamma) > tol * sqrtf(ab)) {
                    const float zeta = (beta - alpha) / (2.0f * gamma);
                    float t;
                    if (fabsf(zeta) > kZetaAsymptotic) t = 0.5f / zeta;
                    else {
                        t = 1.0f / (fabsf(zeta) + sqrtf(1.0f + zeta * zeta));
                        if (zeta < 0.0f) t = -t;
                    }
                    const float c = 1.0f / sqrtf(1.0f + t * t), sn = c * t;
                    for (uint32_t i = 0; i < k; ++i) {
                        const float x = gp[i], y = gq[i];
                        gp[i] = c * x - sn * y;
                        gq[i] = sn * x + c * y;
                    }
                    float *vp = v + p * k, *vq = v + q * k;
                    for (uint32_t i = 0; i < k; ++i) {
                        const float x = vp[i], y = vq[i];
                        vp[i] = c * x - sn * y;
                        vq[i] = sn * x + c * y;
                    }
                    const int one_null = alpha <= null2 || beta <= null2;
                    if (!one_null) rotated = 1;
                    else if (fminf(alpha, beta) > negl2 && gamma * gamma > kCleanCos * kCleanCos * ab) rotated = 1;
                }
            }
        ++sweeps;
        if (!rotated) { converged = 1; break; }
    }

    float* sig = malloc(sizeof(float) * k);
    uint32_t* rank = malloc(sizeof(uint32_t) * k);
    float smax = 0.0f;
    for (uint32_t c = 0; c < k; ++c) {
        float acc = 0.0f;
        for (uint32_t i = 0; i < k; ++i) acc += g[c * k + i] * g[c * k + i];
        sig[c] = sqrtf(acc);
        if (sig[c] > smax) smax = sig[c];
    }
    for (uint32_t c = 0; c < k; ++c) {
        uint32_t before = 0;
        for (uint32_t d = 0; d < k; ++d) before += (sig[d] > sig[c] || (sig[d] == sig[c] && d < c)) ? 1u : 0u;
        rank[c] = nonfinite ? c : before;      /* NaN compares false with everything */
    }
    const float thr = kNullTol * smax;
    int deficient = 0;
    float* vcols = malloc(sizeof(float) * k * k);
    memcpy(vcols, v, sizeof(float) * k * k);
    for (uint32_t c = 0; c < k; ++c) {
        if (!(sig[c] > thr)) deficient = 1;
        s[rank[c]] = nonfinite ? NAN : ldexpf(sig[c], expo);
        for (uint32_t i = 0; i < k; ++i) {
            ur[i * k + rank[c]] = nonfinite ? NAN : (sig[c] > thr ? g[c * k + i] / sig[c] : 0.0f);
            v[i * k + rank[c]] = nonfinite ? NAN : vcols[c * k + i];      /* v: row-major, vectors as columns */
        }
    }
    /* null columns: a unit vector orthogonal to the columns in place (Gram-Schmidt in double, three
     * passes, from a fixed pseudo-random start) */
    if (deficient && !nonfinite) {
        double* w = malloc(sizeof(double) * k);
        char* valid = calloc(k, 1);
        for (uint32_t c = 0; c < k; ++c)
            for (uint32_t i = 0; i < k; ++i)
                if (ur[i * k + c] != 0.0f) valid[c] = 1;
        uint64_t state = 88172645463325252ull;
        for (uint32_t c = 0; c < k; ++c) {
            for (int attempt = 0; attempt < 8 && !valid[c]; ++attempt) {
                double start = 0.0;
                for (uint32_t i = 0; i < k; ++i) {
                    state ^= state << 13; state ^= state >> 7; state ^= state << 17;
                    w[i] = (double)(state >> 11) / 9007199254740992.0 - 0.5;
                    start += w[i] * w[i];
                }
                for (int pass = 0; pass < 3; ++pass)
                    for (uint32_t d = 0; d < k; ++d) {
                        if (!valid[d]) continue;
                        double dot = 0.0;
                        for (uint32_t i = 0; i < k; ++i) dot += (double)ur[i * k + d] * w[i];
                        for (uint32_t i = 0; i < k; ++i) w[i] -= dot * (double)ur[i * k + d];
                    }
                double nrm = 0.0;
                for (uint32_t i = 0; i < k; ++i) nrm += w[i] * w[i];
                if (nrm > 1e-12 * start) {
                    for (uint32_t i = 0; i < k; ++i) ur[i * k + c] = (float)(w[i] / sqrt(nrm));
                    valid[c] = 1;
                }
            }
        }
        free(w); free(valid);
    }
    free(g); free(sig); free(rank); free(vcols);
    return sweeps | (converged ? 1u << 16 : 0u) | (nonfinite ? 1u << 17 : 0u) | ((deficient && !nonfinite) ? 1u << 18 : 0u);
}

/* Thin SVD of `batch` row-major m x n matrices, K = min(m, n) (any K; the cost is O(K^3) a sweep):
 * u [batch, m, K] or NULL (with vt), s [batch, K], vt [batch, K, n], info [batch] or NULL. */
int oracle_svd(const float* a, uint32_t batch, uint32_t m, uint32_t n, float* u, float* s, float* vt, uint32_t* info) {
    const int wide = m < n;
    const uint32_t l = wide ? n : m, k = wide ? m : n;
    if (k == 0 || batch == 0) return 0;
    float *tall = malloc(sizeof(float) * l * k), *q = malloc(sizeof(float) * l * k), *r = malloc(sizeof(float) * k * k),
          *ur = malloc(sizeof(float) * k * k), *v = malloc(sizeof(float) * k * k), *sv = malloc(sizeof(float) * k);
    for (uint32_t b = 0; b < batch; ++b) {
        const float* ab = a + (size_t)b * m * n;
        if (wide) { for (uint32_t i = 0; i < m; ++i) for (uint32_t j = 0; j < n; ++j) tall[j * k + i] = ab[i * n + j]; }
        else memcpy(tall, ab, sizeof(float) * l * k);
        if (oracle_qr(tall, 1, l, k, 0, q, r) != 0) return 1;
        const uint32_t word = jacobi(r, k, l, sv, ur, v);
        if (info) info[b] = word;
        memcpy(s + (size_t)b * k, sv, sizeof(float) * k);
        if (!u) continue;
        float* ub = u + (size_t)b * m * k;
        float* vb = vt + (size_t)b * k * n;
        /* left = Q U_R (l x k); right vectors = columns of v */
        for (uint32_t i = 0; i < l; ++i)
            for (uint32_t j = 0; j < k; ++j) {
                float acc = 0.0f;
                for (uint32_t t = 0; t < k; ++t) acc += q[i * k + t] * ur[t * k + j];
                if (wide) vb[j * n + i] = acc; else ub[i * k + j] = acc;
            }
        for (uint32_t i = 0; i < k; ++i)
            for (uint32_t j = 0; j < k; ++j) {
                if (wide) ub[i * k + j] = v[i * k + j];      /* U = V' */
                else vb[j * n + i] = v[i * k + j];           /* Vt row j = vector j */
            }
    }
    free(tall); free(q); free(r); free(ur); free(v); free(sv);
    return 0;
}
