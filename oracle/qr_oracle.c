/* TEST INFRASTRUCTURE ONLY: the parity checker for the CUDA QR. Nothing in the
 * product library includes, links or calls this file; only tests/, the smoke
 * check and the bench's CPU-baseline leg load it.
 *
 * A plain-C restatement of the reference's CPU QR path, src/qr_cpu.mm:32-121,
 * which is LAPACK's sgeqrf + sorgqr per matrix on a row-major batch. LAPACK is
 * an external dependency of the reference (Apple's Accelerate, not vendored in
 * its tree), so its published algorithm is restated here in unblocked form:
 *
 *   slarfg   one reflector H = I - tau v v^T with v[0] = 1, beta = -sign(alpha) *
 *            ||(alpha, x)||, tau = (beta - alpha) / beta, x scaled by 1/(alpha - beta);
 *            tau = 0 (H = I) when the tail x is exactly zero
 *   sgeqr2   for each column j < K: reflector from A[j:, j], applied to A[j:, j+1:]
 *   sorg2r   Q's first `qc` columns from the K reflectors, backward
 *
 * and the contracts of qr_cpu.mm around them: row-major input and output
 * (qr_cpu.mm:79-83,111), R upper trapezoidal K x N with exact zeros below the
 * diagonal and, for a square Q, zero rows below K (qr_cpu.mm:91-94), R alone
 * skipping Q (qr_cpu.mm:95-104), a wide matrix factored by its leading block with
 * R2 = Q^T A2 (qr_cpu.mm:6-9,112-118; the same reflectors as factoring all
 * columns, which is what is done here), and a matrix holding a NaN or an infinity
 * giving all-NaN Q and R for that matrix alone (qr_cpu.mm:61-76).
 *
 * Arithmetic is float32 as the reference's, except that a reflector's norm is
 * accumulated in double, which stands in for snrm2's overflow-safe scaling.
 * Different LAPACK builds differ in rounding, and so does this: parity with the
 * reference is at tolerance level (checked against the reference's own qr_cpu
 * compiled into oracle/_ref, and against the committed fixtures in
 * tests/golden), never bit level. Parity status: pinned.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* One matrix. w: column-major work copy m x n (overwritten with R above the
 * diagonal and the reflectors below it); tau [K]. */
static void oracle_geqr2(float* w, uint32_t m, uint32_t n, float* tau) {
    const uint32_t K = m < n ? m : n;
    for (uint32_t j = 0; j < K; ++j) {
        float* col = w + (size_t)j * m;
        const float alpha = col[j];
        double ss = 0.0;
        for (uint32_t i = j + 1; i < m; ++i) ss += (double)col[i] * (double)col[i];
        if (ss == 0.0) {
            tau[j] = 0.0f;
            continue;
        }
        const double norm = sqrt((double)alpha * (double)alpha + ss);
        const float  beta = (float)(alpha >= 0.0f ? -norm : norm);
        tau[j] = (float)(((double)beta - (double)alpha) / (double)beta);
        const float scale = (float)(1.0 / ((double)alpha - (double)beta));
        for (uint32_t i = j + 1; i < m; ++i) col[i] *= scale;
        col[j] = beta;
        /* H applied to the columns to the right: c -= tau (v^T c) v */
        for (uint32_t c = j + 1; c < n; ++c) {
            float* x = w + (size_t)c * m;
            float  dot = x[j];
            for (uint32_t i = j + 1; i < m; ++i) dot += col[i] * x[i];
            const float t = tau[j] * dot;
            x[j] -= t;
            for (uint32_t i = j + 1; i < m; ++i) x[i] -= t * col[i];
        }
    }
}

/* Q's first qc columns (column-major m x qc) from the K reflectors in w. */
static void oracle_org2r(const float* w, uint32_t m, uint32_t K, const float* tau, float* q, uint32_t qc) {
    memset(q, 0, (size_t)m * qc * sizeof(float));
    for (uint32_t c = 0; c < qc; ++c) q[(size_t)c * m + c] = 1.0f;
    for (uint32_t jj = K; jj-- > 0;) {
        const float* v = w + (size_t)jj * m;
        if (tau[jj] == 0.0f) continue;
        for (uint32_t c = jj; c < qc; ++c) {
            float* x = q + (size_t)c * m;
            float  dot = x[jj];
            for (uint32_t i = jj + 1; i < m; ++i) dot += v[i] * x[i];
            const float t = tau[jj] * dot;
            x[jj] -= t;
            for (uint32_t i = jj + 1; i < m; ++i) x[i] -= t * v[i];
        }
    }
}

/* mode: 0 reduced, 1 R alone (q unused), 2 complete. Layout as the reference's C
 * API: a [batch, m, n], q [batch, m, QC], r [batch, RR, n], row-major. Returns 0,
 * or 1 if memory ran out. */
int oracle_qr(const float* a, uint32_t batch, uint32_t m, uint32_t n, int mode, float* q, float* r) {
    const uint32_t K = m < n ? m : n;
    if (K == 0 || batch == 0) return 0;
    const uint32_t QC = mode == 1 ? 0 : mode == 2 ? m : K;
    const uint32_t RR = mode == 2 ? m : K;
    int failed = 0;
#pragma omp parallel
    {
        float* w = (float*)malloc(((size_t)m * n + K + (size_t)m * (QC ? QC : 1)) * sizeof(float));
        if (!w) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (int64_t b = 0; b < (int64_t)batch; ++b) {
            if (!w) continue;
            float*       tau = w + (size_t)m * n;
            float*       qw = tau + K;
            const float* ab = a + (size_t)b * m * n;
            float*       qb = QC ? q + (size_t)b * m * QC : NULL;
            float*       rb = r + (size_t)b * RR * n;
            int          finite = 1;
            for (size_t i = 0; i < (size_t)m * n; ++i) finite &= fabsf(ab[i]) <= FLT_MAX;
            if (!finite) {
                for (size_t i = 0; qb && i < (size_t)m * QC; ++i) qb[i] = NAN;
                for (size_t i = 0; i < (size_t)RR * n; ++i) rb[i] = NAN;
                continue;
            }
            for (uint32_t i = 0; i < m; ++i)
                for (uint32_t j = 0; j < n; ++j) w[(size_t)j * m + i] = ab[(size_t)i * n + j];
            oracle_geqr2(w, m, n, tau);
            for (uint32_t i = 0; i < RR; ++i)
                for (uint32_t j = 0; j < n; ++j)
                    rb[(size_t)i * n + j] = (i < K && j >= i) ? w[(size_t)j * m + i] : 0.0f;
            if (!qb) continue;
            oracle_org2r(w, m, K, tau, qw, QC);
            for (uint32_t i = 0; i < m; ++i)
                for (uint32_t j = 0; j < QC; ++j) qb[(size_t)i * QC + j] = qw[(size_t)j * m + i];
        }
        free(w);
    }
    return failed;
}
