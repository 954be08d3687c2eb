// qr_accelerated, the C++ entry point, exercised on a GPU: its results against the C ABI's bit for
// bit, the modes, the input types, strided views, batch shapes and the argument errors. The cases
// follow the reference's dispatcher checks (tests/test_qr.cpp:449-454: 8x8, 32 x 64x64, 64x64,
// 128x128, 1024x512 through qr_accelerated, with its reconstruction / orthogonality / triangle
// properties, tests/test_qr.cpp:76-111) and the entry point's own contract (src/mlx_api.cpp:37-71,
// 122-149). Built by the package Makefile, run by tests/test_qr_accelerated.py. Exit code 0 = all passed.
#include <metal_linalg/c_api.h>
#include <metal_linalg/qr.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

using namespace metal_linalg;

static int g_failed = 0, g_checks = 0;

static void expect(bool ok, const std::string& what) {
    ++g_checks;
    if (!ok) {
        ++g_failed;
        std::printf("  FAIL  %s\n", what.c_str());
    } else {
        std::printf("  ok    %s\n", what.c_str());
    }
}

static std::vector<float> random_matrices(size_t count, unsigned seed) {
    std::mt19937 gen(seed);
    std::vector<float> v(count);
    // a sum of uniforms: the same numbers on every standard library (std::normal_distribution is not)
    for (auto& x : v) {
        double s = 0;
        for (int i = 0; i < 4; ++i) s += (double)(gen() >> 8) / (1 << 24) - 0.5;
        x = (float)(s * 1.7320508);
    }
    return v;
}

static bool same_bits(const std::vector<float>& a, const std::vector<float>& b) {
    return a.size() == b.size() && (a.empty() || std::memcmp(a.data(), b.data(), a.size() * sizeof(float)) == 0);
}

// The properties the reference's tests pin, in double on the host, for `batch` matrices m x n.
static void properties(const std::string& name, const std::vector<float>& A, const std::vector<float>& Q,
                       const std::vector<float>& R, size_t batch, size_t m, size_t n, size_t qc, size_t rr) {
    const size_t k = std::min(m, n);
    double recon = 0, orth = 0, low = 0, below = 0;
    for (size_t b = 0; b < batch; ++b) {
        const float* a = &A[b * m * n];
        const float* q = &Q[b * m * qc];
        const float* r = &R[b * rr * n];
        double num = 0, den = 0;
        for (size_t i = 0; i < m; ++i)
            for (size_t j = 0; j < n; ++j) {
                double s = 0;
                for (size_t t = 0; t < std::min(qc, rr); ++t) s += (double)q[i * qc + t] * r[t * n + j];
                num += (s - a[i * n + j]) * (s - a[i * n + j]);
                den += (double)a[i * n + j] * a[i * n + j];
            }
        recon = std::max(recon, std::sqrt(num / std::max(den, 1e-300)));
        double o = 0;
        for (size_t i = 0; i < qc; ++i)
            for (size_t j = 0; j < qc; ++j) {
                double s = 0;
                for (size_t t = 0; t < m; ++t) s += (double)q[t * qc + i] * q[t * qc + j];
                s -= i == j ? 1.0 : 0.0;
                o += s * s;
            }
        orth = std::max(orth, std::sqrt(o));
        for (size_t i = 0; i < rr; ++i)
            for (size_t j = 0; j < n; ++j) {
                if (i < k && j < i) low = std::max(low, (double)std::fabs(r[i * n + j]));
                if (i >= k) below = std::max(below, (double)std::fabs(r[i * n + j]));
            }
    }
    const double tol = 10.0 * n * std::ldexp(1.0, -23);
    char buf[256];
    std::snprintf(buf, sizeof buf, "%s: recon %.2e orth %.2e (tol %.2e), below-diagonal max %g, rows below K max %g", name.c_str(),
                  recon, orth, tol, low, below);
    expect(recon <= tol && orth <= tol && low == 0.0 && below == 0.0, buf);
}

template <class F>
static bool throws_invalid(F&& f) {
    try {
        f();
    } catch (const std::invalid_argument&) {
        return true;
    } catch (...) {
        return false;
    }
    return false;
}

int main() {
    if (device_count() == 0) {
        std::printf("no CUDA device: this library has no CPU path\n");
        return 2;
    }
    std::printf("[ qr_accelerated on %s ]\n", device_name());

    // 1. the three modes against the C ABI, bit for bit, on a batch of tall matrices
    {
        const uint32_t b = 5, m = 48, n = 20, k = 20;
        const auto host = random_matrices((size_t)b * m * n, 1);
        const Array a = Array::from_host(host.data(), {b, m, n});
        const struct { const char* mode; metal_linalg_qr_mode c; uint32_t qc, rr; } modes[] = {
            {"reduced", METAL_LINALG_QR_REDUCED, k, k}, {"r", METAL_LINALG_QR_R, 0, k}, {"complete", METAL_LINALG_QR_COMPLETE, m, m}};
        for (const auto& md : modes) {
            auto [q, r] = qr_accelerated(a, md.mode);
            Array q2(md.qc ? std::vector<uint32_t>{b, m, md.qc} : std::vector<uint32_t>{0}, 0), r2({b, md.rr, n}, 0);
            const auto status = metal_linalg_qr_with_mode(a.data(), b, m, n, md.c, md.qc ? q2.data() : nullptr, r2.data());
            expect(status == METAL_LINALG_OK, std::string("C ABI call, mode ") + md.mode);
            expect(r.shape() == std::vector<uint32_t>({b, md.rr, n}), std::string("R's shape, mode ") + md.mode);
            if (md.qc) expect(q.shape() == std::vector<uint32_t>({b, m, md.qc}), std::string("Q's shape, mode ") + md.mode);
            else expect(q.size() == 0, "mode r returns an empty first array");
            expect(same_bits(r.to_host(), r2.to_host()), std::string("R equals the C ABI's bit for bit, mode ") + md.mode);
            if (md.qc) {
                expect(same_bits(q.to_host(), q2.to_host()), std::string("Q equals the C ABI's bit for bit, mode ") + md.mode);
                properties(std::string("5 x 48x20 ") + md.mode, host, q.to_host(), r.to_host(), b, m, n, md.qc, md.rr);
            }
        }
        auto [qd, rd] = qr_accelerated(a);
        auto [qr_, rr_] = qr_accelerated(a, "reduced");
        expect(same_bits(qd.to_host(), qr_.to_host()) && same_bits(rd.to_host(), rr_.to_host()), "the default mode is \"reduced\"");
    }

    // 2. the reference's dispatcher cases
    {
        const struct { const char* name; uint32_t b, m, n; unsigned seed; } cases[] = {
            {"micro square 8x8", 1, 8, 8, 20}, {"small batched 32 x 64x64", 32, 64, 64, 21}, {"small unbatched 64x64", 1, 64, 64, 22},
            {"mid unbatched 128x128", 1, 128, 128, 23}, {"large 1024x512", 1, 1024, 512, 24}};
        for (const auto& c : cases) {
            const auto host = random_matrices((size_t)c.b * c.m * c.n, c.seed);
            auto [q, r] = qr_accelerated(Array::from_host(host.data(), {c.b, c.m, c.n}));
            const uint32_t k = std::min(c.m, c.n);
            properties(c.name, host, q.to_host(), r.to_host(), c.b, c.m, c.n, k, k);
        }
    }

    // 3. batch shapes: several leading dimensions, none, and an empty batch
    {
        const auto host = random_matrices(2 * 3 * 12 * 7, 3);
        auto [q4, r4] = qr_accelerated(Array::from_host(host.data(), {2, 3, 12, 7}));
        auto [q3, r3] = qr_accelerated(Array::from_host(host.data(), {6, 12, 7}));
        expect(q4.shape() == std::vector<uint32_t>({2, 3, 12, 7}) && r4.shape() == std::vector<uint32_t>({2, 3, 7, 7}),
               "[2, 3, 12, 7] keeps its leading dimensions");
        expect(same_bits(q4.to_host(), q3.to_host()) && same_bits(r4.to_host(), r3.to_host()),
               "[2, 3, 12, 7] equals [6, 12, 7]: the batch is the product of the leading dimensions");
        auto [q2, r2] = qr_accelerated(Array::from_host(host.data(), {12, 7}));
        expect(q2.shape() == std::vector<uint32_t>({12, 7}) && r2.shape() == std::vector<uint32_t>({7, 7}), "a single matrix [12, 7]");
        const auto q3h = q3.to_host();
        expect(same_bits(q2.to_host(), std::vector<float>(q3h.begin(), q3h.begin() + 84)), "[12, 7] equals the first matrix of the batch");
        auto [q0, r0] = qr_accelerated(Array({0, 9, 4}, 0), "complete");
        expect(q0.shape() == std::vector<uint32_t>({0, 9, 9}) && r0.shape() == std::vector<uint32_t>({0, 9, 4}) && q0.size() == 0,
               "an empty batch gives empty outputs of the right shape");
        auto [qi, ri] = qr_accelerated(Array({2, 5, 0}, 0), "complete");     // no columns: the complete Q is the identity
        const auto qh = qi.to_host();
        bool identity = qh.size() == 50;
        for (size_t i = 0; identity && i < qh.size(); ++i) identity = qh[i] == ((i % 25) / 5 == (i % 25) % 5 ? 1.0f : 0.0f);
        expect(identity && ri.size() == 0, "complete QR of a matrix with no columns: Q = I");
    }

    // 4. element types: computed in float32 whatever the input's real type
    {
        const uint32_t b = 3, m = 10, n = 6;
        std::vector<double> d((size_t)b * m * n);
        std::vector<int32_t> iv(d.size());
        std::vector<int64_t> lv(d.size());
        std::vector<uint8_t> uv(d.size());
        std::vector<float> f_of_d(d.size()), f_of_i(d.size());
        std::mt19937 gen(4);
        for (size_t i = 0; i < d.size(); ++i) {
            d[i] = (double)(gen() % 2000001) / 1e6 - 1.0 + 1e-12;
            f_of_d[i] = (float)d[i];
            iv[i] = (int32_t)(gen() % 19) - 9;
            lv[i] = iv[i];
            uv[i] = (uint8_t)(iv[i] + 9);
            f_of_i[i] = (float)iv[i];
        }
        auto [qf, rf] = qr_accelerated(Array::from_host(f_of_d.data(), {b, m, n}));
        auto [qd, rd] = qr_accelerated(Array::from_host(d.data(), Dtype::float64, {b, m, n}));
        expect(rd.dtype() == Dtype::float32 && same_bits(qd.to_host(), qf.to_host()) && same_bits(rd.to_host(), rf.to_host()),
               "float64 input: the float32 result of the rounded matrix");
        auto [qfi, rfi] = qr_accelerated(Array::from_host(f_of_i.data(), {b, m, n}));
        auto [qi, ri] = qr_accelerated(Array::from_host(iv.data(), Dtype::int32, {b, m, n}));
        auto [ql, rl] = qr_accelerated(Array::from_host(lv.data(), Dtype::int64, {b, m, n}));
        expect(same_bits(qi.to_host(), qfi.to_host()) && same_bits(ri.to_host(), rfi.to_host()), "int32 input");
        expect(same_bits(ql.to_host(), qfi.to_host()) && same_bits(rl.to_host(), rfi.to_host()), "int64 input");
        std::vector<float> f_of_u(d.size());
        for (size_t i = 0; i < d.size(); ++i) f_of_u[i] = (float)uv[i];
        auto [qfu, rfu] = qr_accelerated(Array::from_host(f_of_u.data(), {b, m, n}), "r");
        auto [qu, ru] = qr_accelerated(Array::from_host(uv.data(), Dtype::uint8, {b, m, n}), "r");
        expect(same_bits(ru.to_host(), rfu.to_host()), "uint8 input, mode r");
    }

    // 5. a strided view (the transposes of a batch) is made contiguous first
    {
        const uint32_t b = 4, m = 9, n = 14;
        const auto host = random_matrices((size_t)b * n * m, 5);          // stored [b, n, m]
        std::vector<float> transposed(host.size());
        for (uint32_t x = 0; x < b; ++x)
            for (uint32_t i = 0; i < m; ++i)
                for (uint32_t j = 0; j < n; ++j) transposed[((size_t)x * m + i) * n + j] = host[((size_t)x * n + j) * m + i];
        const Array stored = Array::from_host(host.data(), {b, n, m});
        const Array view = Array::view(stored.raw(), Dtype::float32, {b, m, n}, 0, {(int64_t)n * m, 1, (int64_t)m});
        expect(!view.contiguous(), "the transposed view is not contiguous");
        auto [qv, rv] = qr_accelerated(view, "complete");
        auto [qt, rt] = qr_accelerated(Array::from_host(transposed.data(), {b, m, n}), "complete");
        expect(same_bits(qv.to_host(), qt.to_host()) && same_bits(rv.to_host(), rt.to_host()), "a transposed view equals its contiguous copy");
    }

    // 6. argument errors (src/mlx_api.cpp:38-46,124-129)
    {
        const auto host = random_matrices(64, 6);
        const Array a = Array::from_host(host.data(), {8, 8});
        expect(throws_invalid([&] { qr_accelerated(a, "full"); }), "a bad mode throws std::invalid_argument");
        expect(throws_invalid([&] { qr_accelerated(a, "Reduced"); }), "mode strings are case-sensitive");
        expect(throws_invalid([&] { qr_accelerated(Array::from_host(host.data(), {64})); }), "a 1-D input throws");
        expect(throws_invalid([&] { qr_accelerated(Array::from_host(host.data(), Dtype::complex64, {4, 8})); }), "a complex input throws");
    }

    try {
        synchronize();
        expect(true, "synchronize() reports no kernel that gave up");
    } catch (const std::exception& e) {
        expect(false, std::string("synchronize(): ") + e.what());
    }
    std::printf("%d checks, %d failed\n", g_checks, g_failed);
    return g_failed ? 1 : 0;
}
