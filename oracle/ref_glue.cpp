// TEST INFRASTRUCTURE ONLY: never linked into the product library.
//
// Glue that lets the reference's CPU QR (src/qr_cpu.mm, compiled unchanged from
// the reference checkout) run on Linux: the host helpers it expects from its
// Metal runtime, the thread-count setting of device.h, and a C entry point the
// tests and the bench's CPU-baseline leg call through ctypes.
//
//   scan            follows src/metal_runtime.mm:140-170 (max |x| and finiteness per matrix)
//   lapack_batches  follows src/metal_runtime.mm:402-432 (four chunks per thread, the BLAS
//                   single-threaded inside; one matrix keeps the BLAS's own threads)
//   cpu_threads     follows src/device.mm (every core unless set)
#include "shim/metal_runtime.h"

#include <algorithm>
#include <atomic>
#include <cfloat>
#include <cmath>
#include <exception>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void  scipy_openblas_set_num_threads(int n);
int   scipy_openblas_get_num_threads(void);
char* scipy_openblas_get_config(void);
}

namespace metal_linalg {

namespace {
std::atomic<unsigned> g_threads{0};
}

void     set_cpu_threads(unsigned n) { g_threads = n; }
unsigned cpu_threads() {
    const unsigned n = g_threads.load();
    return n ? n : std::max(1u, std::thread::hardware_concurrency());
}

namespace detail {

void scan(const core::Matrices& a, Part, float* amax, char* finite) {
    const size_t per = (size_t)a.rows * a.cols;
    for (uint32_t b = 0; b < a.batch; ++b) {
        const float* d = a.data + b * per;
        float m = 0.0f;
        unsigned ok = 1;
        for (size_t i = 0; i < per; ++i) {
            const float v = std::fabs(d[i]);
            ok &= (unsigned)(v <= FLT_MAX);
            m = v > m ? v : m;
        }
        amax[b] = m;
        finite[b] = ok ? 1 : 0;
    }
}

void lapack_batches(uint32_t batch, size_t, const std::function<void(uint32_t, uint32_t)>& f) {
    const uint32_t threads = std::min<uint32_t>(cpu_threads(), batch);
    if (threads <= 1) {
        if (batch) {
            const int before = scipy_openblas_get_num_threads();
            scipy_openblas_set_num_threads((int)cpu_threads());
            f(0, batch);
            scipy_openblas_set_num_threads(before);
        }
        return;
    }
    const uint32_t chunks = std::min<uint32_t>(batch, threads * 4);
    std::atomic<uint32_t> next{0};
    std::atomic<bool> failed{false};
    std::mutex m;
    std::exception_ptr error;
    const int before = scipy_openblas_get_num_threads();
    scipy_openblas_set_num_threads(1);
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < threads; ++t) {
        pool.emplace_back([&] {
            for (uint32_t c; !failed && (c = next.fetch_add(1)) < chunks;) {
                const uint32_t b0 = (uint32_t)((uint64_t)batch * c / chunks);
                const uint32_t b1 = (uint32_t)((uint64_t)batch * (c + 1) / chunks);
                try {
                    f(b0, b1);
                } catch (...) {
                    std::lock_guard<std::mutex> lock(m);
                    if (!error) error = std::current_exception();
                    failed = true;
                }
            }
        });
    }
    for (auto& t : pool) t.join();
    scipy_openblas_set_num_threads(before);
    if (error) std::rethrow_exception(error);
}

} // namespace detail
} // namespace metal_linalg

namespace {
thread_local std::string g_error;
}

extern "C" {

// The reference's qr_cpu on `batch` row-major rows x cols matrices. mode: 0 reduced,
// 1 R alone (q may be null), 2 complete. threads: 0 for every core. Returns 0, or 1
// with the message in ref_last_error().
int ref_qr_cpu(const float* a, uint32_t batch, uint32_t rows, uint32_t cols, int mode, float* q, float* r,
               unsigned threads) {
    using namespace metal_linalg;
    try {
        set_cpu_threads(threads);
        const core::QrMode m = mode == 1 ? core::QrMode::r : mode == 2 ? core::QrMode::complete
                                                                        : core::QrMode::reduced;
        core::detail::qr_cpu({a, batch, rows, cols}, m == core::QrMode::r ? nullptr : q, r, m);
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}

const char* ref_last_error(void) { return g_error.c_str(); }
unsigned    ref_cpu_threads(void) { return metal_linalg::cpu_threads(); }
const char* ref_lapack_config(void) { return scipy_openblas_get_config(); }

} // extern "C"
