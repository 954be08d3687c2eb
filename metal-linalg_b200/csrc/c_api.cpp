// The C ABI (include/metal_linalg/c_api.h) over the buffer core: argument checks,
// and exceptions turned into status codes with the message kept per thread
// (reference: src/c_api.cpp:15-35,97-124,301-330).
#include <metal_linalg/c_api.h>
#include <metal_linalg/core.h>

#include "kernels.h"
#include "runtime.h"

#include <algorithm>
#include <new>
#include <stdexcept>
#include <string>

using namespace metal_linalg;

namespace {

thread_local std::string g_last_error;
thread_local std::string g_message;

template <class F>
metal_linalg_status guarded(F&& f) {
    try {
        f();
        return METAL_LINALG_OK;
    } catch (const std::invalid_argument& e) {
        g_last_error = e.what();
        return METAL_LINALG_INVALID_ARGUMENT;
    } catch (const std::bad_alloc&) {
        g_last_error = "out of memory";
        return METAL_LINALG_OUT_OF_MEMORY;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return METAL_LINALG_RUNTIME_ERROR;
    } catch (...) {
        g_last_error = "unknown error";
        return METAL_LINALG_RUNTIME_ERROR;
    }
}

void require(bool ok, const char* what) {
    if (!ok) throw std::invalid_argument(what);
}

// Inputs and required outputs may be null only when they hold nothing.
bool present(const void* p, uint64_t count) { return p != nullptr || count == 0; }

core::QrMode mode_of(metal_linalg_qr_mode mode) {
    require(mode == METAL_LINALG_QR_REDUCED || mode == METAL_LINALG_QR_R || mode == METAL_LINALG_QR_COMPLETE,
            "[qr] mode must be METAL_LINALG_QR_REDUCED, _R or _COMPLETE");
    return mode == METAL_LINALG_QR_R ? core::QrMode::r
           : mode == METAL_LINALG_QR_COMPLETE ? core::QrMode::complete : core::QrMode::reduced;
}

} // namespace

extern "C" {

const char* metal_linalg_last_error(void) { return g_last_error.c_str(); }

metal_linalg_status metal_linalg_qr(const float* a, uint32_t batch, uint32_t rows, uint32_t cols, float* q,
                                    float* r) {
    return guarded([&] {
        const uint64_t k = std::min(rows, cols);
        require(present(a, (uint64_t)batch * rows * cols), "[qr] a is NULL");
        require(present(q, (uint64_t)batch * rows * k), "[qr] q is NULL");
        require(present(r, (uint64_t)batch * k * cols), "[qr] r is NULL");
        core::qr({a, batch, rows, cols}, q, r);
    });
}

metal_linalg_status metal_linalg_qr_with_mode(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                              metal_linalg_qr_mode mode, float* q, float* r) {
    return guarded([&] {
        const core::QrMode m = mode_of(mode);
        const uint64_t qc = core::qr_q_cols(m, rows, cols), rr = core::qr_r_rows(m, rows, cols);
        require(present(a, (uint64_t)batch * rows * cols), "[qr] a is NULL");
        if (qc) require(present(q, (uint64_t)batch * rows * qc), "[qr] q is NULL");
        require(present(r, (uint64_t)batch * rr * cols), "[qr] r is NULL");
        core::qr({a, batch, rows, cols}, qc ? q : nullptr, r, m);
    });
}

metal_linalg_status metal_linalg_qr_no_alloc(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                             metal_linalg_qr_mode mode, float* q, float* r) {
    return guarded([&] {
        const core::QrMode m = mode_of(mode);
        const uint32_t qc = core::qr_q_cols(m, rows, cols), rr = core::qr_r_rows(m, rows, cols);
        require(present(a, (uint64_t)batch * rows * cols), "[qr_no_alloc] a is NULL");
        if (qc) require(present(q, (uint64_t)batch * rows * qc), "[qr_no_alloc] q is NULL");
        require(present(r, (uint64_t)batch * rr * cols), "[qr_no_alloc] r is NULL");
        if (batch == 0 || rows == 0 || cols == 0) return;   // nothing to factor (and nothing to allocate for it)
        const int device = mlb::pointer_device(a);
        require(device >= 0, "[qr_no_alloc] takes CUDA device pointers only (staging host memory would allocate)");
        require(mlb::pointer_device(r) == device && (!qc || mlb::pointer_device(q) == device),
                "[qr_no_alloc] a, q and r must be device pointers on one GPU");
        mlb::QrProblem p{};
        p.a = a; p.q = qc ? q : nullptr; p.r = r;
        p.batch = batch; p.m = rows; p.n = cols; p.qc = qc; p.rr = rr;
        mlb::launch_qr_mid_static(device, mlb::thread_stream(), p);
    });
}

uint64_t metal_linalg_qr_no_alloc_scratch_bytes(void) { return mlb::qr_mid_static_capacity_bytes(); }

metal_linalg_status metal_linalg_svd(const float* a, uint32_t batch, uint32_t rows, uint32_t cols, float* u, float* s,
                                     float* vt, uint32_t* info) {
    return guarded([&] {
        require(present(a, (uint64_t)batch * rows * cols), "[svd] a is NULL");
        require(present(s, (uint64_t)batch * std::min(rows, cols)), "[svd] s is NULL");
        require((u == nullptr) == (vt == nullptr), "[svd] u and vt must both be given or both be NULL");
        core::svd({a, batch, rows, cols}, u, s, vt, info);
    });
}
const char* metal_linalg_svd_backend(uint32_t rows, uint32_t cols, uint32_t batch) {
    return svd_backend(rows, cols, batch) == SvdBackend::qr_jacobi ? "qr_jacobi" : "unavailable";
}
const char* metal_linalg_svdvals_backend(uint32_t rows, uint32_t cols, uint32_t batch) {
    return svdvals_backend(rows, cols, batch) == SvdBackend::qr_jacobi ? "qr_jacobi" : "unavailable";
}

void  metal_linalg_set_stream(void* cuda_stream) { set_stream(cuda_stream); }
void* metal_linalg_stream(void) { return stream(); }

metal_linalg_status metal_linalg_set_device(int device) {
    return guarded([&] { set_device(device); });
}
int metal_linalg_device(void) { return device(); }
int metal_linalg_device_count(void) { return device_count(); }

metal_linalg_status metal_linalg_synchronize(void) {
    return guarded([&] { synchronize(); });
}

const char* metal_linalg_device_name(void) {
    try {
        return device_name();
    } catch (...) {
        return "";
    }
}
uint32_t metal_linalg_gpu_core_count(void) {
    try {
        return gpu_core_count();
    } catch (...) {
        return 0;
    }
}

void        metal_linalg_set_calibration_notices(int) {}
const char* metal_linalg_calibration_message(const char* decomposition) {
    g_message.clear();
    if (!decomposition) return g_message.c_str();
    try {
        const std::string source = qr_policy_source();
        if (std::string(decomposition) == "QR" && source.rfind("default:", 0) == 0)
            g_message = "metal-linalg: the QR routing table was measured on an NVIDIA B200; " + source;
    } catch (...) {
    }
    return g_message.c_str();
}

void     metal_linalg_set_cpu_threads(uint32_t n) { set_cpu_threads(n); }
uint32_t metal_linalg_cpu_threads(void) { return cpu_threads(); }
void     metal_linalg_set_cpu_only(int on) { set_cpu_only(on != 0); }
int      metal_linalg_cpu_only(void) { return cpu_only() ? 1 : 0; }

const char* metal_linalg_qr_backend(uint32_t rows, uint32_t cols, uint32_t batch) {
    try {
        return qr_backend(rows, cols, batch) == QrBackend::streaming_reduced ? "streaming_reduced" : "unblocked";
    } catch (...) {
        return "unblocked";
    }
}

const char* metal_linalg_qr_kernel(uint32_t rows, uint32_t cols, uint32_t batch, metal_linalg_qr_mode mode) {
    try {
        return core::qr_kernel_name(core::qr_kernel(rows, cols, batch, mode_of(mode)));
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return "";
    }
}

metal_linalg_qr_policy metal_linalg_qr_policy_get(void) {
    metal_linalg_qr_policy out{};
    try {
        const QrPolicy p = qr_policy();
        out.m_crossover_small_batch = p.m_crossover_small_batch;
        out.m_crossover_large_batch = p.m_crossover_large_batch;
        out.batch_threshold         = p.batch_threshold;
        out.gpu_max_k               = p.gpu_max_k;
        out.gpu_min_batch_times_k   = p.gpu_min_batch_times_k;
        out.gpu_min_batch           = p.gpu_min_batch;
        out.gpu_cores               = p.gpu_cores;
        out.concurrent_matrices     = p.concurrent_matrices;
        out.gpu_large_min_k         = p.gpu_large_min_k;
        out.gpu_large_max_batch     = p.gpu_large_max_batch;
        out.gpu_min_k               = p.gpu_min_k;
        out.share_min_batch         = p.share_min_batch;
    } catch (...) {
    }
    return out;
}

void metal_linalg_qr_policy_set(const metal_linalg_qr_policy* in) {
    if (!in) return;
    try {
        QrPolicy p = qr_policy();
        p.m_crossover_small_batch = in->m_crossover_small_batch;
        p.m_crossover_large_batch = in->m_crossover_large_batch;
        p.batch_threshold         = in->batch_threshold;
        p.gpu_max_k               = in->gpu_max_k;
        p.gpu_min_batch_times_k   = in->gpu_min_batch_times_k;
        p.gpu_min_batch           = in->gpu_min_batch;
        p.gpu_large_min_k         = in->gpu_large_min_k;
        p.gpu_large_max_batch     = in->gpu_large_max_batch;
        p.gpu_min_k               = in->gpu_min_k;
        p.share_min_batch         = in->share_min_batch;
        set_qr_policy(p);
    } catch (...) {
    }
}

const char* metal_linalg_qr_policy_source(void) {
    try {
        return qr_policy_source();
    } catch (...) {
        return "default:untuned-device";
    }
}

} // extern "C"
