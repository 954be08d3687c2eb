// The C ABI (include/metal_linalg/c_api.h) over the buffer core. Three things
// happen here and nowhere else: a call's buffers are checked against the sizes
// its shape implies, a C++ exception becomes one of the four status codes with
// its message kept for metal_linalg_last_error(), and the C policy struct is
// mapped onto the core's. The contract is the reference's (src/c_api.cpp: status
// per exception class, thread-local message, NULL allowed only for a buffer that
// would hold nothing); the code is this build's own.
#include <metal_linalg/c_api.h>
#include <metal_linalg/core.h>

#include "kernels.h"
#include "runtime.h"

#include <algorithm>
#include <exception>
#include <new>
#include <stdexcept>
#include <string>

namespace ml = metal_linalg;

namespace {

// One message per thread; it lives until that thread's next failure.
thread_local std::string t_error;
thread_local std::string t_notice;

// The status of the exception in flight, its message recorded.
metal_linalg_status status_of_current_exception() {
    try {
        throw;
    } catch (const std::bad_alloc&) {
        t_error = "out of memory";
        return METAL_LINALG_OUT_OF_MEMORY;
    } catch (const std::invalid_argument& bad) {
        t_error = bad.what();
        return METAL_LINALG_INVALID_ARGUMENT;
    } catch (const std::exception& other) {       // CUDA failures, a kernel that gave up on a wait
        t_error = other.what();
        return METAL_LINALG_RUNTIME_ERROR;
    } catch (...) {
        t_error = "an exception that is not a std::exception";
        return METAL_LINALG_RUNTIME_ERROR;
    }
}

template <typename Body>
metal_linalg_status run(Body&& body) noexcept {
    try {
        body();
    } catch (...) {
        return status_of_current_exception();
    }
    return METAL_LINALG_OK;
}

// The same for the queries that return a value and have no status to give: `fallback` on any failure.
template <typename T, typename Body>
T query(T fallback, Body&& body) noexcept {
    try {
        return body();
    } catch (...) {
        status_of_current_exception();
        return fallback;
    }
}

// The buffers of one QR call, with the element counts its shape and mode imply.
struct QrCall {
    const char*      who;
    ml::core::QrMode mode;
    uint32_t         batch, rows, cols, q_cols, r_rows;

    QrCall(const char* who_, int c_mode, uint32_t b, uint32_t m, uint32_t n) : who(who_), batch(b), rows(m), cols(n) {
        switch (c_mode) {
            case METAL_LINALG_QR_REDUCED:  mode = ml::core::QrMode::reduced; break;
            case METAL_LINALG_QR_R:        mode = ml::core::QrMode::r; break;
            case METAL_LINALG_QR_COMPLETE: mode = ml::core::QrMode::complete; break;
            default:
                throw std::invalid_argument(std::string(who) + " mode must be METAL_LINALG_QR_REDUCED, _R or _COMPLETE");
        }
        q_cols = ml::core::qr_q_cols(mode, m, n);
        r_rows = ml::core::qr_r_rows(mode, m, n);
    }
    uint64_t a_count() const { return (uint64_t)batch * rows * cols; }
    uint64_t q_count() const { return (uint64_t)batch * rows * q_cols; }
    uint64_t r_count() const { return (uint64_t)batch * r_rows * cols; }
    // A buffer that holds at least one element has to be there.
    void need(const void* p, uint64_t count, const char* name) const {
        if (count != 0 && p == nullptr) throw std::invalid_argument(std::string(who) + " " + name + " is NULL");
    }
    void check(const float* a, const float* q, const float* r) const {
        need(a, a_count(), "a");
        need(q, q_count(), "q");      // q_count() is 0 for R alone: q is then never looked at
        need(r, r_count(), "r");
    }
};

// The policy's settable fields, C struct member against core struct member.
struct PolicyField {
    uint32_t metal_linalg_qr_policy::*c;
    unsigned ml::QrPolicy::*core;
    bool     informational;      // reported, never set
};
constexpr PolicyField kPolicyFields[] = {
    {&metal_linalg_qr_policy::m_crossover_small_batch, &ml::QrPolicy::m_crossover_small_batch, false},
    {&metal_linalg_qr_policy::m_crossover_large_batch, &ml::QrPolicy::m_crossover_large_batch, false},
    {&metal_linalg_qr_policy::batch_threshold, &ml::QrPolicy::batch_threshold, false},
    {&metal_linalg_qr_policy::gpu_max_k, &ml::QrPolicy::gpu_max_k, false},
    {&metal_linalg_qr_policy::gpu_min_batch_times_k, &ml::QrPolicy::gpu_min_batch_times_k, false},
    {&metal_linalg_qr_policy::gpu_min_batch, &ml::QrPolicy::gpu_min_batch, false},
    {&metal_linalg_qr_policy::gpu_cores, &ml::QrPolicy::gpu_cores, true},
    {&metal_linalg_qr_policy::concurrent_matrices, &ml::QrPolicy::concurrent_matrices, true},
    {&metal_linalg_qr_policy::gpu_large_min_k, &ml::QrPolicy::gpu_large_min_k, false},
    {&metal_linalg_qr_policy::gpu_large_max_batch, &ml::QrPolicy::gpu_large_max_batch, false},
    {&metal_linalg_qr_policy::gpu_min_k, &ml::QrPolicy::gpu_min_k, false},
    {&metal_linalg_qr_policy::share_min_batch, &ml::QrPolicy::share_min_batch, false},
};

} // namespace

extern "C" {

const char* metal_linalg_last_error(void) { return t_error.c_str(); }

// ---------------------------------------------------------------------------
// QR
// ---------------------------------------------------------------------------

metal_linalg_status metal_linalg_qr_with_mode(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                              metal_linalg_qr_mode mode, float* q, float* r) {
    return run([&] {
        const QrCall call("[qr]", (int)mode, batch, rows, cols);
        call.check(a, q, r);
        ml::core::qr({a, batch, rows, cols}, call.q_cols ? q : nullptr, r, call.mode);
    });
}

metal_linalg_status metal_linalg_qr(const float* a, uint32_t batch, uint32_t rows, uint32_t cols, float* q, float* r) {
    return metal_linalg_qr_with_mode(a, batch, rows, cols, METAL_LINALG_QR_REDUCED, q, r);
}

metal_linalg_status metal_linalg_qr_no_alloc(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                             metal_linalg_qr_mode mode, float* q, float* r) {
    return run([&] {
        const QrCall call("[qr_no_alloc]", (int)mode, batch, rows, cols);
        call.check(a, q, r);
        if (call.a_count() == 0) return;      // nothing to factor (and nothing to allocate for it)
        const int device = mlb::pointer_device(a);
        if (device < 0)
            throw std::invalid_argument("[qr_no_alloc] takes CUDA device pointers only (staging host memory would allocate)");
        if (mlb::pointer_device(r) != device || (call.q_cols && mlb::pointer_device(q) != device))
            throw std::invalid_argument("[qr_no_alloc] a, q and r must be device pointers on one GPU");
        mlb::QrProblem p{};
        p.a = a; p.q = call.q_cols ? q : nullptr; p.r = r;
        p.batch = batch; p.m = rows; p.n = cols; p.qc = call.q_cols; p.rr = call.r_rows;
        mlb::launch_qr_mid_static(device, mlb::thread_stream(), p);
    });
}

uint64_t metal_linalg_qr_no_alloc_scratch_bytes(void) { return mlb::qr_mid_static_capacity_bytes(); }

// ---------------------------------------------------------------------------
// SVD
// ---------------------------------------------------------------------------

metal_linalg_status metal_linalg_svd(const float* a, uint32_t batch, uint32_t rows, uint32_t cols, float* u, float* s,
                                     float* vt, uint32_t* info) {
    return run([&] {
        const uint64_t k = std::min(rows, cols);
        if ((uint64_t)batch * rows * cols != 0 && !a) throw std::invalid_argument("[svd] a is NULL");
        if ((uint64_t)batch * k != 0 && !s) throw std::invalid_argument("[svd] s is NULL");
        if ((u == nullptr) != (vt == nullptr))
            throw std::invalid_argument("[svd] u and vt must both be given or both be NULL");
        ml::core::svd({a, batch, rows, cols}, u, s, vt, info);
    });
}

const char* metal_linalg_svd_backend(uint32_t rows, uint32_t cols, uint32_t batch) {
    return query<const char*>("unavailable", [&] {
        return ml::svd_backend(rows, cols, batch) == ml::SvdBackend::qr_jacobi ? "qr_jacobi" : "unavailable";
    });
}
const char* metal_linalg_svdvals_backend(uint32_t rows, uint32_t cols, uint32_t batch) {
    return query<const char*>("unavailable", [&] {
        return ml::svdvals_backend(rows, cols, batch) == ml::SvdBackend::qr_jacobi ? "qr_jacobi" : "unavailable";
    });
}

// ---------------------------------------------------------------------------
// Placement, waiting, memory
// ---------------------------------------------------------------------------

void  metal_linalg_set_stream(void* cuda_stream) { ml::set_stream(cuda_stream); }
void* metal_linalg_stream(void) { return ml::stream(); }

metal_linalg_status metal_linalg_set_device(int device) {
    return run([&] { ml::set_device(device); });
}
int metal_linalg_device(void) { return ml::device(); }
int metal_linalg_device_count(void) { return ml::device_count(); }

metal_linalg_status metal_linalg_synchronize(void) {
    return run([] { ml::synchronize(); });
}

metal_linalg_status metal_linalg_release_workspaces(uint64_t* bytes_freed) {
    return run([&] {
        const size_t freed = ml::release_workspaces();
        if (bytes_freed) *bytes_freed = freed;
    });
}

void metal_linalg_inject_wait_failures(int count) { ml::inject_wait_failures(count); }

// ---------------------------------------------------------------------------
// Device, host threads, routing
// ---------------------------------------------------------------------------

const char* metal_linalg_device_name(void) {
    return query<const char*>("", [] { return ml::device_name(); });
}
uint32_t metal_linalg_gpu_core_count(void) {
    return query<uint32_t>(0u, [] { return (uint32_t)ml::gpu_core_count(); });
}

void        metal_linalg_set_calibration_notices(int) {}
const char* metal_linalg_calibration_message(const char* decomposition) {
    t_notice.clear();
    if (decomposition && std::string(decomposition) == "QR") {
        const std::string source = query<std::string>(std::string(), [] { return std::string(ml::qr_policy_source()); });
        if (source.compare(0, 8, "default:") == 0)
            t_notice = "metal-linalg: the QR routing table was measured on an NVIDIA B200; " + source;
    }
    return t_notice.c_str();
}

void     metal_linalg_set_cpu_threads(uint32_t n) { ml::set_cpu_threads(n); }
uint32_t metal_linalg_cpu_threads(void) { return ml::cpu_threads(); }
void     metal_linalg_set_cpu_only(int on) { ml::set_cpu_only(on != 0); }
int      metal_linalg_cpu_only(void) { return ml::cpu_only() ? 1 : 0; }

const char* metal_linalg_qr_backend(uint32_t rows, uint32_t cols, uint32_t batch) {
    return query<const char*>("unblocked", [&] {
        return ml::qr_backend(rows, cols, batch) == ml::QrBackend::streaming_reduced ? "streaming_reduced" : "unblocked";
    });
}

const char* metal_linalg_qr_kernel(uint32_t rows, uint32_t cols, uint32_t batch, metal_linalg_qr_mode mode) {
    return query<const char*>("", [&] {
        const QrCall call("[qr_kernel]", (int)mode, batch, rows, cols);
        return ml::core::qr_kernel_name(ml::core::qr_kernel(rows, cols, batch, call.mode));
    });
}

metal_linalg_qr_policy metal_linalg_qr_policy_get(void) {
    metal_linalg_qr_policy out{};
    const ml::QrPolicy now = query<ml::QrPolicy>(ml::QrPolicy{}, [] { return ml::qr_policy(); });
    for (const PolicyField& f : kPolicyFields) out.*f.c = now.*f.core;
    return out;
}

void metal_linalg_qr_policy_set(const metal_linalg_qr_policy* wanted) {
    if (!wanted) return;
    run([&] {
        ml::QrPolicy next = ml::qr_policy();      // the informational fields keep what was detected
        for (const PolicyField& f : kPolicyFields)
            if (!f.informational) next.*f.core = wanted->*f.c;
        ml::set_qr_policy(next);
    });
}

const char* metal_linalg_qr_policy_source(void) {
    return query<const char*>("default:untuned-device", [] { return ml::qr_policy_source(); });
}

} // extern "C"
