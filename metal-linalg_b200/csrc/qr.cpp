// The QR router and the buffer-core entry point core::qr: policy resolution
// (reference: src/qr.mm:114-209), kernel choice (reference: src/qr.mm:231-286,
// src/qr_householder.mm:263-275,387-391), pointer placement, and the staged
// pipeline for host pointers.
#include <metal_linalg/core.h>

#include "kernels.h"
#include "qr_enqueue.h"
#include "runtime.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

namespace metal_linalg {

using core::Matrices;
using core::QrKernel;
using core::QrMode;

// ---------------------------------------------------------------------------
// Policy
// ---------------------------------------------------------------------------
namespace {

struct ResolvedPolicy {
    QrPolicy    policy;
    std::string source;
};

// The one measured row: thresholds found on an NVIDIA B200 (148 multiprocessors).
// k from which one matrix is better spread over the grid than given to one block.
struct TunedRow {
    const char* device;
    unsigned    cores;
    unsigned    crossover_small_batch, crossover_large_batch, batch_threshold;
    unsigned    large_min_k, large_max_batch;
};
// Measured 2026-11 by tuning/tune_qr.py (tuning/results/nvidia-b200: 235 (shape, batch) points, two
// passes, shuffled; noise 0.2 % median). The block-per-matrix kernel takes the same time for 1 as for
// 148 matrices (one k x k matrix: 0.15 / 0.61 / 1.95 / 4.3 / 13.4 / 29.9 ms at k = 128 / 256 / 384 /
// 512 / 768 / 1024); the grid-parallel QR takes 0.39 / 0.78 / 1.2 / 1.6 / 2.5 / 3.4 ms for one and
// factors a batch several at a time (those were its times before its panels became one cluster
// launch; it is about a quarter faster now). The rule sqrt(M k) >= L sqrt(max(1, batch / F)) fitted
// on two thirds of the shapes is flat over L = 200 ... 270 and F = 2 ... 4; L = 240, F = 3 is taken (the
// fit's own choice since the block-per-matrix kernel stopped spilling registers on matrices of 330 to
// 512 rows): geometric-mean regret 1.006 on the training shapes, 1.000 on the held-out third. Beyond
// 1024 rows a block cannot hold the matrix.
constexpr TunedRow kTuned[] = {
    {"NVIDIA B200", 148, 1025, 1025, 16, 240, 0},
};

bool env_value(const char* name, unsigned& out) {
    const char* s = std::getenv(name);
    if (!s || !*s) return false;
    char* end = nullptr;
    const long long v = std::strtoll(s, &end, 10);
    if (end == s || v < 0) return false;
    out = v > 0xFFFFFFFFll ? kQrNoLimit : (unsigned)v;
    return true;
}

ResolvedPolicy resolve() {
    ResolvedPolicy r;
    const std::string name = device_name();
    r.policy.gpu_cores = gpu_core_count();
    r.policy.concurrent_matrices = 2 * r.policy.gpu_cores;
    for (const auto& e : kTuned) {
        if (name == e.device && r.policy.gpu_cores == e.cores) {
            r.policy.m_crossover_small_batch = e.crossover_small_batch;
            r.policy.m_crossover_large_batch = e.crossover_large_batch;
            r.policy.batch_threshold         = e.batch_threshold;
            r.policy.gpu_large_min_k         = e.large_min_k;
            r.policy.gpu_large_max_batch     = e.large_max_batch;
            r.source = "tuned:" + name;
        }
    }
    if (r.source.empty()) r.source = "default:untuned-device" + (name.empty() ? "" : " (" + name + ")");

    std::string env;
    unsigned crossover = 0;
    if (env_value("QR_M_CROSSOVER", crossover) && crossover > 0) {
        r.policy.m_crossover_small_batch = crossover;
        r.policy.m_crossover_large_batch = crossover;
        env = "QR_M_CROSSOVER";
    }
    auto over = [&](const char* n, unsigned& field) {
        if (env_value(n, field)) env += (env.empty() ? "" : ",") + std::string(n);
    };
    over("QR_GPU_MAX_K", r.policy.gpu_max_k);
    over("QR_GPU_MIN_BATCH_TIMES_K", r.policy.gpu_min_batch_times_k);
    over("QR_GPU_MIN_BATCH", r.policy.gpu_min_batch);
    over("QR_GPU_MIN_K", r.policy.gpu_min_k);
    over("QR_GPU_LARGE_MIN_K", r.policy.gpu_large_min_k);
    over("QR_GPU_LARGE_MAX_BATCH", r.policy.gpu_large_max_batch);
    over("QR_SHARE_MIN_BATCH", r.policy.share_min_batch);
    if (!env.empty()) r.source = "env:" + env;
    return r;
}

std::mutex g_policy_mutex;
ResolvedPolicy& state() {
    static ResolvedPolicy s = resolve();
    return s;
}

} // namespace

QrPolicy qr_policy() {
    std::lock_guard<std::mutex> lock(g_policy_mutex);
    return state().policy;
}
const char* qr_policy_source() {
    std::lock_guard<std::mutex> lock(g_policy_mutex);
    return state().source.c_str();
}
void set_qr_policy(const QrPolicy& p) {
    std::lock_guard<std::mutex> lock(g_policy_mutex);
    const unsigned cores = state().policy.gpu_cores, conc = state().policy.concurrent_matrices;
    state().policy = p;
    state().policy.gpu_cores = cores;             // informational, ignored when setting
    state().policy.concurrent_matrices = conc;
    state().source = "user";
}

QrBackend qr_gpu_backend(unsigned m, unsigned n, unsigned batch) {
    const QrPolicy p = qr_policy();
    const unsigned k = std::min(m, n);
    const unsigned crossover = batch < p.batch_threshold ? p.m_crossover_small_batch : p.m_crossover_large_batch;
    if (k >= crossover) return QrBackend::streaming_reduced;
    // the large clause on sqrt(M k), which grows with the batch: the grid-parallel QR takes a batch a
    // few matrices at a time, the block-per-matrix kernel a whole wave of matrices at once
    const unsigned long long L = p.gpu_large_min_k;
    if (L && (unsigned long long)m * k * 3 >= L * L * std::max(3u, batch) &&      // sqrt(M k) >= L sqrt(max(1, batch / 3))
        (p.gpu_large_max_batch == 0 || batch <= p.gpu_large_max_batch))
        return QrBackend::streaming_reduced;
    return QrBackend::unblocked;
}
QrBackend qr_backend(unsigned m, unsigned n, unsigned batch) { return qr_gpu_backend(m, n, batch); }
bool      qr_uses_gpu(unsigned, unsigned, unsigned) { return true; }
bool      qr_shares_batch(unsigned, unsigned, unsigned) { return false; }

// ---------------------------------------------------------------------------
// Kernel choice
// ---------------------------------------------------------------------------
namespace {

mlb::QrProblem problem(const Matrices& a, float* q, float* r, QrMode mode) {
    mlb::QrProblem p{};
    p.a = a.data; p.q = q; p.r = r;
    p.batch = a.batch; p.m = a.rows; p.n = a.cols;
    p.qc = core::qr_q_cols(mode, a.rows, a.cols);
    p.rr = core::qr_r_rows(mode, a.rows, a.cols);
    if (!p.qc) p.q = nullptr;
    return p;
}

// A forced kernel, for tuning: QR_KERNEL=small|mid|tsqr|blocked (ignored where it does not fit).
int forced_kernel() {
    const char* e = std::getenv("QR_KERNEL");
    if (!e) return -1;
    if (!std::strcmp(e, "small")) return (int)QrKernel::small;
    if (!std::strcmp(e, "mid")) return (int)QrKernel::mid;
    if (!std::strcmp(e, "tsqr")) return (int)QrKernel::tsqr;
    if (!std::strcmp(e, "blocked")) return (int)QrKernel::blocked;
    return -1;
}

QrKernel choose(mlb::DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t batch, QrMode mode) {
    const uint32_t qc = core::qr_q_cols(mode, m, n);
    const bool small = mlb::qr_small_fits(m, n, qc), mid = mlb::qr_mid_fits(ctx, m, n),
               tsqr = mlb::qr_tsqr_fits(ctx, m, n, qc);
    switch (forced_kernel()) {
        case (int)QrKernel::small:   if (small) return QrKernel::small; break;
        case (int)QrKernel::mid:     if (mid) return QrKernel::mid; break;
        case (int)QrKernel::tsqr:    if (tsqr) return QrKernel::tsqr; break;
        case (int)QrKernel::blocked: return QrKernel::blocked;
        default: break;
    }
    if (small) return QrKernel::small;
    const bool spread = qr_gpu_backend(m, n, batch) == QrBackend::streaming_reduced;
    // a lone tall thin matrix of 64 columns or more is faster through the blocked QR's cluster panels where
    // those hold its rows (8192 x 128: 0.37 ms against 1.43 ms; 4096 x 64: 0.19 against 0.22; 8192 x 64: 0.22
    // against 0.27), and so are up to four of 128 columns (two: 0.71 against 1.43; four: 1.38 against 1.44); two of
    // 64 columns (4096 x 64: 0.35 against 0.22) and any of 32 (16384 x 32: 0.21 against 0.15) go to the tree, as
    // every larger batch does (16 of 8192 x 128: 5.4 ms against 2.1 ms)
    const uint32_t few = n >= 128 ? 4u : n >= 64 ? 1u : 0u;
    const bool lone = batch <= few && mlb::panel_fast_fits(m, 1) && mlb::qr_blocked_fits(m, n);
    // the tree also takes the tall thin matrices a block could hold (512 to 1024 rows): its blocks of 256 rows
    // run the panels with a column per lane, which one block of more rows cannot (1024 x 64: 0.21 against 0.50 ms
    // at any batch up to 64; 512 x 32: 0.09 against 0.15)
    // (a lone matrix leaves the tree for the blocked QR only, never for one block)
    if (tsqr && !(lone && (spread || !mid))) return QrKernel::tsqr;
    if (mid && !spread) return QrKernel::mid;
    if (mid && !mlb::qr_blocked_fits(m, n)) return QrKernel::mid;
    return QrKernel::blocked;
}

// QR_WIDE=0: wide matrices through the general kernels, whole (for comparison and tests)
bool wide_by_leading_block() {
    const char* e = std::getenv("QR_WIDE");
    return !(e && e[0] == '0');
}

void run_on_device(mlb::DeviceContext& ctx, cudaStream_t stream, const Matrices& a, float* q, float* r, QrMode mode,
                   int forced /* -1: route */, bool may_split = true);

// A wide matrix by its leading M x M block and one product (qr_wide.cu; the reference's CPU path does the
// same, src/qr_cpu.mm:6-9,112-118): taken where takes_wide_split says it pays. Q (M x M in every mode of a wide
// matrix) goes to the caller's buffer, or to scratch when R alone was asked for.
// Measured on a B200 (ms, whole against split): one 128 x 1024 0.53 / 0.16, one 64 x 2048 0.43 / 0.075, eight 256 x 2048
// 2.70 / 0.60, 2048 of 48 x 100 0.47 / 0.44; R alone, which otherwise never forms Q: 128 x 1024 0.49 / 0.16, 256 of
// 64 x 256 0.10 / 0.10, 2048 of 48 x 100 0.36 / 0.44, so R alone splits from four times as wide as tall. Where the
// square block itself would go to the grid-parallel blocked QR the split loses (512 x 4096: 0.99 / 1.01; 2000 x 6000:
// 4.4 / 5.2: the blocked QR's own trailing updates run on the tensor cores, the product here on FP32 FMAs) and is not taken.
bool takes_wide_split(mlb::DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t batch, QrMode mode, int forced) {
    if (m >= n || n - m < 32 || !wide_by_leading_block()) return false;
    if (mode == QrMode::r && n < 4 * (uint64_t)m) return false;
    if (mlb::qr_small_fits(m, n, core::qr_q_cols(mode, m, n))) return false;
    if ((uint64_t)batch * m * m >= ((uint64_t)1 << 40)) return false;
    const QrKernel inner = forced >= 0 ? (QrKernel)forced : choose(ctx, m, m, batch, QrMode::reduced);
    return inner != QrKernel::blocked;
}

bool run_wide(mlb::DeviceContext& ctx, cudaStream_t stream, const Matrices& a, float* q, float* r, QrMode mode, int forced) {
    const uint32_t m = a.rows, n = a.cols;
    if (!takes_wide_split(ctx, m, n, a.batch, mode, forced)) return false;
    const bool q_scratch = q == nullptr;
    const size_t block = ((size_t)a.batch * m * m + 63) & ~(size_t)63;
    float* ws = static_cast<float*>(ctx.outer_workspace(stream, mlb::wide_scratch_floats(a.batch, m, q_scratch) * sizeof(float)));
    float* a1 = ws;
    float* r1 = ws + block;
    float* qs = q_scratch ? ws + 2 * block : q;
    unsigned* bad = reinterpret_cast<unsigned*>(ws + (q_scratch ? 3 : 2) * block);
    mlb::launch_wide_gather(stream, a.data, a.batch, m, n, a1, bad);
    // the square block's Q is M x M whether reduced or complete; R1 is M x M
    run_on_device(ctx, stream, {a1, a.batch, m, m}, qs, r1, QrMode::reduced, forced, false);
    mlb::launch_wide_finish(stream, qs, m, a.data, r1, r, a.batch, m, n);
    return true;
}

void run_on_device(mlb::DeviceContext& ctx, cudaStream_t stream, const Matrices& a, float* q, float* r, QrMode mode,
                   int forced /* -1: route */, bool may_split) {
    ctx.last_shape[0] = a.batch; ctx.last_shape[1] = a.rows; ctx.last_shape[2] = a.cols;
    if (may_split && run_wide(ctx, stream, a, q, r, mode, forced)) return;
    const mlb::QrProblem p = problem(a, q, r, mode);
    const QrKernel k = forced >= 0 ? (QrKernel)forced : choose(ctx, a.rows, a.cols, a.batch, mode);
    switch (k) {
        case QrKernel::small:   mlb::launch_qr_small(ctx, stream, p); break;
        case QrKernel::mid:     mlb::launch_qr_mid(ctx, stream, p); break;
        case QrKernel::tsqr:    mlb::launch_qr_tsqr(ctx, stream, p); break;
        case QrKernel::blocked: mlb::launch_qr_blocked(ctx, stream, p); break;
    }
}

} // namespace

void qr_enqueue(mlb::DeviceContext& ctx, cudaStream_t stream, const core::Matrices& a, float* q, float* r, core::QrMode mode) {
    // the library's own callers hold the outer workspace themselves, and hand over tall matrices only
    run_on_device(ctx, stream, a, q, r, mode, -1, false);
}

namespace {

// Host pointers: the batch in chunks through three sets of device buffers, the
// copy in of a later chunk and the copy out of an earlier one running beside the
// kernels of chunk i on the context's three streams. (With two sets the copy in of
// chunk i + 1 had to wait for the copy out of chunk i - 1: at two ranks a machine
// the pipeline then took 1.24 times what its copies alone take.)
void run_staged(mlb::DeviceContext& ctx, const Matrices& a, float* q, float* r, QrMode mode, int forced) {
    constexpr int kSets = mlb::DeviceContext::kStagingSets;
    const uint32_t m = a.rows, n = a.cols;
    const size_t qc = core::qr_q_cols(mode, m, n), rr = core::qr_r_rows(mode, m, n);
    const size_t fa = (size_t)m * n, fq = (size_t)m * qc, fr = rr * n;
    const size_t per = (fa + fq + fr) * sizeof(float);
    // chunks of about 64 MB of traffic, at least one matrix, at most the batch
    size_t chunk = std::max<size_t>(1, ((size_t)64 << 20) / std::max<size_t>(per, 1));
    chunk = std::min<size_t>(chunk, a.batch);
    const size_t align = 64;   // floats; keeps every buffer 256-byte aligned
    auto up = [&](size_t f) { return (f + align - 1) / align * align; };
    const size_t set_floats = up(chunk * fa) + up(chunk * fq) + up(chunk * fr);

    mlb::DeviceGuard guard(ctx.device);
    std::lock_guard<std::mutex> lock(ctx.mutex);
    // the staging buffers belong to the copy-in stream's workspace; the kernels'
    // own scratch to the compute stream's
    float* base = static_cast<float*>(ctx.workspace(ctx.copy_in, kSets * set_floats * sizeof(float)));
    float* da[kSets], *dq[kSets], *dr[kSets];
    for (int s = 0; s < kSets; ++s) {
        da[s] = base + s * set_floats;
        dq[s] = da[s] + up(chunk * fa);
        dr[s] = dq[s] + up(chunk * fq);
    }
    size_t done = 0;
    for (size_t i = 0; done < a.batch; ++i) {
        const int s = (int)(i % kSets);
        const uint32_t count = (uint32_t)std::min<size_t>(chunk, a.batch - done);
        // the set is free once its previous copy out has finished
        if (i >= (size_t)kSets) mlb::cuda_check(cudaStreamWaitEvent(ctx.copy_in, ctx.ev_out[s], 0), "cudaStreamWaitEvent");
        mlb::cuda_check(cudaMemcpyAsync(da[s], a.data + done * fa, count * fa * sizeof(float),
                                        cudaMemcpyHostToDevice, ctx.copy_in), "copy in");
        mlb::cuda_check(cudaEventRecord(ctx.ev_in[s], ctx.copy_in), "cudaEventRecord");
        mlb::cuda_check(cudaStreamWaitEvent(ctx.compute, ctx.ev_in[s], 0), "cudaStreamWaitEvent");
        if (i >= (size_t)kSets) mlb::cuda_check(cudaStreamWaitEvent(ctx.compute, ctx.ev_out[s], 0), "cudaStreamWaitEvent");
        run_on_device(ctx, ctx.compute, {da[s], count, m, n}, dq[s], dr[s], mode, forced);
        mlb::cuda_check(cudaEventRecord(ctx.ev_done[s], ctx.compute), "cudaEventRecord");
        mlb::cuda_check(cudaStreamWaitEvent(ctx.copy_out, ctx.ev_done[s], 0), "cudaStreamWaitEvent");
        if (fq)
            mlb::cuda_check(cudaMemcpyAsync(q + done * fq, dq[s], count * fq * sizeof(float),
                                            cudaMemcpyDeviceToHost, ctx.copy_out), "copy out");
        mlb::cuda_check(cudaMemcpyAsync(r + done * fr, dr[s], count * fr * sizeof(float),
                                        cudaMemcpyDeviceToHost, ctx.copy_out), "copy out");
        mlb::cuda_check(cudaEventRecord(ctx.ev_out[s], ctx.copy_out), "cudaEventRecord");
        done += count;
    }
    mlb::cuda_check(cudaStreamSynchronize(ctx.copy_out), "cudaStreamSynchronize");
    mlb::cuda_check(cudaStreamSynchronize(ctx.compute), "cudaStreamSynchronize");
    if (const unsigned word = ctx.take_status())      // the call is complete here: a kernel that gave up is an error now
        throw std::runtime_error("[qr] a kernel gave up on a bounded wait (status " + std::to_string(word) + ") on a batch of " +
                                 std::to_string(a.batch) + " matrices of " + std::to_string(m) + " x " + std::to_string(n) +
                                 "; their outputs are NaN");
}

void run(const Matrices& a, float* q, float* r, QrMode mode, int forced) {
    const uint32_t M = a.rows, N = a.cols, K = std::min(M, N);
    const size_t qc = core::qr_q_cols(mode, M, N), rr = core::qr_r_rows(mode, M, N);
    if (!qc) q = nullptr;
    if (cpu_only())
        throw std::runtime_error("[qr] this thread is set CPU-only, and this build has no CPU path");
    const bool has_q = q != nullptr && (size_t)a.batch * M * qc > 0;
    const bool has_r = (size_t)a.batch * rr * N > 0;
    const bool has_a = (size_t)a.batch * M * N > 0;
    // where the buffers live: all on one GPU, or all on the host
    int where = -2;
    auto place = [&](const void* p, bool used) {
        if (!used || !p) return;
        const int d = mlb::pointer_device(p);
        if (where == -2) where = d;
        else if (where != d)
            throw std::invalid_argument("[qr] a, q and r must all be host pointers or all device pointers on one GPU");
    };
    place(a.data, has_a);
    place(q, has_q);
    place(r, has_r);
    if (where == -2) return;   // nothing to read or write

    // Nothing to factor: the complete Q is the identity (reference: src/qr.mm:312-317)
    if (K == 0 || a.batch == 0) {
        if (mode == QrMode::complete && N == 0 && has_q) {
            if (where < 0) {
                std::fill(q, q + (size_t)a.batch * M * M, 0.0f);
                for (size_t i = 0; i < (size_t)a.batch * M; ++i) q[i * M + i % M] = 1.0f;
            } else {
                mlb::DeviceContext& ctx = mlb::context(where);
                mlb::DeviceGuard guard(where);
                mlb::launch_fill_identity(mlb::thread_stream(), q, a.batch, M, M);
            }
        }
        return;
    }
    if (where >= 0) {
        mlb::DeviceContext& ctx = mlb::context(where);
        mlb::DeviceGuard guard(where);
        std::lock_guard<std::mutex> lock(ctx.mutex);
        run_on_device(ctx, mlb::thread_stream(), a, q, r, mode, forced);
    } else {
        run_staged(mlb::context(mlb::thread_device()), a, q, r, mode, forced);
    }
}

} // namespace

namespace core {

QrKernel qr_kernel(uint32_t m, uint32_t n, uint32_t batch, QrMode mode) {
    mlb::DeviceContext& ctx = mlb::context(mlb::thread_device());
    // a wide matrix beyond the register kernel is factored by its leading square block (run_wide)
    if (takes_wide_split(ctx, m, n, batch, mode, -1)) return choose(ctx, m, m, batch, QrMode::reduced);
    return choose(ctx, m, n, batch, mode);
}
const char* qr_kernel_name(QrKernel k) {
    switch (k) {
        case QrKernel::small: return "small";
        case QrKernel::mid:   return "mid";
        case QrKernel::tsqr:  return "tsqr";
        default:              return "blocked";
    }
}

void qr(const Matrices& a, float* q, float* r, QrMode mode) { run(a, q, r, mode, -1); }
void qr(const Matrices& a, float* q, float* r) { run(a, q, r, QrMode::reduced, -1); }

namespace detail {

bool qr_householder_fits(uint32_t m, uint32_t n) {
    return m > 0 && n > 0 && mlb::qr_mid_fits(mlb::context(mlb::thread_device()), m, n);
}
bool qr_blocked_fits(uint32_t m, uint32_t n) { return mlb::qr_blocked_fits(m, n); }
bool qr_tsqr_fits(uint32_t m, uint32_t n, QrMode mode) {
    return mlb::qr_tsqr_fits(mlb::context(mlb::thread_device()), m, n, core::qr_q_cols(mode, m, n));
}

void qr_householder(const Matrices& a, float* q, float* r, QrMode mode) {
    if (std::min(a.rows, a.cols) == 0 || a.batch == 0) return run(a, q, r, mode, -1);
    const uint32_t qc = core::qr_q_cols(mode, a.rows, a.cols);
    if (mlb::qr_small_fits(a.rows, a.cols, qc)) return run(a, q, r, mode, (int)QrKernel::small);
    if (!qr_householder_fits(a.rows, a.cols))
        throw std::invalid_argument("[qr_householder] a matrix of " + std::to_string(a.rows) + " x " +
                                    std::to_string(a.cols) + " does not fit a thread block");
    run(a, q, r, mode, (int)QrKernel::mid);
}
void qr_unblocked(const Matrices& a, float* q, float* r, QrMode mode) {
    if (std::min(a.rows, a.cols) == 0 || a.batch == 0) return run(a, q, r, mode, -1);
    const uint32_t qc = core::qr_q_cols(mode, a.rows, a.cols);
    if (mlb::qr_small_fits(a.rows, a.cols, qc) || qr_householder_fits(a.rows, a.cols))
        return qr_householder(a, q, r, mode);
    qr_blocked(a, q, r, mode);
}
void qr_blocked(const Matrices& a, float* q, float* r, QrMode mode) {
    if (std::min(a.rows, a.cols) == 0 || a.batch == 0) return run(a, q, r, mode, -1);
    if (!mlb::qr_blocked_fits(a.rows, a.cols))
        throw std::invalid_argument("[qr_blocked] a matrix of " + std::to_string(a.rows) + " x " +
                                    std::to_string(a.cols) + " is beyond the blocked QR");
    run(a, q, r, mode, (int)QrKernel::blocked);
}
void qr_tsqr(const Matrices& a, float* q, float* r, QrMode mode) {
    if (std::min(a.rows, a.cols) == 0 || a.batch == 0) return run(a, q, r, mode, -1);
    if (!qr_tsqr_fits(a.rows, a.cols, mode))
        throw std::invalid_argument("[qr_tsqr] takes tall matrices of at most 64 columns, reduced or R alone");
    run(a, q, r, mode, (int)QrKernel::tsqr);
}
void qr_streaming_amx_reduced(const Matrices& a, float* q, float* r, QrMode mode) { qr_blocked(a, q, r, mode); }

} // namespace detail
} // namespace core
} // namespace metal_linalg
