// core::svd by the QR-preconditioned route: A = Q R, R = U_R S V^T, A = (Q U_R) S V^T
// (reference: svd_qr_jacobi, src/svd.mm:614-661; the wide case by the transpose, :621-635). The QR
// is this library's own (mode r when the singular values alone are asked for, so Q is never
// formed); the small SVD is the one-sided Jacobi of svd_small.cu, which holds min(M, N) <= 128 (a warp's
// registers up to 32, a thread block's shared memory beyond).
// The reference's other SVD backends (block Jacobi, bidiagonalization, band reduction, LAPACK) are
// not built: a larger min(M, N) is refused with std::invalid_argument.
#include <metal_linalg/core.h>

#include "kernels.h"
#include "qr_enqueue.h"
#include "runtime.h"

#include <algorithm>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace metal_linalg {
namespace {

using core::Matrices;

size_t up64(size_t floats) { return (floats + 63) / 64 * 64; }   // keeps every slice 256-byte aligned

// Everything on ctx.device, enqueued on `stream`; the context's lock is held.
void svd_on_device(mlb::DeviceContext& ctx, cudaStream_t stream, const Matrices& a, float* u, float* s, float* vt,
                   uint32_t* info) {
    const uint32_t M = a.rows, N = a.cols, batch = a.batch;
    const bool wide = M < N, vectors = u != nullptr;
    const uint32_t l = wide ? N : M, k = wide ? M : N;
    const size_t f_at = wide ? up64((size_t)batch * l * k) : 0, f_r = up64((size_t)batch * k * k),
                 f_q = vectors ? up64((size_t)batch * l * k) : 0, f_ur = vectors ? f_r : 0;
    float* ws = static_cast<float*>(ctx.outer_workspace(stream, (f_at + f_r + f_q + f_ur) * sizeof(float)));
    float *at = ws, *r = at + f_at, *q = r + f_r, *ur = q + f_q;
    const float* tall = a.data;
    if (wide) {
        mlb::launch_transpose_batched(stream, a.data, at, batch, M, N);
        tall = at;
    }
    qr_enqueue(ctx, stream, {tall, batch, l, k}, vectors ? q : nullptr, r, vectors ? core::QrMode::reduced : core::QrMode::r);
    if (!vectors) {
        mlb::launch_svd_small(stream, r, batch, k, l, s, nullptr, nullptr, false, info);
        return;
    }
    // tall: vt = V^T; wide: A = V' S U'^T, so u takes V' itself and vt the transpose of Q U_R
    mlb::launch_svd_small(stream, r, batch, k, l, s, ur, wide ? u : vt, wide, info);
    mlb::launch_svd_left_vectors(stream, q, ur, wide ? vt : u, batch, l, k, wide);
}

} // namespace

namespace core {

bool svd_fits(uint32_t m, uint32_t n) { return std::min(m, n) == 0 || mlb::svd_small_fits(std::min(m, n)); }

void svd(const Matrices& a, float* u, float* s, float* vt, uint32_t* info) {
    const uint32_t M = a.rows, N = a.cols, K = std::min(M, N), batch = a.batch;
    if ((u == nullptr) != (vt == nullptr))
        throw std::invalid_argument("[svd] u and vt must both be given or both be null");
    if (cpu_only()) throw std::runtime_error("[svd] this thread is set CPU-only, and this build has no CPU path");
    if (batch == 0) return;
    const bool vectors = u != nullptr;
    // where the buffers live: all on one GPU, or all on the host
    int where = -2;
    auto place = [&](const void* p, bool used) {
        if (!used || !p) return;
        const int d = mlb::pointer_device(p);
        if (where == -2) where = d;
        else if (where != d)
            throw std::invalid_argument("[svd] a, u, s, vt and info must all be host pointers or all device pointers on one GPU");
    };
    place(a.data, (size_t)batch * M * N > 0);
    place(u, vectors && (size_t)batch * M * K > 0);
    place(s, (size_t)batch * K > 0);
    place(vt, vectors && (size_t)batch * K * N > 0);
    place(info, info != nullptr);
    if (where == -2) return;
    if (K == 0) {     // nothing to decompose: every matrix converged in no sweeps
        if (info) {
            if (where < 0) std::fill(info, info + batch, 1u << 16);
            else {
                mlb::DeviceGuard guard(where);
                std::vector<uint32_t> ok(batch, 1u << 16);
                mlb::cuda_check(cudaMemcpyAsync(info, ok.data(), batch * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                                mlb::thread_stream()), "copy");
                mlb::cuda_check(cudaStreamSynchronize(mlb::thread_stream()), "cudaStreamSynchronize");
            }
        }
        return;
    }
    if (!mlb::svd_small_fits(K))
        throw std::invalid_argument("[svd] min(M, N) = " + std::to_string(K) +
                                    ": this build holds the QR-preconditioned Jacobi route alone, min(M, N) <= 128");
    if (where >= 0) {
        mlb::DeviceContext& ctx = mlb::context(where);
        mlb::DeviceGuard guard(where);
        std::lock_guard<std::mutex> lock(ctx.mutex);
        svd_on_device(ctx, mlb::thread_stream(), a, u, s, vt, info);
        return;
    }
    // Host pointers: the batch in chunks of about 64 MB through device buffers, one chunk at a time.
    mlb::DeviceContext& ctx = mlb::context(mlb::thread_device());
    mlb::DeviceGuard guard(ctx.device);
    std::lock_guard<std::mutex> lock(ctx.mutex);
    const size_t fa = (size_t)M * N, fu = vectors ? (size_t)M * K : 0, fv = vectors ? (size_t)K * N : 0;
    const size_t per = (fa + fu + fv + K + 1) * sizeof(float);
    const size_t chunk = std::min<size_t>(batch, std::max<size_t>(1, ((size_t)64 << 20) / per));
    float* base = static_cast<float*>(ctx.workspace(ctx.copy_in, (up64(chunk * fa) + up64(chunk * fu) + up64(chunk * fv) +
                                                                   up64(chunk * K) + up64(chunk)) * sizeof(float)));
    float *da = base, *du = da + up64(chunk * fa), *dv = du + up64(chunk * fu), *ds = dv + up64(chunk * fv);
    uint32_t* di = reinterpret_cast<uint32_t*>(ds + up64(chunk * K));
    cudaStream_t st = ctx.compute;
    for (size_t done = 0; done < batch; done += chunk) {
        const uint32_t count = (uint32_t)std::min<size_t>(chunk, batch - done);
        mlb::cuda_check(cudaMemcpyAsync(da, a.data + done * fa, count * fa * sizeof(float), cudaMemcpyHostToDevice, st), "copy in");
        svd_on_device(ctx, st, {da, count, M, N}, vectors ? du : nullptr, ds, vectors ? dv : nullptr, di);
        mlb::cuda_check(cudaMemcpyAsync(s + done * K, ds, (size_t)count * K * sizeof(float), cudaMemcpyDeviceToHost, st), "copy out");
        if (vectors) {
            mlb::cuda_check(cudaMemcpyAsync(u + done * fu, du, count * fu * sizeof(float), cudaMemcpyDeviceToHost, st), "copy out");
            mlb::cuda_check(cudaMemcpyAsync(vt + done * fv, dv, count * fv * sizeof(float), cudaMemcpyDeviceToHost, st), "copy out");
        }
        if (info)
            mlb::cuda_check(cudaMemcpyAsync(info + done, di, count * sizeof(uint32_t), cudaMemcpyDeviceToHost, st), "copy out");
        mlb::cuda_check(cudaStreamSynchronize(st), "cudaStreamSynchronize");
    }
}

} // namespace core

SvdBackend svd_backend(unsigned m, unsigned n, unsigned) {
    return mlb::svd_small_fits(std::min(m, n)) ? SvdBackend::qr_jacobi : SvdBackend::unavailable;
}
SvdBackend svdvals_backend(unsigned m, unsigned n, unsigned batch) { return svd_backend(m, n, batch); }

} // namespace metal_linalg
