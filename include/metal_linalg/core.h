#pragma once
// The C++ buffer core of the B200 build: the QR on plain float buffers, its
// routing policy and the device queries. Names and meanings follow the
// reference's include/metal_linalg/core.h (QR part: lines 12-135 and 763-876)
// and include/metal_linalg/device.h; the C ABI (c_api.h) and qr_accelerated
// (qr.h) are built on this.
//
// Buffers are either all CUDA device pointers on one GPU (the work is enqueued
// on the calling thread's stream) or all host pointers (staged through the
// GPU; the call returns when the results are written). See c_api.h.
#include <cstddef>
#include <cstdint>

namespace metal_linalg {

    // -------------------------------------------------------------------------
    // Device (reference: include/metal_linalg/device.h)
    // -------------------------------------------------------------------------
    const char* device_name();       // "NVIDIA B200"; "" without a GPU
    unsigned    gpu_core_count();    // multiprocessors
    void        set_cpu_threads(unsigned n);
    unsigned    cpu_threads();
    void        set_cpu_only(bool on);   // thread-local; QR calls then fail (no CPU path here)
    bool        cpu_only();

    // The calling thread's CUDA stream for device-pointer calls (nullptr: the
    // default stream) and its GPU for host-pointer calls. No counterpart in
    // the reference.
    void  set_stream(void* cuda_stream);
    void* stream();
    void  set_device(int device);
    int   device();
    int   device_count();
    // Waits for the calling thread's stream, then throws std::runtime_error if a
    // kernel on any GPU this library has used gave up on one of its bounded
    // waits since the last check (the matrices concerned hold NaN). The
    // reference rethrows a failed command buffer with the shape
    // (src/qr_householder.mm:372-377, src/qr_blocked.mm:146-150); a CUDA launch
    // is asynchronous, so here the failure surfaces at this call, or at the end
    // of a host-pointer call, which waits anyway.
    void  synchronize();
    // Frees the scratch memory kept per (GPU, stream) between calls, after
    // waiting for each GPU it touches; returns the bytes freed. The next call
    // allocates again. For callers that create and destroy streams, or that
    // need the memory back after one large factorisation.
    size_t release_workspaces();
    // Testing aid (no GPU is made to wait or fail): the next `count` matrices
    // of the grid-parallel blocked QR are treated as if a tensor-core product
    // had given up on a wait: NaN outputs, and the error at synchronize().
    void  inject_wait_failures(int count);

    // -------------------------------------------------------------------------
    // Routing policy (reference: core.h:45-135, src/qr.mm:231-286)
    // -------------------------------------------------------------------------
    // Which kernel family takes a matrix, with k = min(M, N):
    //
    //   unblocked           a matrix to a warp ("small": M, N <= 32, in registers)
    //                       or to a thread block ("mid": the panel in shared
    //                       memory, the rest streamed through L2)
    //   streaming_reduced   a matrix spread over the grid: the blocked
    //                       compact-WY QR ("blocked") or, for a tall thin
    //                       matrix, the TSQR tree ("tsqr")
    //
    // streaming_reduced iff k >= m_crossover_* (by batch), or sqrt(M k) >=
    // gpu_large_min_k sqrt(max(1, batch / 3)) in a batch of at most
    // gpu_large_max_batch (the grid-parallel kernels factor a batch a few
    // matrices at a time, so the size from which they win grows with it), or the matrix is
    // beyond what a thread block holds. The reference's GPU-or-CPU fields
    // are kept in the struct, and read back as set, but decide nothing: there
    // is no CPU path.
    constexpr unsigned kQrNoLimit = 0xFFFFFFFFu;

    struct QrPolicy {
        unsigned m_crossover_small_batch = 768;   // batch <  batch_threshold
        unsigned m_crossover_large_batch = 768;   // batch >= batch_threshold
        unsigned batch_threshold         = 16;
        unsigned gpu_max_k               = kQrNoLimit;
        unsigned gpu_min_batch_times_k   = 0;
        unsigned gpu_min_batch           = 1;
        unsigned gpu_min_k               = 0;
        unsigned gpu_large_min_k         = 0;
        unsigned gpu_large_max_batch     = 0;
        unsigned share_min_batch         = 0;
        unsigned gpu_cores               = 0;
        unsigned concurrent_matrices     = 0;
    };

    QrPolicy    qr_policy();
    const char* qr_policy_source();
    void        set_qr_policy(const QrPolicy& p);

    enum class QrBackend { unblocked, streaming_reduced, cpu };   // cpu: never returned here
    QrBackend qr_backend(unsigned m, unsigned n, unsigned batch);
    QrBackend qr_gpu_backend(unsigned m, unsigned n, unsigned batch);
    bool      qr_uses_gpu(unsigned m, unsigned n, unsigned batch);      // always true
    bool      qr_shares_batch(unsigned m, unsigned n, unsigned batch);  // always false

    // The SVD's one backend here: the QR of this library, then one-sided Jacobi on the small factor
    // (reference: SvdBackend, core.h:550-574, of which qr_jacobi is one of ten). `unavailable`: a shape
    // beyond it (min(M, N) > 128), which core::svd refuses.
    enum class SvdBackend { qr_jacobi, unavailable };
    SvdBackend svd_backend(unsigned m, unsigned n, unsigned batch);
    SvdBackend svdvals_backend(unsigned m, unsigned n, unsigned batch);

    namespace core {

        // `batch` matrices of rows x cols (reference: core.h:776-781).
        struct Matrices {
            const float* data;
            uint32_t     batch;
            uint32_t     rows;
            uint32_t     cols;
        };

        // reference: core.h:783-797
        enum class QrMode {
            reduced,    // q [batch, M, K], r [batch, K, N]
            r,          // r [batch, K, N] alone; q unused (may be null), Q never formed
            complete,   // q [batch, M, M], r [batch, M, N] (zero rows below K)
        };
        inline uint32_t qr_q_cols(QrMode mode, uint32_t m, uint32_t n) {
            return mode == QrMode::r ? 0 : mode == QrMode::complete ? m : (m < n ? m : n);
        }
        inline uint32_t qr_r_rows(QrMode mode, uint32_t m, uint32_t n) {
            return mode == QrMode::complete ? m : (m < n ? m : n);
        }

        // A = Q R, routed by the policy (reference: core.h:799-803,
        // src/qr.mm:310-329). Throws std::invalid_argument for pointers in
        // different memories, std::runtime_error for a CUDA failure,
        // std::bad_alloc when device memory runs out.
        void qr(const Matrices& a, float* q, float* r, QrMode mode);
        void qr(const Matrices& a, float* q, float* r);   // QrMode::reduced

        // Thin SVD A = U diag(s) Vt, K = min(M, N): u [batch, M, K], s [batch, K] descending,
        // vt [batch, K, N]; u and vt both null for the singular values alone (then Q is never
        // formed: the QR runs in mode r). info [batch] or null: bits 0-15 the sweeps taken, bit 16
        // converged, bit 17 the matrix held a NaN or an infinity (its outputs are NaN), bit 18
        // rank-deficient (reference: core.h:811-814, c_api.h:96-102). The QR-preconditioned route
        // of the reference's svd_qr_jacobi (src/svd.mm:614-661), for min(M, N) <= 128; anything
        // larger throws std::invalid_argument. Pointers as for qr: all on the host or all on one GPU.
        void svd(const Matrices& a, float* u, float* s, float* vt, uint32_t* info = nullptr);
        bool svd_fits(uint32_t m, uint32_t n);

        // The kernel a call of that shape and mode runs.
        enum class QrKernel { small, mid, tsqr, blocked };
        QrKernel    qr_kernel(uint32_t m, uint32_t n, uint32_t batch, QrMode mode);
        const char* qr_kernel_name(QrKernel k);

        // Each kernel family on its own, whatever the policy says; same
        // contracts as above (reference: core.h:818-876). For tests and tuning.
        namespace detail {
            // small where it fits, else mid, else qr_blocked (reference: qr_unblocked)
            void qr_unblocked(const Matrices& a, float* q, float* r, QrMode mode);
            // the warp-per-matrix and block-per-matrix kernels (reference: qr_householder)
            void qr_householder(const Matrices& a, float* q, float* r, QrMode mode);
            bool qr_householder_fits(uint32_t m, uint32_t n);
            // the grid-parallel blocked compact-WY QR (reference: qr_blocked)
            void qr_blocked(const Matrices& a, float* q, float* r, QrMode mode);
            bool qr_blocked_fits(uint32_t m, uint32_t n);
            // tall thin matrices by a tree of row blocks (reference: the TSQR
            // panels inside qr_blocked, src/band_reduce.mm:196-251)
            void qr_tsqr(const Matrices& a, float* q, float* r, QrMode mode);
            bool qr_tsqr_fits(uint32_t m, uint32_t n, QrMode mode);
            // the reference's second grid-parallel entry point hands every
            // call to qr_blocked wherever that fits; so does this one
            void qr_streaming_amx_reduced(const Matrices& a, float* q, float* r, QrMode mode);
        }
    }
}
