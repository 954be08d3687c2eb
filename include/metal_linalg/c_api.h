/* The C ABI of the B200 build of metal-linalg's QR path: batched float32
 * Householder QR on NVIDIA B200 (sm_100a) behind the entry points a binding of
 * the reference library already resolves. Each declaration names the reference
 * declaration it stands in for (paths inside the reference project).
 *
 * Matrices are float32, row-major and contiguous: a batch is its matrices one
 * after another. The caller allocates every output. A NaN or an infinity in a
 * matrix gives NaN output for that matrix alone.
 *
 * Pointers. The reference takes host-addressable memory (unified memory on
 * Apple silicon). Here a, q and r are either all CUDA device pointers on one
 * GPU, or all host pointers:
 *   device pointers  the work is enqueued on the calling thread's stream (see
 *                    metal_linalg_set_stream; the default stream if none was
 *                    set) and the call returns without waiting, as any CUDA
 *                    library call does;
 *   host pointers    the matrices are staged to the calling thread's device
 *                    (metal_linalg_set_device; GPU 0 by default) in chunks,
 *                    factored there and copied back; the call returns when q
 *                    and r are written, as the reference's does.
 * There is no CPU path in this build: nothing is ever computed on the host.
 */
#ifndef METAL_LINALG_C_API_H
#define METAL_LINALG_C_API_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* include/metal_linalg/c_api.h:19-24 */
typedef enum metal_linalg_status {
    METAL_LINALG_OK               = 0,
    METAL_LINALG_INVALID_ARGUMENT = 1,  /* a null pointer, pointers in different memories, a bad mode */
    METAL_LINALG_RUNTIME_ERROR    = 2,  /* a CUDA failure, or a kernel that gave up on a bounded wait */
    METAL_LINALG_OUT_OF_MEMORY    = 3
} metal_linalg_status;

/* include/metal_linalg/c_api.h:26-28. The message of the most recent failure on
 * this thread, or "" if there has been none. Valid until the next failure on
 * this thread. */
const char* metal_linalg_last_error(void);

/* ---------------------------------------------------------------------------
 * QR
 * ------------------------------------------------------------------------- */

/* include/metal_linalg/c_api.h:34-37. A = Q R with K = min(rows, cols):
 * q [batch, rows, K] with orthonormal columns, r [batch, K, cols] upper
 * triangular (every entry below the diagonal exactly 0). */
metal_linalg_status metal_linalg_qr(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                    float* q, float* r);

/* include/metal_linalg/c_api.h:39-50. The same with a mode, as numpy.linalg.qr's
 * and torch.linalg.qr's: METAL_LINALG_QR_REDUCED as above; METAL_LINALG_QR_R,
 * R alone, r [batch, K, cols], q unused (NULL is fine) and Q never formed;
 * METAL_LINALG_QR_COMPLETE, q [batch, rows, rows] square, r [batch, rows, cols]
 * with zero rows below K. */
typedef enum metal_linalg_qr_mode {
    METAL_LINALG_QR_REDUCED  = 0,
    METAL_LINALG_QR_R        = 1,
    METAL_LINALG_QR_COMPLETE = 2,
} metal_linalg_qr_mode;
metal_linalg_status metal_linalg_qr_with_mode(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                              metal_linalg_qr_mode mode, float* q, float* r);

/* No counterpart in the reference. The QR for callers that must not allocate
 * device memory at call time, or trigger the device-wide stall of a cudaFree:
 * a request loop with a latency budget, or a process whose framework has
 * already taken the GPU's memory for its own pool so that a library's
 * cudaMalloc may fail. metal_linalg_qr_with_mode keeps the scratch memory of
 * its block-per-matrix kernel in a workspace that grows on demand; this entry
 * point runs the same kernel on a scratch array built into the library image
 * instead (metal_linalg_qr_no_alloc_scratch_bytes() bytes, 32 MiB, held by every
 * GPU that loads the library until the process exits). It calls no cudaMalloc,
 * no cudaFree and no allocating library routine.
 *
 * a, q and r as metal_linalg_qr_with_mode's, but CUDA device pointers on one
 * GPU only; the work is enqueued on the calling thread's stream. Limits: at most
 * 1024 rows, and one matrix's scratch, 4 * (rows * cols + 1024 * ceil(min(rows,
 * cols) / 32)) bytes, must fit the array; beyond either the call fails with
 * METAL_LINALG_INVALID_ARGUMENT and a message that says which. Batches of any
 * size are fine: fewer matrices are in flight at once when the array holds
 * fewer slots.
 *
 * The first call on a GPU looks up the array's device address (once per GPU);
 * make that call before any stream capture. Every call on a GPU shares the one
 * array: each slot is rewritten in full before it is read, so nothing from an
 * earlier call leaks into a later one, but two calls that overlap on the GPU
 * (different streams or threads) race on it. Serialise them. */
metal_linalg_status metal_linalg_qr_no_alloc(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                             metal_linalg_qr_mode mode, float* q, float* r);
uint64_t            metal_linalg_qr_no_alloc_scratch_bytes(void);

/* ---------------------------------------------------------------------------
 * SVD: the QR's first caller inside the library
 * ------------------------------------------------------------------------- */

/* include/metal_linalg/c_api.h:59-63. Thin SVD A = U diag(s) Vt with K =
 * min(rows, cols): u [batch, rows, K], s [batch, K] descending, vt [batch, K,
 * cols]; u and vt both NULL for the singular values alone; info [batch] or
 * NULL. Pointers as for metal_linalg_qr: all on the host or all on one GPU.
 * Of the reference's SVD backends this library holds the QR-preconditioned
 * one alone (A = Q R by the QR above, then one-sided Jacobi on R), for K <= 128:
 * a larger K fails with METAL_LINALG_INVALID_ARGUMENT. */
metal_linalg_status metal_linalg_svd(const float* a, uint32_t batch, uint32_t rows, uint32_t cols,
                                     float* u, float* s, float* vt, uint32_t* info);

/* include/metal_linalg/c_api.h:96-102. An `info` word: bits 0-15 the sweeps
 * taken, bit 16 converged, bit 17 the matrix held a NaN or an infinity (its
 * outputs are all NaN), bit 18 rank-deficient. */
#define METAL_LINALG_INFO_SWEEPS(info)         ((info) & 0xFFFFu)
#define METAL_LINALG_INFO_CONVERGED(info)      (((info) >> 16) & 1u)
#define METAL_LINALG_INFO_NONFINITE(info)      (((info) >> 17) & 1u)
#define METAL_LINALG_INFO_RANK_DEFICIENT(info) (((info) >> 18) & 1u)

/* include/metal_linalg/c_api.h:175-176. "qr_jacobi", or "unavailable" for a
 * shape metal_linalg_svd refuses. The strings are static. */
const char* metal_linalg_svd_backend(uint32_t rows, uint32_t cols, uint32_t batch);
const char* metal_linalg_svdvals_backend(uint32_t rows, uint32_t cols, uint32_t batch);   /* values alone */

/* ---------------------------------------------------------------------------
 * CUDA placement (no counterpart in the reference, whose memory is unified)
 * ------------------------------------------------------------------------- */

/* The CUDA stream (a cudaStream_t as a pointer; NULL for the default stream)
 * this thread's calls on device pointers are enqueued on. Thread-local, and one
 * stream for every GPU: a stream belongs to the GPU it was created on, so set it
 * again before passing pointers that live on another GPU (a stream of the wrong
 * GPU makes the launch fail with METAL_LINALG_RUNTIME_ERROR). */
void  metal_linalg_set_stream(void* cuda_stream);
void* metal_linalg_stream(void);

/* The GPU this thread's calls on host pointers run on (device pointers run on
 * the GPU that owns them). Thread-local; 0 by default. Returns
 * METAL_LINALG_INVALID_ARGUMENT for an ordinal the machine does not have. */
metal_linalg_status metal_linalg_set_device(int device);
int                 metal_linalg_device(void);
int                 metal_linalg_device_count(void);

/* Waits for everything this thread has enqueued on its stream. Then reports, as
 * METAL_LINALG_RUNTIME_ERROR with the GPU, the kind of wait and the last shape
 * enqueued in the message, a kernel that gave up on one of its bounded waits on
 * any GPU this library has used since the last report. Such a kernel has
 * written NaN to the outputs of the matrices concerned, which by itself cannot
 * be told from a NaN in the input: this call (or the status of a host-pointer
 * call, which checks before it returns) is where the two differ. The
 * reference reports a failed GPU command the same way, with the shape
 * (src/qr_householder.mm:372-377, src/qr_blocked.mm:146-150, src/c_api.cpp:17-35). */
metal_linalg_status metal_linalg_synchronize(void);

/* No counterpart in the reference (whose buffers are the caller's). The library
 * keeps scratch memory per (GPU, stream) between calls, as large as the largest
 * call so far needed (hundreds of MB after a large blocked QR). This frees all
 * of it, after waiting for every GPU concerned, and stores the bytes freed in
 * *bytes_freed (may be NULL). Later calls allocate again. Call it after
 * destroying streams the library has seen, or to hand the memory back. Not to
 * be called while another thread is inside a call of this library. */
metal_linalg_status metal_linalg_release_workspaces(uint64_t* bytes_freed);

/* Testing aid, no counterpart in the reference: the next `count` matrices that
 * the grid-parallel blocked QR factors are treated as if one of its tensor-core
 * products had given up on a wait at once (NaN outputs, the error at the next
 * metal_linalg_synchronize). Nothing on the GPU is made to wait, fault or fail. */
void metal_linalg_inject_wait_failures(int count);

/* ---------------------------------------------------------------------------
 * Device and routing
 * ------------------------------------------------------------------------- */

/* include/metal_linalg/c_api.h:136-138,147. The device's name, e.g. "NVIDIA
 * B200" ("" if there is no GPU), and its multiprocessor count (0 if none). */
const char* metal_linalg_device_name(void);
uint32_t    metal_linalg_gpu_core_count(void);

/* include/metal_linalg/c_api.h:140-146. The reference prints a notice when its
 * routing table was not measured on the machine it runs on. This build has one
 * table, measured on B200; the notice is "" on a B200 and says so elsewhere. */
void        metal_linalg_set_calibration_notices(int enabled);
const char* metal_linalg_calibration_message(const char* decomposition);

/* include/metal_linalg/c_api.h:149-153. Kept for bindings that resolve them:
 * the host threads the staging of host-pointer calls may use. */
void     metal_linalg_set_cpu_threads(uint32_t n);
uint32_t metal_linalg_cpu_threads(void);

/* include/metal_linalg/c_api.h:155-161. The reference routes the calling
 * thread's calls to its CPU paths while this is non-zero. This build has no CPU
 * path: while it is non-zero, QR calls on this thread fail with
 * METAL_LINALG_RUNTIME_ERROR rather than run on the GPU behind the caller's back. */
void metal_linalg_set_cpu_only(int on);
int  metal_linalg_cpu_only(void);

/* include/metal_linalg/c_api.h:163-172. The backend a call of that shape uses
 * under the policy in effect: "unblocked" (a matrix to a warp or a thread
 * block) or "streaming_reduced" (a matrix spread over the grid: the blocked
 * compact-WY QR and the TSQR tree). Never "cpu". The strings are static. */
const char* metal_linalg_qr_backend(uint32_t rows, uint32_t cols, uint32_t batch);

/* The kernel behind that backend, by name: "small" (a matrix in a warp's
 * registers), "mid" (a matrix to a thread block), "tsqr" (a tall thin matrix as
 * a tree of row blocks), "blocked" (compact-WY panels and rank-k updates over
 * the grid). No counterpart in the reference. The strings are static. */
const char* metal_linalg_qr_kernel(uint32_t rows, uint32_t cols, uint32_t batch, metal_linalg_qr_mode mode);

/* include/metal_linalg/c_api.h:186-201. The routing policy, field for field as
 * the reference's so that a binding's struct keeps its layout. */
#define METAL_LINALG_NO_LIMIT 0xFFFFFFFFu

typedef struct metal_linalg_qr_policy {
    uint32_t m_crossover_small_batch;   /* k = min(rows, cols) from which a matrix is spread over */
    uint32_t m_crossover_large_batch;   /* the grid, for batches below / from batch_threshold */
    uint32_t batch_threshold;
    uint32_t gpu_max_k;                 /* the reference's GPU-or-CPU rule: kept, and read back, */
    uint32_t gpu_min_batch_times_k;     /* but without effect (every call runs on the GPU) */
    uint32_t gpu_min_batch;
    uint32_t gpu_cores;                 /* informational: multiprocessors */
    uint32_t concurrent_matrices;       /* informational: thread blocks of the mid kernel resident at once */
    uint32_t gpu_large_min_k;           /* a matrix is spread over the grid also from sqrt(rows k) >= this x sqrt(max(1, batch / 3)) */
    uint32_t gpu_large_max_batch;       /* (0: never) in a batch of at most this (0: any) */
    uint32_t gpu_min_k;                 /* without effect */
    uint32_t share_min_batch;           /* without effect (no CPU to share a batch with) */
} metal_linalg_qr_policy;

/* include/metal_linalg/c_api.h:301,308,319 */
metal_linalg_qr_policy metal_linalg_qr_policy_get(void);
void                   metal_linalg_qr_policy_set(const metal_linalg_qr_policy* p);
/* "tuned:<device>", "env:<variables>", "user" or "default:untuned-device (<device>)". */
const char*            metal_linalg_qr_policy_source(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* METAL_LINALG_C_API_H */
