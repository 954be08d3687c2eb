#pragma once
// The QR kernel families and their launchers. Every pointer is a device pointer
// on ctx.device; everything is enqueued on `stream` and nothing waits.
#include "runtime.h"

#include <cstdint>

namespace mlb {

enum QrModeInt { kReduced = 0, kROnly = 1, kComplete = 2 };

struct QrProblem {
    const float* a;      // [batch, m, n] row-major
    float*       q;      // [batch, m, qc] or null when qc == 0
    float*       r;      // [batch, rr, n]
    uint32_t     batch, m, n;
    uint32_t     qc;     // Q's columns: K, 0 (R alone) or m
    uint32_t     rr;     // R's rows: K or m
};

inline uint32_t qr_k(const QrProblem& p) { return p.m < p.n ? p.m : p.n; }

// A matrix in one warp's registers (or a part of a warp's): m, n, qc <= 32.
bool qr_small_fits(uint32_t m, uint32_t n, uint32_t qc);
void launch_qr_small(DeviceContext& ctx, cudaStream_t stream, const QrProblem& p);
// The same for square matrices of 8, 16 or 32 rows on 16-byte boundaries, streamed through shared
// memory by bulk asynchronous copies; false (nothing launched) for any other call.
bool launch_qr_small_stream(DeviceContext& ctx, cudaStream_t stream, const QrProblem& p);

// A matrix to a thread block: panels of 32 columns factored in shared memory,
// the trailing matrix streamed through a per-block scratch copy that stays in L2.
bool   qr_mid_fits(const DeviceContext& ctx, uint32_t m, uint32_t n);
void   launch_qr_mid(DeviceContext& ctx, cudaStream_t stream, const QrProblem& p);
// The same on `count` independent matrices read with a row stride and scaled on
// load or not; used by the TSQR tree for its row blocks. See qr_mid.cu.
struct MidOptions {
    uint32_t lda      = 0;      // row stride of a (0: n)
    uint64_t a_stride = 0;      // floats between matrices of a (0: m * lda)
    uint64_t q_stride = 0;      // floats between matrices of q (0: m * qc)
    uint64_t r_stride = 0;      // floats between matrices of r (0: rr * n)
    bool     scale    = true;   // scan and scale each matrix by a power of two; NaN-fill non-finite ones
    // two-level indexing: with inner_count > 0, matrix i starts at (i / inner_count) * *_outer +
    // (i % inner_count) * *_stride (row blocks of several tall matrices in one launch)
    uint32_t inner_count = 0;
    uint64_t a_outer = 0, q_outer = 0, r_outer = 0;
    float*   ws       = nullptr;   // scratch of at least qr_mid_workspace_floats(...) floats (null: the stream's workspace)
};
size_t qr_mid_workspace_floats(const DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t batch);
void launch_qr_mid(DeviceContext& ctx, cudaStream_t stream, const QrProblem& p, const MidOptions& o);

// The block-per-matrix kernel on scratch slots that are part of the library
// image instead of the workspace: allocates and frees nothing. Device pointers
// on `device`; throws std::invalid_argument beyond 1024 rows or when one matrix
// needs more scratch than qr_mid_static_capacity_bytes().
void   launch_qr_mid_static(int device, cudaStream_t stream, const QrProblem& p);
size_t qr_mid_static_capacity_bytes();

// A tall thin matrix as a tree of row blocks (qr_tsqr.cu; at most 64 columns: qr_tsqr_vt.cu).
bool qr_tsqr_fits(const DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t qc);
void launch_qr_tsqr(DeviceContext& ctx, cudaStream_t stream, const QrProblem& p);

// The tree on strided input with caller-provided scratch (the blocked QR's panels use it): thin QR of
// `batch` m x n matrices (n <= 128, m >= n) read with row stride lda and matrix stride a_outer; q
// [batch][m][n] contiguous or null (R alone); r n x n per matrix at stride r_outer.
size_t tsqr_workspace_floats(const DeviceContext& ctx, uint32_t m, uint32_t n, uint32_t batch, bool want_q);
void   tsqr_core(DeviceContext& ctx, cudaStream_t stream, const float* a, uint32_t lda, uint64_t a_outer, uint32_t m,
                 uint32_t n, uint32_t batch, float* q, float* r, uint64_t r_outer, float* ws);
// The tree with the row blocks kept as reflectors (qr_tsqr_vt.cu), which tsqr_core and tsqr_workspace_floats
// hand over to where tsqr_vt_takes() says so (at most 64 columns; QR_TSQR_VT=0 keeps the older scheme).
bool   tsqr_vt_takes(uint32_t m, uint32_t n);
size_t tsqr_vt_workspace_floats(uint32_t m, uint32_t n, uint32_t batch, bool want_q);
void   tsqr_vt_core(cudaStream_t stream, const float* a, uint32_t lda, uint64_t a_outer, uint32_t m, uint32_t n,
                    uint32_t batch, float* q, float* r, uint64_t r_outer, float* ws);
// out_block = q_block * factor for row blocks of n columns (see qr_tsqr.cu).
void   launch_tsqr_apply(DeviceContext& ctx, cudaStream_t stream, const float* q, uint64_t q_outer, uint64_t q_stride,
                         float* out, uint64_t out_outer, uint64_t out_stride, uint64_t out_ld, const float* up,
                         bool shared_up, uint32_t batch, uint32_t blocks, uint32_t rows, uint32_t last_rows, uint32_t n);

// A panel of the blocked QR (mp x jb, jb <= 32, mp <= 16384) to compact-WY form in three launches
// (qr_panel.cu): its R into the working copy's upper triangle, Y (unit lower trapezoidal) into y,
// T into t[32][32]. A wait inside it that ran out sets kStatusTensorWait in *bad (where given).
bool   panel_fast_fits(uint32_t mp, uint32_t jb);
size_t panel_fast_workspace_floats(uint32_t mp);
void   panel_factor_fast(cudaStream_t stream, float* panel, size_t ldw, uint32_t mp, uint32_t jb, float* y, size_t ldy,
                         float* t, float* ws, unsigned* bad = nullptr);

// The rank-128 products of the blocked QR on the tcgen05 tensor cores, 3xTF32 (tc_gemm.cu).
// `error` is set non-zero if a bounded wait inside the kernel ran out.
void launch_tc_ytc(cudaStream_t stream, const float* Y, size_t ldy, const float* C, size_t ldc, uint32_t mp, uint32_t kw,
                   uint32_t nc, float* zp, uint32_t ncp, uint32_t chunk_rows, unsigned* error);
void launch_tc_yz(cudaStream_t stream, const float* Y, size_t ldy, const float* Z, uint32_t ncp, float* C, size_t ldc,
                  uint32_t mp, uint32_t kw, uint32_t nc, unsigned* error);
// The same with Y and Z split into their tf32 parts once, ahead of the product, and fetched by bulk
// asynchronous copies (tc_gemm2.cu); ysp and zsp: scratch of tc_split_floats(mp) and tc_split_floats(nc) floats.
size_t tc_split_floats(uint32_t extent);
size_t tc_split_t_floats(uint32_t rows);
void launch_tc_ytc_split(cudaStream_t stream, const float* Y, size_t ldy, const float* C, size_t ldc, uint32_t mp,
                         uint32_t kw, uint32_t nc, float* zp, uint32_t ncp, uint32_t chunk_rows, uint32_t sub_rows, float* ytsp,
                         unsigned* error, float* ysp = nullptr);
void launch_tc_yz_split(cudaStream_t stream, const float* Y, size_t ldy, const float* Z, uint32_t ncp, float* C, size_t ldc,
                        uint32_t mp, uint32_t kw, uint32_t nc, float* ysp, float* zsp, unsigned* error);

// Blocked compact-WY QR over the whole grid, any shape.
bool qr_blocked_fits(uint32_t m, uint32_t n);
void launch_qr_blocked(DeviceContext& ctx, cudaStream_t stream, const QrProblem& p);

// A wide matrix (m < n) by its leading m x m block and one product (qr_wide.cu). `a1` [batch][m][m] takes the
// leading blocks (a matrix with a NaN or an infinity anywhere gets NaN into its block); after the QR of a1 into q
// (row stride ldq >= m) and r1 [batch][m][m], launch_wide_finish writes r [batch][m][n] = [r1 | q^T a(:, m:)].
// Scratch: wide_scratch_floats() floats hold a1, r1, `bad` (one word a matrix) and, when the caller asked for no Q, Q.
size_t wide_scratch_floats(uint32_t batch, uint32_t m, bool need_q_scratch);
void   launch_wide_gather(cudaStream_t stream, const float* a, uint32_t batch, uint32_t m, uint32_t n, float* a1, unsigned* bad);
void   launch_wide_finish(cudaStream_t stream, const float* q, uint32_t ldq, const float* a, const float* r1, float* r,
                          uint32_t batch, uint32_t m, uint32_t n);

// Small utilities shared by the launchers.
void launch_fill_identity(cudaStream_t stream, float* q, uint32_t batch, uint32_t m, uint32_t cols);
// out (row-major, contiguous float32) = the tensor `in` of element type `dtype` (the order of
// metal_linalg::Dtype: float32, float64, float16, bfloat16, int8, uint8, int16, int32, int64, bool), of
// `dims` <= kMaxConvertDims dimensions with the given shape and element strides.
constexpr int kMaxConvertDims = 8;
void launch_convert_to_f32(cudaStream_t stream, const void* in, int dtype, const uint32_t* shape, const int64_t* strides,
                           int dims, float* out);

// The small SVD behind a QR (svd_small.cu): one-sided Jacobi on the k x k factors r [batch, k, k],
// k <= 128. s [batch, k] descending; with ur non-null also the factors' left vectors ur [batch, k, k]
// (as columns) and the right vectors v [batch, k, k] (V^T, or V itself with v_as_columns);
// info [batch] or null. `effective_rows`: the rows of the matrix the factor came from (the rotation
// tolerance is sqrt(max(rows, 64)) eps).
bool svd_small_fits(uint32_t k);
void launch_svd_small(cudaStream_t stream, const float* r, uint32_t batch, uint32_t k, uint32_t effective_rows,
                      float* s, float* ur, float* v, bool v_as_columns, uint32_t* info);
// out = Q U_R per matrix (q [batch, l, k], ur [batch, k, k]); out [batch, l, k], or [batch, k, l] when transposed.
void launch_svd_left_vectors(cudaStream_t stream, const float* q, const float* ur, float* out, uint32_t batch, uint32_t l,
                             uint32_t k, bool transposed);
// out [batch, cols, rows] = in [batch, rows, cols] transposed.
void launch_transpose_batched(cudaStream_t stream, const float* in, float* out, uint32_t batch, uint32_t rows, uint32_t cols);

} // namespace mlb
