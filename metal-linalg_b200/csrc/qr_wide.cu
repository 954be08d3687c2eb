// A wide matrix (M < N) by its leading block and one product: A = [A1 | A2] with A1 M x M is factored
// as A1 = Q R1 by whichever kernel takes an M x M matrix, and R2 = Q^T A2 is one matrix product, so
// that R = [R1 | R2]: the same reflectors and the same R as Householder QR of the whole matrix (the
// columns right of column M never influence a reflector). The reference does this on its CPU path
// (src/qr_cpu.mm:6-9,112-118), where LAPACK on the whole wide matrix ran 10-40 times slower; here it
// replaces, for one wide matrix or a few, a thread block walking all N / 32 column strips of its matrix
// one after another by a product that the whole grid shares.
//
// Three kernels: the leading blocks gathered into a contiguous batch (with the scan for NaN and Inf over
// the WHOLE matrix, since the inner factorisation sees A1 alone: a matrix with a non-finite entry anywhere
// gets NaN written into its A1, and with that NaN Q, R1 and R2); R1 copied into R's leading columns; and
// R2 = Q^T A2 by FP32 FMA tiles of 64 x 64.
#include "common.cuh"
#include "kernels.h"

namespace mlb {

namespace {

// a1 [batch][m][m] = a [batch][m][n](:, :m); grid (row groups, batch). A block whose rows hold a NaN or an
// infinity, in any column, marks the matrix in bad[b].
__global__ void __launch_bounds__(256) wide_gather_kernel(const float* __restrict__ a, float* a1, unsigned* bad, uint32_t m, uint32_t n,
                                                          uint32_t rows_per_block) {
    const uint32_t b = blockIdx.y;
    const uint32_t r_begin = blockIdx.x * rows_per_block, r_end = min(m, r_begin + rows_per_block);
    const float* src = a + (size_t)b * m * n;
    float* dst = a1 + (size_t)b * m * m;
    int seen = 0;
    for (uint32_t r = r_begin + (threadIdx.x >> 5); r < r_end; r += 8)
        for (uint32_t c = threadIdx.x & 31; c < n; c += 32) {
            const float v = src[(size_t)r * n + c];
            seen |= nonfinite(v);
            if (c < m) dst[(size_t)r * m + c] = v;
        }
    if (__any_sync(0xffffffffu, seen) && (threadIdx.x & 31) == 0) atomicOr(&bad[b], 1u);
}

// the first entry of a marked matrix's leading block becomes NaN (the inner factorisation then gives NaN Q and R1)
__global__ void wide_poison_kernel(float* a1, const unsigned* bad, uint32_t batch, uint32_t m) {
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch && bad[b]) a1[(size_t)b * m * m] = qnan();
}

// r [batch][rr][n](:, :m) = r1 [batch][rr][m]
__global__ void __launch_bounds__(256) wide_r1_kernel(const float* __restrict__ r1, float* r, uint32_t rr, uint32_t m, uint32_t n) {
    const uint32_t b = blockIdx.y;
    const size_t total = (size_t)rr * m;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        const size_t row = i / m, c = i % m;
        r[((size_t)b * rr + row) * n + c] = r1[(size_t)b * total + i];
    }
}

// r [b][i][m + j] = sum_k q [b][k][i] a [b][k][m + j]: i < m, j < n - m, k < m. q has row stride ldq (its
// first m columns are used). Grid (column tiles, row tiles, batch), tiles of 64 x 64, 16 k's a step, a thread 4 x 4.
__global__ void __launch_bounds__(256) wide_r2_kernel(const float* __restrict__ q, uint32_t ldq, const float* __restrict__ a,
                                                      float* r, uint32_t m, uint32_t n) {
    __shared__ __align__(16) float Qs[16][64];      // [k][i]
    __shared__ __align__(16) float As[16][64];      // [k][j]
    const uint32_t b = blockIdx.z, i0 = blockIdx.y * 64, j0 = blockIdx.x * 64, w = n - m;
    const float* qb = q + (size_t)b * m * ldq;
    const float* ab = a + (size_t)b * m * n + m;
    float* rb = r + (size_t)b * m * n + m;
    const int ti = threadIdx.x >> 4, tj = threadIdx.x & 15;
    float acc[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) acc[x][y] = 0.0f;
    for (uint32_t k0 = 0; k0 < m; k0 += 16) {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + 256 * e, k = idx >> 6, c = idx & 63;
            Qs[k][c] = (k0 + k < m && i0 + c < m) ? qb[(size_t)(k0 + k) * ldq + i0 + c] : 0.0f;
            As[k][c] = (k0 + k < m && j0 + c < w) ? ab[(size_t)(k0 + k) * n + j0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float4 qv = *reinterpret_cast<const float4*>(&Qs[k][4 * ti]);
            const float4 av = *reinterpret_cast<const float4*>(&As[k][4 * tj]);
            const float qe[4] = {qv.x, qv.y, qv.z, qv.w}, ae[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(qe[x], ae[y], acc[x][y]);
        }
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const uint32_t i = i0 + 4 * ti + x, j = j0 + 4 * tj + y;
            if (i < m && j < w) rb[(size_t)i * n + j] = acc[x][y];
        }
}

} // namespace

size_t wide_scratch_floats(uint32_t batch, uint32_t m, bool need_q_scratch) {
    const size_t block = (size_t)batch * m * m;
    auto up64 = [](size_t f) { return (f + 63) & ~(size_t)63; };
    return up64(block) * (need_q_scratch ? 3 : 2) + up64(batch);
}

void launch_wide_gather(cudaStream_t stream, const float* a, uint32_t batch, uint32_t m, uint32_t n, float* a1, unsigned* bad) {
    cuda_check(cudaMemsetAsync(bad, 0, (size_t)batch * sizeof(unsigned), stream), "cudaMemsetAsync");
    // enough blocks a matrix to fill the GPU for a lone matrix, whole rows a block
    uint32_t rows_per_block = 8;
    while ((uint64_t)batch * ((m + rows_per_block - 1) / rows_per_block) > 148u * 16 && rows_per_block < m) rows_per_block *= 2;
    for (uint32_t b0 = 0; b0 < batch; b0 += 65535) {
        const uint32_t nb = batch - b0 < 65535 ? batch - b0 : 65535;
        wide_gather_kernel<<<dim3((m + rows_per_block - 1) / rows_per_block, nb), 256, 0, stream>>>(
            a + (size_t)b0 * m * n, a1 + (size_t)b0 * m * m, bad + b0, m, n, rows_per_block);
    }
    wide_poison_kernel<<<(batch + 255) / 256, 256, 0, stream>>>(a1, bad, batch, m);
    cuda_check(cudaGetLastError(), "wide gather launch");
}

void launch_wide_finish(cudaStream_t stream, const float* q, uint32_t ldq, const float* a, const float* r1, float* r,
                        uint32_t batch, uint32_t m, uint32_t n) {
    for (uint32_t b0 = 0; b0 < batch; b0 += 65535) {
        const uint32_t nb = batch - b0 < 65535 ? batch - b0 : 65535;
        const unsigned copy_blocks = (unsigned)std::min<size_t>(((size_t)m * m + 255) / 256, 64);
        wide_r1_kernel<<<dim3(copy_blocks, nb), 256, 0, stream>>>(r1 + (size_t)b0 * m * m, r + (size_t)b0 * m * n, m, m, n);
        wide_r2_kernel<<<dim3((n - m + 63) / 64, (m + 63) / 64, nb), 256, 0, stream>>>(
            q + (size_t)b0 * m * ldq, ldq, a + (size_t)b0 * m * n, r + (size_t)b0 * m * n, m, n);
    }
    cuda_check(cudaGetLastError(), "wide finish launch");
}

} // namespace mlb
