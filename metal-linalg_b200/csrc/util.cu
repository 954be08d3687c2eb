// Small utility kernels shared by the launchers.
#include "kernels.h"

namespace mlb {

namespace {
__global__ void fill_identity_kernel(float* q, size_t total, uint32_t m, uint32_t cols) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t in = i % ((size_t)m * cols);
        q[i] = (in / cols == in % cols) ? 1.0f : 0.0f;
    }
}
}

// q [batch, m, cols] = the leading columns of the identity, per matrix.
void launch_fill_identity(cudaStream_t stream, float* q, uint32_t batch, uint32_t m, uint32_t cols) {
    const size_t total = (size_t)batch * m * cols;
    if (!total) return;
    const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 16);
    fill_identity_kernel<<<blocks, 256, 0, stream>>>(q, total, m, cols);
    cuda_check(cudaGetLastError(), "fill_identity launch");
}

} // namespace mlb
