// Small utility kernels shared by the launchers.
#include "kernels.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

namespace mlb {

namespace {
__global__ void fill_identity_kernel(float* q, size_t total, uint32_t m, uint32_t cols) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t in = i % ((size_t)m * cols);
        q[i] = (in / cols == in % cols) ? 1.0f : 0.0f;
    }
}

struct ConvertLayout {
    uint32_t shape[kMaxConvertDims];
    int64_t  strides[kMaxConvertDims];      // elements
    int      dims;
};

template <typename T>
__device__ __forceinline__ float as_float(T v) { return static_cast<float>(v); }
template <>
__device__ __forceinline__ float as_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float as_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// out (row-major, contiguous) = float32 of the strided tensor `in`
template <typename T>
__global__ void convert_kernel(const T* in, ConvertLayout lay, size_t total, float* out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t  rest = i;
        int64_t at = 0;
        for (int d = lay.dims - 1; d >= 0; --d) {
            at += (int64_t)(rest % lay.shape[d]) * lay.strides[d];
            rest /= lay.shape[d];
        }
        out[i] = as_float(in[at]);
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

void launch_convert_to_f32(cudaStream_t stream, const void* in, int dtype, const uint32_t* shape, const int64_t* strides,
                           int dims, float* out) {
    ConvertLayout lay{};
    lay.dims = dims;
    size_t total = 1;
    for (int d = 0; d < dims; ++d) {
        lay.shape[d] = shape[d];
        lay.strides[d] = strides[d];
        total *= shape[d];
    }
    if (!total) return;
    const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 16);
#define MLB_CONVERT(T) convert_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T*>(in), lay, total, out)
    switch (dtype) {       // the order of metal_linalg::Dtype
        case 0: MLB_CONVERT(float); break;
        case 1: MLB_CONVERT(double); break;
        case 2: MLB_CONVERT(__half); break;
        case 3: MLB_CONVERT(__nv_bfloat16); break;
        case 4: MLB_CONVERT(int8_t); break;
        case 5: MLB_CONVERT(uint8_t); break;
        case 6: MLB_CONVERT(int16_t); break;
        case 7: MLB_CONVERT(int32_t); break;
        case 8: MLB_CONVERT(int64_t); break;
        case 9: MLB_CONVERT(bool); break;
        default: throw std::invalid_argument("a tensor of this element type cannot be converted to float32");
    }
#undef MLB_CONVERT
    cuda_check(cudaGetLastError(), "convert launch");
}

} // namespace mlb
