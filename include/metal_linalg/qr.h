#pragma once
// qr_accelerated, the C++ entry point (reference: include/metal_linalg/qr.h:22-24,
// src/mlx_api.cpp:37-71,122-149). The reference's takes and returns MLX arrays;
// MLX does not exist off Apple silicon, so this one takes and returns `Array`:
// a typed, possibly strided tensor in one GPU's memory, which is all the entry
// point uses of an MLX array (dtype, shape, strides, data).
#include <metal_linalg/core.h>

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace metal_linalg {

    // Element types an input may have. Every real type is converted to float32
    // before the factorisation (reference: src/mlx_api.cpp:50, astype float32);
    // complex64 is listed so that it can be refused, as the reference refuses it
    // (src/mlx_api.cpp:41-46: the real parts alone would be another matrix).
    enum class Dtype { float32, float64, float16, bfloat16, int8, uint8, int16, int32, int64, boolean, complex64 };
    size_t      dtype_size(Dtype t);
    const char* dtype_name(Dtype t);

    // A tensor [..., M, N] in one GPU's memory. Owning arrays are row-major and
    // contiguous; a view may carry any element strides (a transposed or sliced
    // tensor of a framework).
    class Array {
    public:
        Array() = default;
        // Uninitialised device memory of that shape on `device`.
        Array(std::vector<uint32_t> shape, int device, Dtype dtype = Dtype::float32);
        // A copy of contiguous host data on `device`.
        static Array from_host(const void* data, Dtype dtype, std::vector<uint32_t> shape, int device = 0);
        static Array from_host(const float* data, std::vector<uint32_t> shape, int device = 0) {
            return from_host(data, Dtype::float32, std::move(shape), device);
        }
        // Memory someone else owns (a framework's tensor); not freed. `strides` in elements, one per
        // dimension; empty for row-major contiguous.
        static Array view(void* device_data, Dtype dtype, std::vector<uint32_t> shape, int device,
                          std::vector<int64_t> strides = {});
        static Array view(float* device_data, std::vector<uint32_t> shape, int device) {
            return view(device_data, Dtype::float32, std::move(shape), device);
        }

        // The elements of a contiguous float32 array back on the host, after waiting for the calling
        // thread's stream. Throws std::invalid_argument for any other array.
        std::vector<float> to_host() const;

        const std::vector<uint32_t>& shape() const { return shape_; }
        const std::vector<int64_t>&  strides() const { return strides_; }   // elements
        Dtype  dtype() const { return dtype_; }
        size_t size() const;                  // elements
        bool   contiguous() const;            // row-major, no gaps
        void*  raw() const { return data_.get(); }
        float* data() const { return static_cast<float*>(data_.get()); }   // meaningful for float32
        int    device() const { return device_; }

        // This array as contiguous float32 on the same GPU: itself if it already is, else a converted
        // copy made on the calling thread's stream.
        Array as_float32() const;

    private:
        std::vector<uint32_t> shape_;
        std::vector<int64_t>  strides_;
        std::shared_ptr<void> data_;
        Dtype                 dtype_  = Dtype::float32;
        int                   device_ = 0;
    };

    // For a batch of matrices A [..., M, N], A = Q R with K = min(M, N):
    // Q [..., M, K] with orthonormal columns and R [..., K, N] upper
    // triangular, float32 whatever A's (real) type. `mode` as torch.linalg.qr's:
    // "reduced" (the above), "r" (R alone; the first array returned is empty and
    // Q is never formed) or "complete" (Q [..., M, M], R [..., M, N] with zero
    // rows below K). Throws std::invalid_argument for any other mode, for fewer
    // than two dimensions, for a complex input and for a batch of 2^32 matrices
    // or more. The work is enqueued on the calling thread's stream
    // (set_stream); the arrays are safe to use on that stream at once, and from
    // the host after synchronize().
    std::pair<Array, Array> qr_accelerated(const Array& a, const std::string& mode);
    std::pair<Array, Array> qr_accelerated(const Array& a);   // "reduced"

} // namespace metal_linalg
