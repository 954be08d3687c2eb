#pragma once
// qr_accelerated, the C++ entry point (reference: include/metal_linalg/qr.h:22-24,
// src/mlx_api.cpp:135-149). The reference's takes and returns MLX arrays; MLX
// does not exist off Apple silicon, so this one takes and returns `Array`, a
// float32 tensor in CUDA device memory with a shape, which is all the entry
// point uses of an MLX array.
#include <metal_linalg/core.h>

#include <cstddef>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace metal_linalg {

    // A float32 tensor [..., M, N] in one GPU's memory, row-major and contiguous.
    class Array {
    public:
        Array() = default;
        // Uninitialised device memory of that shape on `device`.
        Array(std::vector<uint32_t> shape, int device);
        // A copy of host data on `device` / back on the host.
        static Array from_host(const float* data, std::vector<uint32_t> shape, int device = 0);
        std::vector<float> to_host() const;
        // Memory someone else owns (a framework's tensor); not freed.
        static Array view(float* device_data, std::vector<uint32_t> shape, int device);

        const std::vector<uint32_t>& shape() const { return shape_; }
        size_t size() const;
        float* data() const { return data_.get(); }
        int    device() const { return device_; }

    private:
        std::vector<uint32_t>  shape_;
        std::shared_ptr<float> data_;
        int                    device_ = 0;
    };

    // For a batch of matrices A [..., M, N], A = Q R with K = min(M, N):
    // Q [..., M, K] with orthonormal columns and R [..., K, N] upper
    // triangular, float32. `mode` as torch.linalg.qr's: "reduced" (the above),
    // "r" (R alone; the first array returned is empty and Q is never formed)
    // or "complete" (Q [..., M, M], R [..., M, N] with zero rows below K).
    // Anything else throws std::invalid_argument. The work is enqueued on the
    // calling thread's stream (set_stream); the arrays are safe to use on that
    // stream at once, and from the host after synchronize().
    std::pair<Array, Array> qr_accelerated(const Array& a, const std::string& mode);
    std::pair<Array, Array> qr_accelerated(const Array& a);   // "reduced"

} // namespace metal_linalg
