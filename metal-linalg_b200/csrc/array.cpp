// Array and qr_accelerated (include/metal_linalg/qr.h): the C++ entry point
// (reference: src/mlx_api.cpp:37-71,122-149).
#include <metal_linalg/qr.h>

#include "runtime.h"

#include <stdexcept>

namespace metal_linalg {

size_t Array::size() const {
    if (shape_.empty()) return 0;
    size_t n = 1;
    for (uint32_t d : shape_) n *= d;
    return n;
}

Array::Array(std::vector<uint32_t> shape, int device) : shape_(std::move(shape)), device_(device) {
    const size_t n = size();
    if (!n) return;
    mlb::DeviceGuard guard(device);
    float* p = nullptr;
    mlb::cuda_check(cudaMalloc(&p, n * sizeof(float)), "cudaMalloc");
    data_ = std::shared_ptr<float>(p, [device](float* d) {
        int before = 0;
        cudaGetDevice(&before);
        cudaSetDevice(device);
        cudaFree(d);
        cudaSetDevice(before);
    });
}

Array Array::from_host(const float* data, std::vector<uint32_t> shape, int device) {
    Array a(std::move(shape), device);
    if (a.size()) {
        mlb::DeviceGuard guard(device);
        mlb::cuda_check(cudaMemcpy(a.data(), data, a.size() * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy");
    }
    return a;
}

std::vector<float> Array::to_host() const {
    std::vector<float> out(size());
    if (!out.empty()) {
        mlb::DeviceGuard guard(device_);
        mlb::cuda_check(cudaStreamSynchronize(mlb::thread_stream()), "cudaStreamSynchronize");
        mlb::cuda_check(cudaMemcpy(out.data(), data(), out.size() * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy");
    }
    return out;
}

Array Array::view(float* device_data, std::vector<uint32_t> shape, int device) {
    Array a;
    a.shape_ = std::move(shape);
    a.device_ = device;
    a.data_ = std::shared_ptr<float>(device_data, [](float*) {});
    return a;
}

std::pair<Array, Array> qr_accelerated(const Array& a, const std::string& mode) {
    core::QrMode m;
    if (mode == "reduced") m = core::QrMode::reduced;
    else if (mode == "r") m = core::QrMode::r;
    else if (mode == "complete") m = core::QrMode::complete;
    else throw std::invalid_argument("[qr_accelerated] mode must be \"reduced\", \"r\" or \"complete\", got \"" + mode + "\"");
    const auto& shape = a.shape();
    if (shape.size() < 2) throw std::invalid_argument("[qr_accelerated] expected a tensor of shape [..., M, N]");
    const uint32_t M = shape[shape.size() - 2], N = shape[shape.size() - 1];
    uint64_t batch = 1;
    for (size_t i = 0; i + 2 < shape.size(); ++i) batch *= shape[i];
    if (batch > 0xFFFFFFFFull) throw std::invalid_argument("[qr_accelerated] the batch must be below 2^32");
    std::vector<uint32_t> qs(shape.begin(), shape.end() - 2), rs = qs;
    const uint32_t qc = core::qr_q_cols(m, M, N), rr = core::qr_r_rows(m, M, N);
    if (qc) { qs.push_back(M); qs.push_back(qc); } else qs = {0};
    rs.push_back(rr); rs.push_back(N);
    Array q(qs, a.device()), r(rs, a.device());
    core::qr({a.data(), (uint32_t)batch, M, N}, q.data(), r.data(), m);
    return {q, r};
}

std::pair<Array, Array> qr_accelerated(const Array& a) { return qr_accelerated(a, "reduced"); }

} // namespace metal_linalg
