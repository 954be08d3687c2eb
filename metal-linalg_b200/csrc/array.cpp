// Array and qr_accelerated (include/metal_linalg/qr.h): the C++ entry point. What the reference's
// does with an MLX array (src/mlx_api.cpp:37-71: refuse fewer than two dimensions and complex
// input, convert to float32, make row-contiguous, batch = the product of the leading dimensions,
// below 2^32; :122-149: parse the mode, allocate Q and R, call the core) is done here with `Array`.
#include <metal_linalg/qr.h>

#include "kernels.h"
#include "runtime.h"

#include <stdexcept>

namespace metal_linalg {

size_t dtype_size(Dtype t) {
    switch (t) {
        case Dtype::float64: case Dtype::int64: case Dtype::complex64: return 8;
        case Dtype::float32: case Dtype::int32: return 4;
        case Dtype::float16: case Dtype::bfloat16: case Dtype::int16: return 2;
        default: return 1;
    }
}
const char* dtype_name(Dtype t) {
    switch (t) {
        case Dtype::float32: return "float32";
        case Dtype::float64: return "float64";
        case Dtype::float16: return "float16";
        case Dtype::bfloat16: return "bfloat16";
        case Dtype::int8: return "int8";
        case Dtype::uint8: return "uint8";
        case Dtype::int16: return "int16";
        case Dtype::int32: return "int32";
        case Dtype::int64: return "int64";
        case Dtype::boolean: return "bool";
        default: return "complex64";
    }
}

size_t Array::size() const {
    if (shape_.empty()) return 0;
    size_t n = 1;
    for (uint32_t d : shape_) n *= d;
    return n;
}

bool Array::contiguous() const {
    if (strides_.empty()) return true;
    int64_t expect = 1;
    for (size_t i = shape_.size(); i-- > 0;) {
        if (shape_[i] != 1 && strides_[i] != expect) return false;
        expect *= shape_[i];
    }
    return true;
}

Array::Array(std::vector<uint32_t> shape, int device, Dtype dtype) : shape_(std::move(shape)), dtype_(dtype), device_(device) {
    const size_t n = size();
    if (!n) return;
    mlb::DeviceGuard guard(device);
    void* p = nullptr;
    mlb::cuda_check(cudaMalloc(&p, n * dtype_size(dtype)), "cudaMalloc");
    data_ = std::shared_ptr<void>(p, [device](void* d) {
        int before = 0;
        cudaGetDevice(&before);
        cudaSetDevice(device);
        cudaFree(d);
        cudaSetDevice(before);
    });
}

Array Array::from_host(const void* data, Dtype dtype, std::vector<uint32_t> shape, int device) {
    Array a(std::move(shape), device, dtype);
    if (a.size()) {
        mlb::DeviceGuard guard(device);
        mlb::cuda_check(cudaMemcpy(a.raw(), data, a.size() * dtype_size(dtype), cudaMemcpyHostToDevice), "cudaMemcpy");
    }
    return a;
}

std::vector<float> Array::to_host() const {
    if (dtype_ != Dtype::float32 || !contiguous())
        throw std::invalid_argument("[Array::to_host] takes a contiguous float32 array");
    std::vector<float> out(size());
    if (!out.empty()) {
        mlb::DeviceGuard guard(device_);
        mlb::cuda_check(cudaStreamSynchronize(mlb::thread_stream()), "cudaStreamSynchronize");
        mlb::cuda_check(cudaMemcpy(out.data(), data(), out.size() * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy");
    }
    return out;
}

Array Array::view(void* device_data, Dtype dtype, std::vector<uint32_t> shape, int device, std::vector<int64_t> strides) {
    if (!strides.empty() && strides.size() != shape.size())
        throw std::invalid_argument("[Array::view] one stride per dimension, or none");
    Array a;
    a.shape_ = std::move(shape);
    a.strides_ = std::move(strides);
    a.dtype_ = dtype;
    a.device_ = device;
    a.data_ = std::shared_ptr<void>(device_data, [](void*) {});
    return a;
}

Array Array::as_float32() const {
    if (dtype_ == Dtype::complex64)
        throw std::invalid_argument("complex input is not supported: the decompositions are real (float32)");
    if (dtype_ == Dtype::float32 && contiguous()) return *this;
    if (shape_.size() > (size_t)mlb::kMaxConvertDims)
        throw std::invalid_argument("at most " + std::to_string(mlb::kMaxConvertDims) + " dimensions can be converted");
    Array out(shape_, device_, Dtype::float32);
    if (!out.size()) return out;
    std::vector<int64_t> strides = strides_;
    if (strides.empty()) {      // row-major
        strides.assign(shape_.size(), 1);
        for (size_t i = shape_.size() - 1; i-- > 0;) strides[i] = strides[i + 1] * shape_[i + 1];
    }
    mlb::DeviceGuard guard(device_);
    mlb::launch_convert_to_f32(mlb::thread_stream(), raw(), (int)dtype_, shape_.data(), strides.data(), (int)shape_.size(),
                               out.data());
    return out;
}

std::pair<Array, Array> qr_accelerated(const Array& a, const std::string& mode) {
    core::QrMode m;
    if (mode == "reduced") m = core::QrMode::reduced;
    else if (mode == "r") m = core::QrMode::r;
    else if (mode == "complete") m = core::QrMode::complete;
    else throw std::invalid_argument("[qr_accelerated] mode must be \"reduced\", \"r\" or \"complete\", got \"" + mode + "\"");
    const auto& shape = a.shape();
    if (shape.size() < 2) throw std::invalid_argument("[qr_accelerated] expected a tensor of shape [..., M, N]");
    if (a.dtype() == Dtype::complex64)
        throw std::invalid_argument("[qr_accelerated] complex input is not supported: the decompositions are real (float32)");
    const uint32_t M = shape[shape.size() - 2], N = shape[shape.size() - 1];
    uint64_t batch = 1;
    for (size_t i = 0; i + 2 < shape.size(); ++i) batch *= shape[i];
    if (batch > 0xFFFFFFFFull) throw std::invalid_argument("[qr_accelerated] the batch must be below 2^32");
    const Array x = a.as_float32();
    std::vector<uint32_t> qs(shape.begin(), shape.end() - 2), rs = qs;
    const uint32_t qc = core::qr_q_cols(m, M, N), rr = core::qr_r_rows(m, M, N);
    if (qc) { qs.push_back(M); qs.push_back(qc); } else qs = {0};
    rs.push_back(rr); rs.push_back(N);
    Array q(qs, a.device()), r(rs, a.device());
    core::qr({x.data(), (uint32_t)batch, M, N}, q.data(), r.data(), m);
    // the converted copy, if one was made, is freed when x goes out of scope: cudaFree waits for the
    // work that reads it
    return {q, r};
}

std::pair<Array, Array> qr_accelerated(const Array& a) { return qr_accelerated(a, "reduced"); }

} // namespace metal_linalg
