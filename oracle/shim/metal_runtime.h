// TEST INFRASTRUCTURE ONLY. The three host helpers the reference's CPU QR
// (src/qr_cpu.mm) takes from its Metal runtime header, declared here without
// Metal so that file compiles unchanged on Linux. Their behaviour follows
// src/metal_runtime.mm:140-170 (scan) and :402-432 (lapack_batches); the
// definitions are in ref_glue.cpp.
#pragma once
#include <metal_linalg/core.h>

#include <cstddef>
#include <cstdint>
#include <functional>

namespace metal_linalg::detail {

enum class Part { all, lower, upper };

// Largest magnitude and finiteness (no NaN, no infinity) of each matrix.
void scan(const core::Matrices& a, Part part, float* amax, char* finite);

// f(b0, b1) on chunks of [0, batch), four chunks per thread over cpu_threads()
// threads with the BLAS single-threaded meanwhile; one matrix or one thread
// runs f(0, batch) on the caller with the BLAS's own threading.
void lapack_batches(uint32_t batch, size_t per, const std::function<void(uint32_t, uint32_t)>& f);

} // namespace metal_linalg::detail
