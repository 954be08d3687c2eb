#pragma once
// The routed QR on device pointers, enqueued on `stream` with the context's lock already held:
// for the library's own callers of core::qr (the QR-preconditioned SVD).
#include <metal_linalg/core.h>

#include "runtime.h"

namespace metal_linalg {

void qr_enqueue(mlb::DeviceContext& ctx, cudaStream_t stream, const core::Matrices& a, float* q, float* r,
                core::QrMode mode);

} // namespace metal_linalg
