#pragma once
// Device helpers shared by the QR kernels: power-of-two scaling, the Householder
// reflector, warp reductions.
#include <cuda_runtime.h>

#include <cstdint>

namespace mlb {

// A reflector whose tail has a plain sum of squares below this, on a matrix
// scaled so that its largest entry lies in [0.5, 1), is taken as zero (tau = 0,
// H = I): the same cut as the reference's kernels (shaders/QR_Householder.metal:
// 123-142), 2^-80, under which squares begin to underflow unevenly.
constexpr float kTinySumsq = 8.271806e-25f;

__device__ __forceinline__ bool nonfinite(float v) {
    return (__float_as_uint(v) & 0x7F800000u) == 0x7F800000u;
}

// e with amax * 2^-e in [0.5, 1); 0 for amax == 0.
__device__ __forceinline__ int amax_exponent(float amax) {
    if (!(amax > 0.0f)) return 0;
    int e;
    frexpf(amax, &e);
    return e;
}

// 2^e for e in [-126, 127].
__device__ __forceinline__ float pow2f(int e) { return __uint_as_float((uint32_t)(e + 127) << 23); }

// x * 2^e, exact wherever the result is representable, as two multiplications
// by normal powers of two (|e| <= 160).
struct Pow2 {
    float s1, s2;
    __device__ __forceinline__ explicit Pow2(int e) {
        const int e1 = e / 2;
        s1 = pow2f(e1);
        s2 = pow2f(e - e1);
    }
    __device__ __forceinline__ float operator()(float x) const { return x * s1 * s2; }
};

// LAPACK slarfg's reflector for a column (alpha; tail) whose tail has sum of
// squares ss: H = I - tau v v^T with v = (1; sc * tail), H (alpha; tail) =
// (beta; 0). tau = 0 and sc = 0 (H = I, beta = alpha) for a tail taken as zero.
__device__ __forceinline__ void reflector(float alpha, float ss, float& beta, float& tau, float& sc) {
    beta = alpha;
    tau  = 0.0f;
    sc   = 0.0f;
    if (ss >= kTinySumsq) {
        beta = -copysignf(sqrtf(fmaf(alpha, alpha, ss)), alpha);
        tau  = (beta - alpha) / beta;
        sc   = 1.0f / (alpha - beta);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// First thing in a kernel that may be launched with programmatic stream serialization
// (launch_dependent in runtime.h): wait until the kernels before it in the stream have completed
// and their memory is visible, then let the next kernel in the stream be brought onto the
// multiprocessors, where it waits at the same place. The launch latency of a chain of short
// kernels is hidden this way, one kernel ahead. Without that launch attribute both are no-ops.
__device__ __forceinline__ void dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// The same for a kernel whose grid may be larger than the GPU holds at once: it waits, but lets the
// next kernel come only when it ends (waiting blocks would take the places of its own).
__device__ __forceinline__ void dependency_wait_only() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float qnan() { return __uint_as_float(0x7FC00000u); }

} // namespace mlb
