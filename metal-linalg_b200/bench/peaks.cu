// Measured compute ceilings of the GPU the benchmark runs on, for the roofline fractions bench.py
// reports: the FP32 FMA pipe (scalar and packed FMAs from registers) and the dense TF32 tensor
// pipe (tcgen05.mma kind::tf32, 128 x 256 x 8, operands resident in shared memory, accumulator in
// tensor memory). Nothing but the arithmetic runs in the timed loops, so these are ceilings no kernel
// that also moves data reaches. Not part of the product library: built into lib/libmlb_peaks.so
// and loaded by bench.py alone.
//
// Each entry point launches its kernel back to back for about `seconds`, times every launch with
// CUDA events and returns TFLOP/s over the whole period (sustained) and of the best launch
// (burst). bench.py samples the SM clock meanwhile and reports it beside the figures.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

namespace {

// ---------------------------------------------------------------------------
// FP32 FMA
// ---------------------------------------------------------------------------
constexpr int kChains = 16;

template <bool Packed>
__global__ void __launch_bounds__(1024, 1) ffma_kernel(float* sink, int iters, float seed) {
    float a = seed + threadIdx.x * 1e-7f, b = 0.999f;
    if (!Packed) {
        float acc[kChains];
#pragma unroll
        for (int i = 0; i < kChains; ++i) acc[i] = (float)i;
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int i = 0; i < kChains; ++i) acc[i] = fmaf(acc[i], b, a);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kChains; ++i) s += acc[i];
        if (s == 12345.678f) sink[0] = s;       // never true; keeps the arithmetic
    } else {
        unsigned long long acc[kChains / 2], a2, b2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(a2) : "f"(a));
        asm("mov.b64 %0, {%1, %1};" : "=l"(b2) : "f"(b));
#pragma unroll
        for (int i = 0; i < kChains / 2; ++i) asm("mov.b64 %0, {%1, %2};" : "=l"(acc[i]) : "f"((float)i), "f"((float)i + 0.5f));
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int i = 0; i < kChains / 2; ++i) asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[i]) : "l"(b2), "l"(a2));
        }
        unsigned long long s = 0;
#pragma unroll
        for (int i = 0; i < kChains / 2; ++i) s ^= acc[i];
        if (s == 0x123456789abcdefull) sink[0] = 1.0f;
    }
}

// ---------------------------------------------------------------------------
// TF32 tensor pipe
// ---------------------------------------------------------------------------
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr int kBatch = 32;                 // products per commit

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major, unswizzled canonical layout: 8 rows x 16 bytes core matrices, 128 bytes between 8-row
// groups, `lbo` bytes between the 16-byte columns of K
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (((lbo >> 4) & 0x3FFFu) << 16);
    const uint32_t hi = ((128u >> 4) & 0x3FFFu) | (1u << 14);
    return ((uint64_t)hi << 32) | lo;
}
// kind::tf32, float32 accumulator, A and B K-major, M = 128, N = 256
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// One block a multiprocessor: `batches` batches of kBatch products 128 x 256 x 8 into one accumulator.
// A wait that runs out sets *error and ends the block (its tensor memory freed).
__global__ void __launch_bounds__(128, 1) tf32_kernel(int batches, unsigned* error, float* sink) {
    __shared__ __align__(1024) float a_tile[128 * 8];
    __shared__ __align__(1024) float b_tile[256 * 8];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 128 * 8; i += 128) a_tile[i] = __uint_as_float(0x3f800000u + ((i * 2654435761u) & 0x7fe000u)) - 1.5f;
    for (int i = threadIdx.x; i < 256 * 8; i += 128) b_tile[i] = __uint_as_float(0x3f800000u + ((i * 40503u) & 0x7fe000u)) - 1.5f;
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" :: "r"(smem_u32(&tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;
    bool ok = true;
    if (threadIdx.x == 0) {
        const uint64_t da = make_desc(smem_u32(a_tile), 128 * 16), db = make_desc(smem_u32(b_tile), 256 * 16);
        for (int b = 0; b < batches && ok; ++b) {
            // at most two batches in flight: the batch issued two rounds ago has completed
            if (b >= 2 && !wait_barrier(smem_u32(&bars[b & 1]), ((b >> 1) - 1) & 1)) ok = false;
            if (!ok) break;
#pragma unroll 8
            for (int i = 0; i < kBatch; ++i) {
                const uint32_t acc = (b > 0 || i > 0) ? 1u : 0u;
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tmem_d), "l"(da), "l"(db), "r"(kInstrDesc), "r"(acc) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(smem_u32(&bars[b & 1])) : "memory");
        }
        for (int b = batches > 2 ? batches - 2 : 0; b < batches && ok; ++b)
            if (!wait_barrier(smem_u32(&bars[b & 1]), (b >> 1) & 1)) ok = false;
        if (!ok) atomicExch(error, 1u);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (threadIdx.x < 32 && *reinterpret_cast<volatile unsigned*>(error) == 0) {      // read one word back so that the products are observable
        uint32_t v;
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v) : "r"(tmem_d) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (__uint_as_float(v) == 12345.678f) sink[0] = 1.0f;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" :: "r"(tmem_d) : "memory");
}

struct Timed {
    double sustained = 0, burst = 0;
    int    launches = 0;
};

template <typename Launch>
int run_for(double seconds, double flops_per_launch, Launch&& launch, Timed& out) {
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return 1;
    for (int i = 0; i < 3; ++i) launch();
    if (cudaDeviceSynchronize() != cudaSuccess) return 2;
    double total_ms = 0, best_ms = 1e30;
    while (total_ms < seconds * 1e3 && out.launches < 100000) {
        cudaEventRecord(e0);
        launch();
        cudaEventRecord(e1);
        if (cudaEventSynchronize(e1) != cudaSuccess) return 3;
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        total_ms += ms;
        if (ms < best_ms) best_ms = ms;
        ++out.launches;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (cudaGetLastError() != cudaSuccess) return 4;
    out.sustained = flops_per_launch * out.launches / (total_ms * 1e-3) / 1e12;
    out.burst = flops_per_launch / (best_ms * 1e-3) / 1e12;
    return 0;
}

} // namespace

extern "C" {

// FP32 FMA peak, TFLOP/s (2 flops an FMA). packed != 0: fma.rn.f32x2. Returns 0 on success.
int mlb_peak_ffma(double seconds, int packed, double* sustained, double* burst, int* launches) {
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    float* sink = nullptr;
    if (cudaMalloc(&sink, 256) != cudaSuccess) return 10;
    const int iters = 4096;
    const double flops = (double)sms * 2 * 1024 * iters * 8.0 * kChains * 2.0;
    Timed t;
    const int rc = run_for(seconds, flops, [&] {
        if (packed) ffma_kernel<true><<<sms * 2, 1024>>>(sink, iters, 0.5f);
        else ffma_kernel<false><<<sms * 2, 1024>>>(sink, iters, 0.5f);
    }, t);
    cudaFree(sink);
    *sustained = t.sustained; *burst = t.burst; *launches = t.launches;
    return rc;
}

// Dense TF32 tensor-pipe peak, TFLOP/s: 128 x 256 x 8 products from shared memory, one block a
// multiprocessor. Returns 0 on success, 20 if a bounded wait inside the kernel ran out.
int mlb_peak_tf32(double seconds, double* sustained, double* burst, int* launches) {
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    unsigned* error = nullptr;
    if (cudaMalloc(&error, 512) != cudaSuccess) return 10;
    cudaMemset(error, 0, 512);
    float* sink = reinterpret_cast<float*>(error) + 64;
    const int batches = 2048;      // x 32 products of 0.52 MFLOP: about 5 ms a launch
    const double flops = (double)sms * batches * kBatch * (2.0 * 128 * 256 * 8);
    Timed t;
    int rc = run_for(seconds, flops, [&] { tf32_kernel<<<sms, 128>>>(batches, error, sink); }, t);
    unsigned word = 0;
    cudaMemcpy(&word, error, sizeof word, cudaMemcpyDeviceToHost);
    cudaFree(error);
    if (rc == 0 && word) rc = 20;
    *sustained = t.sustained; *burst = t.burst; *launches = t.launches;
    return rc;
}

} // extern "C"
