#pragma once
// The thin CUDA runtime under the QR kernels: per-GPU contexts (properties, a
// grow-only workspace per stream, staging streams), the calling thread's stream
// and device, and pointer classification. It stands where the reference has
// src/metal_runtime.{h,mm} (buffers, command queues) and src/device.mm.
#include <cuda_runtime.h>

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

namespace mlb {

// Throws std::runtime_error (std::bad_alloc for cudaErrorMemoryAllocation).
void cuda_check(cudaError_t e, const char* what);

struct Workspace {
    void*  data  = nullptr;
    size_t bytes = 0;
};

// What a kernel records when it gives up on a bounded wait: bits of the context's status word
// (DeviceContext::status, one word of device memory per GPU). The matrices concerned get NaN
// outputs; take_status() turns the word into an error for the caller.
enum : unsigned {
    kStatusTensorWait = 2u,   // an mbarrier wait of a tensor-core product (tc_gemm.cu, tc_gemm2.cu) or of a panel's cluster (qr_panel_cols.cuh)
    kStatusStreamWait = 4u,   // an mbarrier wait of the streaming small-matrix kernel (qr_small_stream.cu)
};

struct DeviceContext {
    int            device      = 0;
    int            sm_count    = 0;
    size_t         smem_optin  = 0;     // bytes of shared memory a block may opt into
    std::string    name;
    std::mutex     mutex;               // held while a call enqueues on this GPU
    unsigned*      status      = nullptr;   // device word: kStatus* bits set by kernels that gave up on a wait
    uint32_t       last_shape[3] = {0, 0, 0};   // batch, rows, cols of the last QR enqueued here (for that error's message)
    std::map<cudaStream_t, Workspace> workspaces;
    std::map<cudaStream_t, Workspace> outer_workspaces;   // of a caller of the QR (the SVD), beside the QR's own
    cudaStream_t   copy_in = nullptr, copy_out = nullptr, compute = nullptr;   // host-pointer staging
    static constexpr int kStagingSets = 3;      // device buffer sets of the host-pointer pipeline
    cudaEvent_t    ev_in[kStagingSets] = {}, ev_done[kStagingSets] = {}, ev_out[kStagingSets] = {};
    // the blocked QR's second stream (trailing updates beside the next panels) and its events
    cudaStream_t   aux = nullptr;
    cudaEvent_t    ev_panel[2] = {nullptr, nullptr}, ev_update[2] = {nullptr, nullptr};
    // and its third: what the next aggregate's columns need of the current one, beside the chain of panels
    static constexpr int kLookEvents = 3;       // a panel is factored; the next aggregate's columns are complete; the aggregate's T is built
    cudaStream_t   look = nullptr;
    cudaEvent_t    ev_look[kLookEvents] = {};
    // further pairs of streams for a batch of large matrices, factored several at a time (the first
    // matrix of a round runs on the caller's stream and `aux`); created on first use
    struct Lane {
        cudaStream_t update = nullptr, panel = nullptr, look = nullptr;
        cudaEvent_t  ev_panel[2] = {nullptr, nullptr}, ev_update[2] = {nullptr, nullptr}, ev_done = nullptr;
        cudaEvent_t  ev_look[3] = {};
    };
    static constexpr int kExtraLanes = 3;
    Lane           lanes[kExtraLanes];
    cudaEvent_t    ev_fork = nullptr;
    Lane&          lane(int i);         // i < kExtraLanes

    // At least `bytes` of device scratch for work on `stream`, 256-byte aligned,
    // kept for later calls. Growing it waits for the GPU (cudaFree does).
    void* workspace(cudaStream_t stream, size_t bytes);
    // The same for a routine that calls the QR on `stream` and needs scratch that outlives that call.
    void* outer_workspace(cudaStream_t stream, size_t bytes);
    // Frees every stream's workspace after waiting for the GPU; they are allocated again on demand.
    // Returns the bytes given back.
    size_t release_workspaces();
    // Reads and clears the status word (the caller has synchronised the work it asks about).
    unsigned take_status();
};

// Throws std::runtime_error naming the wait and the last shape enqueued if any created context's
// status word is set (and clears it). The caller has synchronised the work it asks about.
void throw_if_a_kernel_gave_up();

// The contexts created so far (a context is created by the first call that uses its GPU).
int created_contexts(DeviceContext** out, int capacity);

// The GPU that is current for the calling thread (every launcher runs under a DeviceGuard).
int current_device();

// True the first time it is asked about `device` (and again if two threads ask at once, which is
// harmless for idempotent set-up): for per-GPU set-up of a kernel, such as the opt-in to more than
// 48 KB of shared memory, which cudaFuncSetAttribute records for the current device only.
class PerDeviceOnce {
public:
    bool first(int device) const { return !((done_.load(std::memory_order_acquire) >> (device & 63)) & 1u); }
    void mark(int device) { done_.fetch_or((uint64_t)1 << (device & 63), std::memory_order_release); }
private:
    std::atomic<uint64_t> done_{0};
};

int            device_count();
DeviceContext& context(int device);   // created on first use; throws without a GPU

// Launches `kernel`, whose first statement is dependency_wait() (common.cuh), so that it may be
// brought onto the multiprocessors while the kernel before it in the stream still runs
// (programmatic stream serialization). QR_NO_PDL=1 in the environment makes it an ordinary launch.
bool dependent_launches_enabled();
template <typename... Params, typename... Args>
void launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent_launches_enabled() ? 1 : 0;
    cuda_check(cudaLaunchKernelEx(&cfg, kernel, Params(args)...), "cudaLaunchKernelEx");
}

// Testing aid: the next `count` matrices that go through the blocked QR behave as if a tensor-core
// product's bounded wait had run out at once (their products return without touching memory, their
// outputs are NaN, the context's status word is set). Nothing on the GPU is made to wait or fail.
void inject_wait_failures(int count);
bool take_injected_wait_failure();

// The calling thread's stream (device-pointer calls) and device (host-pointer calls).
cudaStream_t thread_stream();
void         set_thread_stream(cudaStream_t s);
int          thread_device();
void         set_thread_device(int device);

// Where a pointer lives: device >= 0 for CUDA device (or managed) memory, -1 for the host.
int pointer_device(const void* p);

// RAII: makes `device` current, restores the previous one.
class DeviceGuard {
public:
    explicit DeviceGuard(int device);
    ~DeviceGuard();
private:
    int previous_ = 0;
};

} // namespace mlb
