#pragma once
// The thin CUDA runtime under the QR kernels: per-GPU contexts (properties, a
// grow-only workspace per stream, staging streams), the calling thread's stream
// and device, and pointer classification. It stands where the reference has
// src/metal_runtime.{h,mm} (buffers, command queues) and src/device.mm.
#include <cuda_runtime.h>

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

// Status words the kernels write: one per stream workspace, in device memory,
// read back by synchronize(). Non-zero means a bounded wait ran out.
struct DeviceContext {
    int            device      = 0;
    int            sm_count    = 0;
    size_t         smem_optin  = 0;     // bytes of shared memory a block may opt into
    std::string    name;
    std::mutex     mutex;               // held while a call enqueues on this GPU
    std::map<cudaStream_t, Workspace> workspaces;
    cudaStream_t   copy_in = nullptr, copy_out = nullptr, compute = nullptr;   // host-pointer staging
    cudaEvent_t    ev_in[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr},
                   ev_out[2] = {nullptr, nullptr};
    // the blocked QR's second stream (trailing updates beside the next panels) and its events
    cudaStream_t   aux = nullptr;
    cudaEvent_t    ev_panel[2] = {nullptr, nullptr}, ev_update[2] = {nullptr, nullptr};

    // At least `bytes` of device scratch for work on `stream`, 256-byte aligned,
    // kept for later calls. Growing it waits for the GPU (cudaFree does).
    void* workspace(cudaStream_t stream, size_t bytes);
};

int            device_count();
DeviceContext& context(int device);   // created on first use; throws without a GPU

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
