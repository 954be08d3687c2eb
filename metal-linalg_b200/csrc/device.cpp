// Device queries and the calling thread's settings (reference: src/device.mm,
// include/metal_linalg/device.h).
#include <metal_linalg/core.h>

#include "runtime.h"

#include <atomic>
#include <mutex>
#include <thread>

namespace metal_linalg {

namespace {
std::atomic<unsigned> g_cpu_threads{0};
thread_local bool     t_cpu_only = false;
}

const char* device_name() {
    if (mlb::device_count() == 0) return "";
    return mlb::context(0).name.c_str();
}
unsigned gpu_core_count() {
    if (mlb::device_count() == 0) return 0;
    return (unsigned)mlb::context(0).sm_count;
}

void     set_cpu_threads(unsigned n) { g_cpu_threads = n; }
unsigned cpu_threads() {
    const unsigned n = g_cpu_threads.load();
    return n ? n : std::max(1u, std::thread::hardware_concurrency());
}

void set_cpu_only(bool on) { t_cpu_only = on; }
bool cpu_only() { return t_cpu_only; }

void  set_stream(void* s) { mlb::set_thread_stream(static_cast<cudaStream_t>(s)); }
void* stream() { return mlb::thread_stream(); }
void  set_device(int device) { mlb::set_thread_device(device); }
int   device() { return mlb::thread_device(); }
int   device_count() { return mlb::device_count(); }

void synchronize() {
    mlb::cuda_check(cudaStreamSynchronize(mlb::thread_stream()), "cudaStreamSynchronize");
    mlb::throw_if_a_kernel_gave_up();
}

void inject_wait_failures(int count) { mlb::inject_wait_failures(count); }

size_t release_workspaces() {
    mlb::DeviceContext* all[64];
    const int n = mlb::created_contexts(all, 64);
    size_t freed = 0;
    for (int i = 0; i < n; ++i) {
        std::lock_guard<std::mutex> lock(all[i]->mutex);
        freed += all[i]->release_workspaces();
    }
    return freed;
}

} // namespace metal_linalg
