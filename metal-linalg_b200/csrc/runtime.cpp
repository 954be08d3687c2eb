// Per-GPU contexts, the calling thread's stream and device, workspaces.
#include "runtime.h"

#include <cstdlib>
#include <memory>
#include <new>
#include <vector>

namespace mlb {

void cuda_check(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return;
    cudaGetLastError();   // clear the sticky-less error so the next call starts clean
    if (e == cudaErrorMemoryAllocation) throw std::bad_alloc();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

bool dependent_launches_enabled() {
    static const bool v = [] {
        const char* e = std::getenv("QR_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return v;
}

int current_device() {
    int d = 0;
    cuda_check(cudaGetDevice(&d), "cudaGetDevice");
    return d;
}

int device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

DeviceGuard::DeviceGuard(int device) {
    cuda_check(cudaGetDevice(&previous_), "cudaGetDevice");
    if (device != previous_) cuda_check(cudaSetDevice(device), "cudaSetDevice");
    else previous_ = -1;
}
DeviceGuard::~DeviceGuard() {
    if (previous_ >= 0) cudaSetDevice(previous_);
}

namespace {
std::mutex g_contexts_mutex;
std::vector<std::unique_ptr<DeviceContext>> g_contexts;

thread_local cudaStream_t t_stream = nullptr;
thread_local int          t_device = 0;
}

DeviceContext& context(int device) {
    std::lock_guard<std::mutex> lock(g_contexts_mutex);
    const int n = device_count();
    if (n == 0) throw std::runtime_error("no CUDA device: this library has no CPU path");
    if (device < 0 || device >= n) throw std::invalid_argument("no such CUDA device: " + std::to_string(device));
    if (g_contexts.size() < (size_t)n) g_contexts.resize(n);
    if (!g_contexts[device]) {
        auto c = std::make_unique<DeviceContext>();
        c->device = device;
        cudaDeviceProp prop{};
        cuda_check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
        c->sm_count   = prop.multiProcessorCount;
        c->smem_optin = prop.sharedMemPerBlockOptin;
        c->name       = prop.name;
        DeviceGuard guard(device);
        cuda_check(cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking), "cudaStreamCreate");
        cuda_check(cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking), "cudaStreamCreate");
        cuda_check(cudaStreamCreateWithFlags(&c->compute, cudaStreamNonBlocking), "cudaStreamCreate");
        int least = 0, greatest = 0;   // the panel chain of the blocked QR goes ahead of the bulk updates
        cuda_check(cudaDeviceGetStreamPriorityRange(&least, &greatest), "cudaDeviceGetStreamPriorityRange");
        cuda_check(cudaStreamCreateWithPriority(&c->aux, cudaStreamNonBlocking, greatest), "cudaStreamCreate");
        cuda_check(cudaStreamCreateWithPriority(&c->look, cudaStreamNonBlocking, greatest), "cudaStreamCreate");
        for (int i = 0; i < DeviceContext::kLookEvents; ++i)
            cuda_check(cudaEventCreateWithFlags(&c->ev_look[i], cudaEventDisableTiming), "cudaEventCreate");
        cuda_check(cudaMalloc(&c->status, 256), "cudaMalloc");
        cuda_check(cudaMemset(c->status, 0, 256), "cudaMemset");
        for (int i = 0; i < 2; ++i) {
            cuda_check(cudaEventCreateWithFlags(&c->ev_panel[i], cudaEventDisableTiming), "cudaEventCreate");
            cuda_check(cudaEventCreateWithFlags(&c->ev_update[i], cudaEventDisableTiming), "cudaEventCreate");
        }
        for (int i = 0; i < DeviceContext::kStagingSets; ++i) {
            cuda_check(cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming), "cudaEventCreate");
            cuda_check(cudaEventCreateWithFlags(&c->ev_done[i], cudaEventDisableTiming), "cudaEventCreate");
            cuda_check(cudaEventCreateWithFlags(&c->ev_out[i], cudaEventDisableTiming), "cudaEventCreate");
        }
        g_contexts[device] = std::move(c);
    }
    return *g_contexts[device];
}

DeviceContext::Lane& DeviceContext::lane(int i) {
    Lane& l = lanes[i];
    if (!l.update) {
        DeviceGuard guard(device);
        int least = 0, greatest = 0;
        cuda_check(cudaDeviceGetStreamPriorityRange(&least, &greatest), "cudaDeviceGetStreamPriorityRange");
        cuda_check(cudaStreamCreateWithFlags(&l.update, cudaStreamNonBlocking), "cudaStreamCreate");
        cuda_check(cudaStreamCreateWithPriority(&l.panel, cudaStreamNonBlocking, greatest), "cudaStreamCreate");
        cuda_check(cudaStreamCreateWithPriority(&l.look, cudaStreamNonBlocking, greatest), "cudaStreamCreate");
        for (int k = 0; k < kLookEvents; ++k)
            cuda_check(cudaEventCreateWithFlags(&l.ev_look[k], cudaEventDisableTiming), "cudaEventCreate");
        for (int k = 0; k < 2; ++k) {
            cuda_check(cudaEventCreateWithFlags(&l.ev_panel[k], cudaEventDisableTiming), "cudaEventCreate");
            cuda_check(cudaEventCreateWithFlags(&l.ev_update[k], cudaEventDisableTiming), "cudaEventCreate");
        }
        cuda_check(cudaEventCreateWithFlags(&l.ev_done, cudaEventDisableTiming), "cudaEventCreate");
        if (!ev_fork) cuda_check(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming), "cudaEventCreate");
    }
    return l;
}

namespace {
void* grown(Workspace& w, int device, size_t bytes) {
    if (w.bytes < bytes) {
        DeviceGuard guard(device);
        if (w.data) cuda_check(cudaFree(w.data), "cudaFree");   // waits for the work that may still use it
        w.data = nullptr;
        w.bytes = 0;
        const size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
        cuda_check(cudaMalloc(&w.data, want), "cudaMalloc");
        w.bytes = want;
    }
    return w.data;
}
} // namespace

void* DeviceContext::workspace(cudaStream_t stream, size_t bytes) { return grown(workspaces[stream], device, bytes); }
void* DeviceContext::outer_workspace(cudaStream_t stream, size_t bytes) {
    return grown(outer_workspaces[stream], device, bytes);
}

size_t DeviceContext::release_workspaces() {
    DeviceGuard guard(device);
    cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    size_t freed = 0;
    for (auto* table : {&workspaces, &outer_workspaces}) {
        for (auto& entry : *table) {
            if (entry.second.data) cuda_check(cudaFree(entry.second.data), "cudaFree");
            freed += entry.second.bytes;
        }
        table->clear();
    }
    return freed;
}

unsigned DeviceContext::take_status() {
    DeviceGuard guard(device);
    unsigned word = 0;
    cuda_check(cudaMemcpy(&word, status, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy");
    if (word) cuda_check(cudaMemset(status, 0, sizeof(word)), "cudaMemset");
    return word;
}

void throw_if_a_kernel_gave_up() {
    DeviceContext* all[64];
    const int n = created_contexts(all, 64);
    for (int i = 0; i < n; ++i) {
        const unsigned word = all[i]->take_status();
        if (!word) continue;
        std::string what = "a kernel on GPU " + std::to_string(all[i]->device) + " gave up on a bounded wait (";
        if (word & kStatusTensorWait) what += "a tensor-core product of the blocked QR";
        if ((word & kStatusTensorWait) && (word & kStatusStreamWait)) what += ", ";
        if (word & kStatusStreamWait) what += "a bulk copy of the streaming small-matrix kernel";
        what += "); the outputs of the matrices concerned are NaN; last QR enqueued there: batch " +
                std::to_string(all[i]->last_shape[0]) + " of " + std::to_string(all[i]->last_shape[1]) + " x " +
                std::to_string(all[i]->last_shape[2]);
        throw std::runtime_error(what);
    }
}

int created_contexts(DeviceContext** out, int capacity) {
    std::lock_guard<std::mutex> lock(g_contexts_mutex);
    int n = 0;
    for (auto& c : g_contexts)
        if (c && n < capacity) out[n++] = c.get();
    return n;
}

namespace {
std::atomic<int> g_injected_wait_failures{0};
}
void inject_wait_failures(int count) { g_injected_wait_failures = count > 0 ? count : 0; }
bool take_injected_wait_failure() {
    int left = g_injected_wait_failures.load();
    while (left > 0)
        if (g_injected_wait_failures.compare_exchange_weak(left, left - 1)) return true;
    return false;
}

cudaStream_t thread_stream() { return t_stream; }
void         set_thread_stream(cudaStream_t s) { t_stream = s; }
int          thread_device() { return t_device; }
void         set_thread_device(int device) {
    if (device < 0 || device >= device_count())
        throw std::invalid_argument("no such CUDA device: " + std::to_string(device));
    t_device = device;
}

int pointer_device(const void* p) {
    if (!p) return -1;
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) return attr.device;
    return -1;
}

} // namespace mlb
