// The small-matrix kernel for square matrices of 8, 16 or 32 rows, streaming:
// persistent warps that take their matrices through shared memory with bulk
// asynchronous copies, so that no warp ever waits on a load from, or a store to,
// global memory while it holds the registers of a factorisation.
//
// The arithmetic is that of qr_small.cu (qr_small_steps.cuh; it takes the place
// of the reference's register kernel, shaders/QR_Householder.metal:189-300). What
// differs is the traffic. A warp owns two staging buffers and one mbarrier in
// shared memory and loops over units of 32 / G matrices:
//
//   buffer A   the unit's input, landed by cp.async.bulk (one copy a matrix,
//              completion counted in bytes on the mbarrier); once the matrices
//              are in registers it takes R, which leaves by a bulk store
//   buffer B   the reflectors while the unit is factored and Q is formed, then Q,
//              which leaves by a bulk store (when only R is asked for, R is staged
//              here and buffer A is free for the next unit from the start)
//
// The next unit's input is requested as soon as buffer A is free: half way through
// the Q pass, when the bulk store of R has read it (at once when only R is asked
// for). It arrives while the warp computes; the stores drain while the next unit
// is loaded and scaled. Matrices sit G floats apart in the buffers so that the
// lanes of a warp, which read and write 32 / G different matrices at once, fall in
// different banks.
//
// The only wait that spins is the mbarrier wait, and it is bounded: if it runs out
// the warp gives up its remaining units, fills their outputs with NaN (visible, not
// silent), waits once more, bounded, for the copy in flight, and returns.
#include "kernels.h"
#include "qr_small_steps.cuh"

#include <algorithm>
#include <cstdlib>

namespace mlb {

using namespace small;

namespace {

struct StreamParams {
    const float* a;
    float*       q;      // null: R alone
    float*       r;
    uint32_t     batch;
    unsigned*    status; // the context's status word: kStatusStreamWait is set by a warp that gives up
};

constexpr int      kWarps     = 4;            // warps a block; every warp works alone
constexpr uint32_t kSpinLimit = 1u << 22;     // polls of the mbarrier before a warp gives up

template <int R, int G, int C>
struct Shape {
    static constexpr int kMats = 32 / G;                     // matrices a warp
    static constexpr int kMat  = R * R;                      // floats a matrix
    static constexpr int kIo   = kMat + G;                   // floats from one matrix to the next in a staging buffer
    static constexpr int kSlot = slot_floats(R, R);          // floats of reflectors a matrix
    static constexpr int kBufA = kMats * kIo;
    static constexpr int kBufB = kMats * (kSlot > kIo ? kSlot : kIo);
    static constexpr int kWarpFloats = kBufA + kBufB + 4;    // and the mbarrier, 16 bytes
    // blocks a multiprocessor is to hold: by shared memory (227 KB less 1 KB a block), capped so
    // that the registers of a lane (R * C matrix entries and some 60 more) are there
    static constexpr int kBlocks = R == 32 ? 3 : R == 16 ? 5 : 10;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// global -> shared, completion in bytes on the mbarrier; both addresses and the size multiples of 16
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// shared -> global, in the calling thread's bulk group
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(dst), "r"(src), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// the calling thread's bulk stores have read their shared memory
__device__ __forceinline__ void stores_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void stores_done() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// the shared-memory writes above, visible to the bulk copy engine
__device__ __forceinline__ void fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int R, int G, int C>
__global__ void __launch_bounds__(kWarps * 32, Shape<R, G, C>::kBlocks) qr_small_stream_kernel(const StreamParams p) {
    using S = Shape<R, G, C>;
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane % G;              // this lane's first column
    const int h = lane / G;              // its matrix within the unit
    float* bufA = smem + (size_t)warp * S::kWarpFloats;
    float* bufB = bufA + S::kBufA;
    const uint32_t bar = smem_u32(bufB + S::kBufB);
    const bool with_q = p.q != nullptr;

    const uint32_t units = (p.batch + S::kMats - 1) / S::kMats;
    const uint32_t gw = blockIdx.x * kWarps + warp, GW = gridDim.x * kWarps;
    if (gw >= units) return;

    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // request unit u's matrices into buffer A: lane 0 announces the bytes, lane i copies matrix i
    auto request = [&](uint32_t u) {
        const uint32_t first = u * S::kMats;
        const uint32_t count = min((uint32_t)S::kMats, p.batch - first);
        if (lane == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                         :: "r"(bar), "r"(count * (uint32_t)(S::kMat * sizeof(float))) : "memory");
        __syncwarp();
        if (lane < (int)count)
            bulk_load(smem_u32(bufA + lane * S::kIo), p.a + (size_t)(first + lane) * S::kMat, S::kMat * sizeof(float), bar);
    };
    // send the unit's staged matrices (R or Q) from `buf` to `out`: lane i stores matrix i
    auto send = [&](const float* buf, float* out, uint32_t u) {
        fence_async();
        __syncwarp();
        const uint32_t first = u * S::kMats;
        if (lane < S::kMats && first + lane < p.batch)
            bulk_store(out + (size_t)(first + lane) * S::kMat, smem_u32(buf + lane * S::kIo), S::kMat * sizeof(float));
    };

    request(gw);
    uint32_t parity = 0;
    for (uint32_t u = gw; u < units; u += GW) {
        const uint32_t next = u + GW;
        const bool arrived = wait_barrier(bar, parity);
        parity ^= 1;
        if (!__all_sync(0xffffffffu, arrived)) {
            // give up: NaN in every output this warp still owes, a last bounded wait for the copy
            // in flight, the stores drained; the context's status word tells the host
            if (lane == 0) atomicOr(p.status, (unsigned)kStatusStreamWait);
            for (uint32_t v = u; v < units; v += GW)
                for (uint32_t i = 0; i < (uint32_t)S::kMats; ++i) {
                    const uint32_t mat = v * S::kMats + i;
                    if (mat >= p.batch) break;
                    for (int e = lane; e < S::kMat; e += 32) {
                        p.r[(size_t)mat * S::kMat + e] = qnan();
                        if (with_q) p.q[(size_t)mat * S::kMat + e] = qnan();
                    }
                }
            wait_barrier(bar, parity ^ 1);
            break;
        }

        // 1. the matrices from buffer A to registers: rows 2p and 2p+1 of column l + c G in x2[c][p]
        pair_t x2[C][R / 2];
        {
            const float* in = bufA + h * S::kIo;
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < R / 2; ++i)
                    x2[c][i] = pack(in[(2 * i) * R + l + c * G], in[(2 * i + 1) * R + l + c * G]);
        }
        __syncwarp();
        if (!with_q && next < units) request(next);       // buffer A is free for the whole unit
        bool bad;
        int  expo;
        scan_scale<R, G, C>(x2, bad, expo);

        // 2. factor, once the last store out of buffer B has read it
        if (lane < S::kMats) stores_read();
        __syncwarp();
        float* slot = bufB + h * S::kSlot;
        factor<R, G, C>(x2, slot, l, R);

        // 3. R, with exact zeros below the diagonal, staged and sent
        scale_up<R, G, C>(x2, expo, bad);
        {
            float* stage = (with_q ? bufA : bufB) + h * S::kIo;
            const float zero = bad ? qnan() : 0.0f;
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const float v = (i & 1) ? hi_of(x2[c][i / 2]) : lo_of(x2[c][i / 2]);
                    stage[i * R + l + c * G] = l + c * G >= i ? v : zero;
                }
            send(with_q ? bufA : bufB, p.r, u);
        }
        if (!with_q) continue;

        // 4. Q; half way, when the store of R has read buffer A, the next unit is requested
        pair_t q2[C][R / 2];
        form_q<R, G, C>(q2, slot, l, R, bad, [&] {
            if (lane < S::kMats) stores_read();
            __syncwarp();
            if (next < units) request(next);
        });
        __syncwarp();            // every lane has read the last reflector: buffer B takes Q
        {
            float* stage = bufB + h * S::kIo;
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int i = 0; i < R / 2; ++i) {
                    float a, b;
                    unpack(q2[c][i], a, b);
                    stage[(2 * i) * R + l + c * G] = a;
                    stage[(2 * i + 1) * R + l + c * G] = b;
                }
            send(bufB, p.q, u);
        }
    }
    if (lane < S::kMats) stores_done();     // shared memory is read, and global memory written, before the warp leaves
}

template <int R, int G, int C>
void launch(const DeviceContext& ctx, cudaStream_t stream, const StreamParams& p) {
    using S = Shape<R, G, C>;
    constexpr size_t smem = (size_t)kWarps * S::kWarpFloats * sizeof(float);
    static PerDeviceOnce once;                 // the opt-in is recorded per GPU
    static std::atomic<int> blocks_per_sm{1};  // the same on every GPU of a machine
    if (once.first(ctx.device)) {
        cuda_check(cudaFuncSetAttribute(qr_small_stream_kernel<R, G, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                   "qr_small_stream shared memory");
        cuda_check(cudaFuncSetAttribute(qr_small_stream_kernel<R, G, C>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared),
                   "qr_small_stream shared memory carveout");
        int n = 0;
        cuda_check(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, qr_small_stream_kernel<R, G, C>, kWarps * 32, smem),
                   "qr_small_stream occupancy");
        blocks_per_sm = n > 0 ? n : 1;
        once.mark(ctx.device);
    }
    const uint32_t units  = (p.batch + S::kMats - 1) / S::kMats;
    const uint32_t wanted = (units + kWarps - 1) / kWarps;
    const uint32_t blocks = std::min<uint32_t>(wanted, (uint32_t)(blocks_per_sm * ctx.sm_count));
    qr_small_stream_kernel<R, G, C><<<blocks, kWarps * 32, smem, stream>>>(p);
}

// QR_SMALL_STREAM: 0 never, 1 (default) where measured faster, 2 wherever the shape allows
int stream_mode() {
    const char* e = std::getenv("QR_SMALL_STREAM");      // read at every call: tests switch it
    const int m = e && *e ? std::atoi(e) : 1;
    return m >= 0 && m <= 2 ? m : 1;
}

} // namespace

// Square matrices of 8, 16 or 32 rows with Q square or not asked for, every pointer on a 16-byte
// boundary: true when the streaming kernel has taken the call. By default it takes the shapes
// where it was measured faster than the kernel of qr_small.cu (millions of matrices a second on a
// B200, streaming against direct): 16 x 16 with Q 1370 against 1137, R alone 1990 against 1557;
// 32 x 32 R alone 322 against 276. It leaves 32 x 32 with Q (188 against 197: its shared memory
// holds 12 warps a multiprocessor where the other kernel runs 16) and 8 x 8 (4330 against 4630).
// QR_SMALL_STREAM=0 turns it off, QR_SMALL_STREAM=2 gives it every shape it can take.
bool launch_qr_small_stream(DeviceContext& ctx, cudaStream_t stream, const QrProblem& pr) {
    const uint32_t n = pr.n;
    if (stream_mode() == 0 || pr.m != n || (n != 8 && n != 16 && n != 32)) return false;
    if (pr.rr != n || (pr.qc != 0 && pr.qc != n)) return false;
    if (stream_mode() == 1 && !(n == 16 || (n == 32 && pr.qc == 0))) return false;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(pr.a) | reinterpret_cast<uintptr_t>(pr.r) |
                           (pr.qc ? reinterpret_cast<uintptr_t>(pr.q) : 0);
    if (bits & 15) return false;
    if (pr.batch == 0) return true;
    const StreamParams p{pr.a, pr.qc ? pr.q : nullptr, pr.r, pr.batch, ctx.status};
    if (n == 32) launch<32, 16, 2>(ctx, stream, p);
    else if (n == 16) launch<16, 8, 2>(ctx, stream, p);
    else launch<8, 8, 1>(ctx, stream, p);
    cuda_check(cudaGetLastError(), "qr_small_stream launch");
    return true;
}

} // namespace mlb
