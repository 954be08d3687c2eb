// The two large products of the blocked QR's rank-128 updates on the fifth-generation tensor
// cores (tcgen05.mma with the accumulator in tensor memory), in float32 accuracy by the 3xTF32
// split:
//
//   a = a_hi + a_lo,  a_hi = tf32(a),  a_lo = a - a_hi  (exact in float32)
//   a b ~ a_hi b_hi + a_hi b_lo + a_lo b_hi             (the a_lo b_lo term, 2^-22 relative, dropped)
//
// with float32 accumulation in tensor memory. They stand where the reference calls
// MPSMatrixMultiplication for the trailing update and for Q's formation
// (src/band_reduce.mm:421-449).
//
//   tc_ytc   Zp[chunk] = Y^T C over a chunk of rows        (M = 128 reflectors, N = 128 columns, K = rows)
//   tc_yz    C -= Y Z on a 128 x 128 tile of C             (M = 128 rows, N = 128 columns, K = reflectors)
//
// One kernel serves both. Operands cannot come by TMA, because every float32 has to be split in
// two on the way: 256 threads load 128 x 32 tiles of A and B from global memory, split them and
// write hi and lo parts to shared memory in the K-major, unswizzled canonical layout (8 x 16-byte
// core matrices; SBO = 128 B between 8-row groups, LBO between the 16-byte columns of K). Two
// stages: while the tensor core works on one, the threads fill the other. One thread issues the
// twelve tcgen05.mma (128 x 128 x 8, kind::tf32) of a stage and commits them to the stage's
// mbarrier; the accumulator (128 lanes x 128 columns of tensor memory) is read back with
// tcgen05.ld for the epilogue. Every wait on an mbarrier is bounded: a wait that runs out sets
// an error word, and the block frees its tensor memory and returns.
#include "common.cuh"
#include "kernels.h"

#include <cuda_runtime.h>

namespace mlb {

namespace {

constexpr int TCT   = 256;                 // threads
constexpr int KT    = 16;                  // K elements per stage
constexpr int SBO   = 128;                 // bytes between 8-row groups
constexpr int LBO   = 16 * 128 + 16;       // bytes between 16-byte columns of K (16 row groups, padded one word)
constexpr int TILE  = (KT / 4) * LBO;      // bytes of one 128 x 32 operand tile
constexpr int STAGE = 4 * TILE;            // A_hi, A_lo, B_hi, B_lo
constexpr uint32_t kSpinLimit = 1u << 20;
constexpr int CLD   = 132;                 // leading dimension of the output tile in shared memory

struct TcParams {
    const float* a;        // operand A source
    const float* b;        // operand B source
    float*       out;      // Zp (ytc) or C (yz)
    size_t       lda, ldb, ldo;
    uint32_t     m_valid;  // ytc: kw (columns of Y that exist). yz: rows of the tile's matrix (mp)
    uint32_t     n_valid;  // columns of C (nc)
    uint32_t     k_total;  // ytc: rows mp. yz: kw
    uint32_t     k_chunk;  // ytc: rows per chunk (grid.y chunks). yz: unused
    uint32_t     mode;     // 0: ytc, 1: yz
    unsigned*    error;    // set non-zero when a bounded wait ran out
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (((uint32_t)(LBO >> 4) & 0x3FFFu) << 16);
    const uint32_t hi = ((uint32_t)(SBO >> 4) & 0x3FFFu) | (1u << 14);   // version 1 (Blackwell), no swizzle
    return ((uint64_t)hi << 32) | lo;
}

// kind::tf32, float32 accumulator, A and B K-major, M = 128, N = 128
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
    hi = __uint_as_float(h);
    lo = v - hi;
}

// Four K-consecutive values of one row (MN index r) of a tile, split, to the hi and lo tiles.
__device__ __forceinline__ void put_word(char* hi_tile, char* lo_tile, int r, int kq, float v0, float v1, float v2, float v3) {
    float h0, h1, h2, h3, l0, l1, l2, l3;
    split_tf32(v0, h0, l0); split_tf32(v1, h1, l1); split_tf32(v2, h2, l2); split_tf32(v3, h3, l3);
    const int off = kq * LBO + (r >> 3) * SBO + (r & 7) * 16;
    *reinterpret_cast<float4*>(hi_tile + off) = make_float4(h0, h1, h2, h3);
    *reinterpret_cast<float4*>(lo_tile + off) = make_float4(l0, l1, l2, l3);
}

// A 128 x 32 tile is fetched into registers (16 floats a thread) one tile ahead of its use, so that
// the global loads are in flight while the tensor core works and the block waits; `put` splits the
// values and writes them to shared memory.
//
// Tiles whose MN index runs along contiguous memory (element (mn, k) at src[k * ld + mn]): lanes
// along mn (coalesced), four k's a thread and word.
constexpr int WPT = KT / 8;                // 16-byte words per thread and tile
__device__ __forceinline__ void fetch_mn_contiguous(float (&v)[4 * WPT], const float* src, size_t ld, uint32_t mn_valid,
                                                    uint32_t k_valid) {
    const int mn = threadIdx.x & 127;
#pragma unroll
    for (int e = 0; e < WPT; ++e) {
        const int kq = (threadIdx.x >> 7) + 2 * e;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t k = 4 * kq + i;
            v[4 * e + i] = ((uint32_t)mn < mn_valid && k < k_valid) ? src[(size_t)k * ld + mn] : 0.0f;
        }
    }
}
__device__ __forceinline__ void put_mn_contiguous(const float (&v)[4 * WPT], char* hi_tile, char* lo_tile) {
    const int mn = threadIdx.x & 127;
#pragma unroll
    for (int e = 0; e < WPT; ++e)
        put_word(hi_tile, lo_tile, mn, (threadIdx.x >> 7) + 2 * e, v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
}

// Tiles whose K index runs along contiguous memory (element (mn, k) at src[mn * ld + k]).
__device__ __forceinline__ void fetch_k_contiguous(float (&v)[4 * WPT], const float* src, size_t ld, uint32_t mn_valid,
                                                   uint32_t k_valid, bool aligned) {
#pragma unroll
    for (int e = 0; e < WPT; ++e) {
        const int idx = threadIdx.x + TCT * e;
        const int kq = idx & (KT / 4 - 1), mn = idx / (KT / 4);
        if (aligned && k_valid == KT) {      // whole 16-byte words
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if ((uint32_t)mn < mn_valid) f = *reinterpret_cast<const float4*>(src + (size_t)mn * ld + 4 * kq);
            v[4 * e] = f.x; v[4 * e + 1] = f.y; v[4 * e + 2] = f.z; v[4 * e + 3] = f.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t k = 4 * kq + i;
                v[4 * e + i] = ((uint32_t)mn < mn_valid && k < k_valid) ? src[(size_t)mn * ld + k] : 0.0f;
            }
        }
    }
}
__device__ __forceinline__ void put_k_contiguous(const float (&v)[4 * WPT], char* hi_tile, char* lo_tile) {
#pragma unroll
    for (int e = 0; e < WPT; ++e) {
        const int idx = threadIdx.x + TCT * e;
        put_word(hi_tile, lo_tile, idx / (KT / 4), idx & (KT / 4 - 1), v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
    }
}

// Waits for the phase of `parity` of the mbarrier; false if the wait ran out.
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

__global__ void __launch_bounds__(TCT, 2) tc_gemm_kernel(const TcParams p) {
    dependency_wait_only();
    extern __shared__ __align__(1024) char smem[];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t j0 = blockIdx.x * 128;
    if (threadIdx.x == 0) failed = *reinterpret_cast<volatile unsigned*>(p.error) != 0;
    __syncthreads();
    if (failed) return;   // an earlier block or launch gave up: do nothing (the same answer for the whole block)

    // this block's part of the product
    const float *a_src, *b_src;
    uint32_t k_begin = 0, k_end, m_valid, n_valid = p.n_valid > j0 ? p.n_valid - j0 : 0;
    if (p.mode == 0) {          // Zp[chunk] = Y^T C: A[m = i][k = r] = Y[r][i], B[n = j][k = r] = C[r][j0 + j]
        k_begin = blockIdx.y * p.k_chunk;
        k_end = min(p.k_total, k_begin + p.k_chunk);
        a_src = p.a + (size_t)k_begin * p.lda;
        b_src = p.b + (size_t)k_begin * p.ldb + j0;
        m_valid = p.m_valid;
    } else {                    // C -= Y Z: A[m = r][k] = Y[r0 + r][k], B[n = j][k] = Z[k][j0 + j]
        const uint32_t r0 = blockIdx.y * 128;
        k_end = p.k_total;
        a_src = p.a + (size_t)r0 * p.lda;
        b_src = p.b + j0;
        m_valid = p.m_valid > r0 ? p.m_valid - r0 : 0;
    }
    const uint32_t k_len = k_end - k_begin, tiles = (k_len + KT - 1) / KT;

    // The block's 128 x 128 tile of the output goes through shared memory, so that global memory
    // sees whole rows. It takes the stages' place once the products are done (two blocks fit a
    // multiprocessor that way, and one block's waits hide behind the other's work).
    float (*Ct)[CLD] = reinterpret_cast<float (*)[CLD]>(smem);
    float* out_tile = p.out + (size_t)blockIdx.y * 128 * p.ldo + j0;
    const uint32_t out_rows = p.mode == 0 ? 128u : min(m_valid, 128u);
    const bool out_vec = (p.ldo & 3) == 0 && (reinterpret_cast<size_t>(out_tile) & 15) == 0 && n_valid >= 128;

    // C -= Y Z: the tile of C is fetched now, a warp a row and sixteen rows a warp all in flight, and waits in
    // registers until the products are done (read row by row afterwards, every row waited for L2)
    float4 creg[128 / (TCT / 32)];
    const bool c_early = p.mode == 1 && out_vec;
    if (c_early) {
#pragma unroll
        for (int u = 0; u < 128 / (TCT / 32); ++u) {
            const uint32_t r = warp + (TCT / 32) * u;
            creg[u] = r < out_rows ? *reinterpret_cast<const float4*>(out_tile + (size_t)r * p.ldo + 4 * lane)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&bars[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {            // 128 columns of tensor memory for the 128 x 128 float32 accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" :: "r"(smem_u32(&tmem_base_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    const bool a_aligned = (p.lda & 3) == 0 && (reinterpret_cast<size_t>(a_src) & 15) == 0;
    float ra[4 * WPT], rb[4 * WPT];
    auto fetch = [&](uint32_t kt) {
        const uint32_t k0 = kt * KT, kv = min(k_len - k0, (uint32_t)KT);
        if (p.mode == 0) fetch_mn_contiguous(ra, a_src + (size_t)k0 * p.lda, p.lda, m_valid, kv);
        else             fetch_k_contiguous(ra, a_src + k0, p.lda, m_valid, kv, a_aligned);
        fetch_mn_contiguous(rb, b_src + (size_t)k0 * p.ldb, p.ldb, n_valid, kv);
    };
    if (tiles > 0) fetch(0);
    for (uint32_t kt = 0; kt < tiles; ++kt) {
        const int stage = kt & 1;
        char* base = smem + stage * STAGE;
        // the stage is free once the products issued from it two tiles ago have completed
        if (kt >= 2 && !failed) {
            if (!wait_barrier(smem_u32(&bars[stage]), ((kt >> 1) - 1) & 1)) failed = 1;
        }
        if (p.mode == 0) put_mn_contiguous(ra, base, base + TILE);
        else             put_k_contiguous(ra, base, base + TILE);
        put_mn_contiguous(rb, base + 2 * TILE, base + 3 * TILE);
        if (kt + 1 < tiles) fetch(kt + 1);                             // in flight while the tensor core works
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the writes above, visible to the tensor core
        __syncthreads();
        if (threadIdx.x == 0 && !failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(base), a_lo = a_hi + TILE, b_hi = a_hi + 2 * TILE, b_lo = a_hi + 3 * TILE;
#pragma unroll
            for (int ks = 0; ks < KT / 8; ++ks) {
                const uint32_t koff = ks * 2 * LBO;             // two 16-byte columns of K per instruction
                const uint64_t dah = make_desc(a_hi + koff), dal = make_desc(a_lo + koff);
                const uint64_t dbh = make_desc(b_hi + koff), dbl = make_desc(b_lo + koff);
                const uint32_t acc0 = (kt > 0 || ks > 0) ? 1u : 0u;
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tmem_d), "l"(dal), "l"(dbh), "r"(kInstrDesc), "r"(acc0) : "memory");
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tmem_d), "l"(dah), "l"(dbl), "r"(kInstrDesc), "r"(1u) : "memory");
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tmem_d), "l"(dah), "l"(dbh), "r"(kInstrDesc), "r"(1u) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(smem_u32(&bars[stage])) : "memory");
        }
    }
    // every product has completed when the last commit has arrived
    if (tiles > 0 && !failed) {
        const uint32_t last = tiles - 1;
        if (!wait_barrier(smem_u32(&bars[last & 1]), (last >> 1) & 1)) failed = 1;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool ok = !failed;
    if (!ok && threadIdx.x == 0) atomicOr(p.error, (unsigned)kStatusTensorWait);
    if (ok && tiles > 0 && c_early) {
#pragma unroll
        for (int u = 0; u < 128 / (TCT / 32); ++u) {
            const uint32_t r = warp + (TCT / 32) * u;
            if (r < out_rows) *reinterpret_cast<float4*>(&Ct[r][4 * lane]) = creg[u];
        }
        __syncthreads();
    } else if (ok && tiles > 0 && p.mode == 1) {   // C's tile, a warp a row
        for (uint32_t r = warp; r < out_rows; r += TCT / 32) {
            const float* src = out_tile + (size_t)r * p.ldo + 4 * lane;
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (out_vec) {
                f = *reinterpret_cast<const float4*>(src);
            } else {
                if (4 * lane + 0 < n_valid) f.x = src[0];
                if (4 * lane + 1 < n_valid) f.y = src[1];
                if (4 * lane + 2 < n_valid) f.z = src[2];
                if (4 * lane + 3 < n_valid) f.w = src[3];
            }
            *reinterpret_cast<float4*>(&Ct[r][4 * lane]) = f;
        }
        __syncthreads();
    }

    if (ok && tiles > 0) {
        // warp w reads lanes 32 (w % 4) .. + 31 (its rows of the tile), columns 64 (w / 4) .. + 63
        const uint32_t row = 32 * (warp & 3) + lane;
        const uint32_t c_base = 64 * (warp >> 2);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint32_t c0 = c_base + 32 * half;
            uint32_t v[32];
            const uint32_t taddr = tmem_d + ((32u * (warp & 3)) << 16) + c0;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                         "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                         "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                         : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                           "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                           "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                           "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                         : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (p.mode == 0) {          // the chunk's partial sums
#pragma unroll
                for (int c = 0; c < 32; ++c) Ct[row][c0 + c] = __uint_as_float(v[c]);
            } else {                    // C's tile minus the product
#pragma unroll
                for (int c = 0; c < 32; ++c) Ct[row][c0 + c] -= __uint_as_float(v[c]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (ok && tiles > 0) {              // rows of the tile to global memory, a warp a row, 16 bytes a lane
        for (uint32_t r = warp; r < out_rows; r += TCT / 32) {
            float* dst = out_tile + (size_t)r * p.ldo + 4 * lane;
            const float4 f = *reinterpret_cast<const float4*>(&Ct[r][4 * lane]);
            if (out_vec) {
                *reinterpret_cast<float4*>(dst) = f;
            } else {
                const float e[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (4 * lane + i < n_valid) dst[i] = e[i];
            }
        }
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" :: "r"(tmem_d) : "memory");
}

constexpr size_t kTcSmem = (2 * STAGE > 128 * CLD * (int)sizeof(float) ? 2 * STAGE : 128 * CLD * (int)sizeof(float)) + 1024;

void configure() {
    static PerDeviceOnce once;      // the opt-in is recorded per GPU
    if (const int device = current_device(); once.first(device)) {
        cuda_check(cudaFuncSetAttribute(tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem),
                   "tc_gemm shared memory");
        once.mark(device);
    }
}

} // namespace

// Zp[chunk][i][j] = sum over the chunk's rows of Y[r][i] C[r][j]; i < 128 (columns of Y from kw on as zero).
// Chunks of `chunk_rows` rows; Zp [chunks][128][ncp].
void launch_tc_ytc(cudaStream_t stream, const float* Y, size_t ldy, const float* C, size_t ldc, uint32_t mp, uint32_t kw,
                   uint32_t nc, float* zp, uint32_t ncp, uint32_t chunk_rows, unsigned* error) {
    configure();
    TcParams p{Y, C, zp, ldy, ldc, ncp, kw, nc, mp, chunk_rows, 0, error};
    const dim3 grid((nc + 127) / 128, (mp + chunk_rows - 1) / chunk_rows);
    launch_dependent(tc_gemm_kernel, grid, TCT, kTcSmem, stream, p);
    cuda_check(cudaGetLastError(), "tc_ytc launch");
}

// C[r][j] -= sum_k Y[r][k] Z[k][j], k < kw <= 128.
void launch_tc_yz(cudaStream_t stream, const float* Y, size_t ldy, const float* Z, uint32_t ncp, float* C, size_t ldc,
                  uint32_t mp, uint32_t kw, uint32_t nc, unsigned* error) {
    configure();
    TcParams p{Y, Z, C, ldy, ncp, ldc, mp, nc, kw, 0, 1, error};
    const dim3 grid((nc + 127) / 128, (mp + 127) / 128);
    launch_dependent(tc_gemm_kernel, grid, TCT, kTcSmem, stream, p);
    cuda_check(cudaGetLastError(), "tc_yz launch");
}

} // namespace mlb
