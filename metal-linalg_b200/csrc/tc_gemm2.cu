// C -= Y Z on tcgen05 tensor cores by 3xTF32, with BOTH operands split once, ahead of the
// product, into hi and lo tf32 parts laid out in global memory exactly as the tensor core reads
// them from shared memory, so that a stage of the product is two bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier) and six tcgen05.mma, with no thread touching
// an operand. It takes the wide trailing updates and Q accumulations of the blocked QR from
// tc_gemm.cu's kernel, in which every thread loads, splits and stores operand words at every
// stage (the tensor pipe was 14 % busy there): Y is reused by every column tile of the update and
// Z by every row tile, so splitting them once saves that work (mp / 128) and (nc / 128) times over.
//
//   split_y_kernel   Y (mp x kw, kw <= 128) -> ysp[row tile][k stage][hi | lo], a (row tile, stage)
//                    being 128 rows x 16 columns of Y: 8 KB hi then 8 KB lo, K-major unswizzled
//                    canonical layout (16-byte words of four K values; eight rows 128 bytes apart;
//                    the four words of a stage 2 KB apart)
//   split_z_kernel   Z (128 x nc) -> zsp[column tile][k stage][hi | lo], the same with N = column
//   tc_yz2_kernel    a block per 128 x 128 tile of C: one elected thread streams the stages through
//                    three shared-memory slots (bulk copies ahead, products behind, tcgen05.commit
//                    frees a slot), the accumulator in 128 columns of tensor memory; then the whole
//                    block reads it back (tcgen05.ld) and subtracts it from C's tile through shared
//                    memory, whole rows to global memory.
//
//   split_yt_kernel  Y -> ytsp[16-row stage][hi | lo] with M = column of Y, K = row: the A operand of Y^T C
//   tc_ytc2_kernel   Zp[chunk] = Y^T C over a chunk of rows: A by bulk copies from ytsp (a ring of three
//                    slots), B = C's rows split by the block's threads as they are loaded (C changes with
//                    every update, so there is nothing to split ahead), two stages
//
// Every mbarrier wait is bounded; a wait that runs out sets the error word (the matrix's outputs
// become NaN) and the block leaves without touching C.
#include "common.cuh"
#include "kernels.h"
#include "tc_split.cuh"

#include <cstdlib>

namespace mlb {

namespace {

constexpr int      T2     = 256;                  // threads
constexpr int      KS2    = tcsplit::kStageK;     // K values a stage
constexpr int      TILE2  = tcsplit::kTileBytes;  // bytes of a 128 x 16 tf32 operand tile (8 KB)
constexpr int      HALF2  = 2 * TILE2;            // hi and lo of one operand
constexpr int      STAGE2 = 2 * HALF2;            // A hi, A lo, B hi, B lo (32 KB)
constexpr int      NS2    = 3;                    // stages in flight
constexpr int      LBO2   = tcsplit::kLbo;        // bytes between the 16-byte K words of a tile
constexpr int      SBO2   = tcsplit::kSbo;        // bytes between groups of eight rows
constexpr int      CLD2   = 132;                  // leading dimension of C's tile in shared memory
constexpr uint32_t kSpin2 = 1u << 22;
constexpr uint32_t kPairFloats = tcsplit::kPairFloats;       // floats of a (tile, stage): hi then lo
using tcsplit::split4;
using tcsplit::word_offset;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc2(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (((uint32_t)(LBO2 >> 4) & 0x3FFFu) << 16);
    const uint32_t hi = ((uint32_t)(SBO2 >> 4) & 0x3FFFu) | (1u << 14);   // version 1 (Blackwell), no swizzle
    return ((uint64_t)hi << 32) | lo;
}
// kind::tf32, float32 accumulator, A and B K-major, M = 128, N = 128
constexpr uint32_t kInstrDesc2 = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ bool wait_barrier2(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpin2; ++spin) {
        uint32_t done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// A thread a word: row r of Y, columns 4 q ... 4 q + 3. Rows from mp on and columns from kw on are zero.
__global__ void __launch_bounds__(256) split_y_kernel(const float* __restrict__ Y, size_t ldy, uint32_t mp, uint32_t kw,
                                                      uint32_t stages, float* __restrict__ ysp) {
    dependency_wait_only();
    const uint32_t idx = blockIdx.x * 256 + threadIdx.x;
    const uint32_t q = idx % (4 * stages), r = idx / (4 * stages);
    const uint32_t tiles = (mp + 127) / 128;
    if (r >= tiles * 128) return;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (r < mp && 4 * q + i < kw) ? Y[(size_t)r * ldy + 4 * q + i] : 0.0f;
    float4 hi, lo;
    split4(v, hi, lo);
    float* dst = ysp + ((size_t)(r / 128) * stages + q / 4) * kPairFloats + word_offset(r % 128, q % 4);
    *reinterpret_cast<float4*>(dst) = hi;
    *reinterpret_cast<float4*>(dst + TILE2 / 4) = lo;
}

// A thread a word: column n of Z, rows 4 q ... 4 q + 3. Columns from nc on and rows from kw on are zero.
__global__ void __launch_bounds__(256) split_z_kernel(const float* __restrict__ Z, size_t ldz, uint32_t kw, uint32_t nc,
                                                      uint32_t stages, float* __restrict__ zsp) {
    dependency_wait_only();
    const uint32_t tiles = (nc + 127) / 128;
    const uint32_t idx = blockIdx.x * 256 + threadIdx.x;
    const uint32_t n = idx % (tiles * 128), q = idx / (tiles * 128);       // lanes along n: coalesced reads of Z's rows
    if (q >= 4 * stages) return;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (n < nc && 4 * q + i < kw) ? Z[(size_t)(4 * q + i) * ldz + n] : 0.0f;
    float4 hi, lo;
    split4(v, hi, lo);
    float* dst = zsp + ((size_t)(n / 128) * stages + q / 4) * kPairFloats + word_offset(n % 128, q % 4);
    *reinterpret_cast<float4*>(dst) = hi;
    *reinterpret_cast<float4*>(dst + TILE2 / 4) = lo;
}

struct Yz2Params {
    const float* ysp;
    const float* zsp;
    float*       c;
    size_t       ldc;
    uint32_t     mp, nc, stages;
    unsigned*    error;
};

__global__ void __launch_bounds__(T2, 2) tc_yz2_kernel(const Yz2Params p) {
    dependency_wait_only();
    extern __shared__ __align__(1024) char smem[];
    __shared__ __align__(8) unsigned long long full[NS2], freed[NS2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ct = blockIdx.x, rt = blockIdx.y, j0 = ct * 128, r0 = rt * 128;
    if (threadIdx.x == 0) failed = *reinterpret_cast<volatile unsigned*>(p.error) != 0;
    __syncthreads();
    if (failed) return;   // an earlier block or launch gave up: do nothing (the same answer for the whole block)

    const uint32_t n_valid = min(p.nc - j0, 128u), out_rows = min(p.mp - r0, 128u), stages = p.stages;
    float (*Ct)[CLD2] = reinterpret_cast<float (*)[CLD2]>(smem);      // takes the slots' place once the products are done
    float* out_tile = p.c + (size_t)r0 * p.ldc + j0;
    const bool out_vec = (p.ldc & 3) == 0 && (reinterpret_cast<size_t>(out_tile) & 15) == 0 && n_valid == 128;

    // C's tile is needed only after the products (its place in shared memory is the slots'), but it is fetched
    // now, into registers, a warp a row and 16 bytes a lane, sixteen rows a warp all in flight: the loads
    // complete while one thread issues the products, and the epilogue starts with the tile at hand. (Read row by
    // row after the products, every row waited for L2: a third of a block's life.) A tile that cannot be read
    // by whole aligned words is asked into L2 instead and read after the products, entry by entry.
    float4 creg[128 / (T2 / 32)];
    if (out_vec) {
#pragma unroll
        for (int u = 0; u < 128 / (T2 / 32); ++u) {
            const uint32_t r = warp + (T2 / 32) * u;
            creg[u] = r < out_rows ? *reinterpret_cast<const float4*>(out_tile + (size_t)r * p.ldc + 4 * lane)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else if (threadIdx.x / 2 < out_rows) {
        const float* line = out_tile + (size_t)(threadIdx.x / 2) * p.ldc + 64 * (threadIdx.x & 1);
        if (64 * (threadIdx.x & 1) < n_valid) {
            asm volatile("prefetch.global.L2 [%0];" :: "l"(line));
            if (64 * (threadIdx.x & 1) + 32 < n_valid) asm volatile("prefetch.global.L2 [%0];" :: "l"(line + 32));
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS2; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&freed[s])));
        }
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

    if (threadIdx.x == 0) {
        const float* ya = p.ysp + (size_t)rt * stages * kPairFloats;
        const float* zb = p.zsp + (size_t)ct * stages * kPairFloats;
        auto request = [&](uint32_t s) {      // stage s into its slot: Y's hi and lo, Z's hi and lo
            const uint32_t slot = s % NS2, base = smem_u32(smem + slot * STAGE2), bar = smem_u32(&full[slot]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"((uint32_t)STAGE2) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         :: "r"(base), "l"(ya + (size_t)s * kPairFloats), "r"((uint32_t)HALF2), "r"(bar) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         :: "r"(base + HALF2), "l"(zb + (size_t)s * kPairFloats), "r"((uint32_t)HALF2), "r"(bar) : "memory");
        };
        int bad = 0;
        for (uint32_t s = 0; s < stages && s < (uint32_t)NS2; ++s) request(s);
        for (uint32_t s = 0; s < stages && !bad; ++s) {
            const uint32_t slot = s % NS2, parity = (s / NS2) & 1;
            if (!wait_barrier2(smem_u32(&full[slot]), parity)) { bad = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(smem + slot * STAGE2), a_lo = a_hi + TILE2, b_hi = a_hi + HALF2, b_lo = b_hi + TILE2;
#pragma unroll
            for (int h = 0; h < KS2 / 8; ++h) {
                const uint32_t koff = h * 2 * LBO2;             // two 16-byte words of K an instruction
                const uint64_t dah = make_desc2(a_hi + koff), dal = make_desc2(a_lo + koff);
                const uint64_t dbh = make_desc2(b_hi + koff), dbl = make_desc2(b_lo + koff);
                const uint32_t acc0 = (s > 0 || h > 0) ? 1u : 0u;
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tmem_d), "l"(dal), "l"(dbh), "r"(kInstrDesc2), "r"(acc0) : "memory");
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tmem_d), "l"(dah), "l"(dbl), "r"(kInstrDesc2), "r"(1u) : "memory");
                asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                             " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                             :: "r"(tmem_d), "l"(dah), "l"(dbh), "r"(kInstrDesc2), "r"(1u) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(smem_u32(&freed[slot])) : "memory");
            if (s + NS2 < stages) {       // the slot is free when these products have completed: the stage after next
                if (!wait_barrier2(smem_u32(&freed[slot]), parity)) { bad = 1; break; }
                request(s + NS2);
            }
        }
        if (bad) failed = 1;
    }
    // every product has completed when the last commit has arrived
    if (stages > 0) {
        const uint32_t last = stages - 1;
        if (!wait_barrier2(smem_u32(&freed[last % NS2]), (last / NS2) & 1)) failed = 1;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool ok = !failed;
    if (!ok && threadIdx.x == 0) atomicOr(p.error, (unsigned)kStatusTensorWait);
    if (ok) {
        // The product's tile from tensor memory into shared memory: warp w reads lanes 32 (w % 4) .. + 31 (its rows of the
        // tile), columns 64 (w / 4) .. + 63, a row per lane, and stores 16-byte words (rows 528 bytes apart: the eight
        // lanes of a quarter-warp fall into eight different groups of four banks). Entry by entry, subtracting in place,
        // every access collided four ways.
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
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4*>(&Ct[row][c0 + 4 * q]) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (ok) {              // C's rows minus the product's, to global memory, a warp a row, 16 bytes a lane
        if (out_vec) {
#pragma unroll
            for (int u = 0; u < 128 / (T2 / 32); ++u) {
                const uint32_t r = warp + (T2 / 32) * u;
                if (r < out_rows) {
                    const float4 f = *reinterpret_cast<const float4*>(&Ct[r][4 * lane]);
                    *reinterpret_cast<float4*>(out_tile + (size_t)r * p.ldc + 4 * lane) =
                        make_float4(creg[u].x - f.x, creg[u].y - f.y, creg[u].z - f.z, creg[u].w - f.w);
                }
            }
        } else {
            for (uint32_t r = warp; r < out_rows; r += T2 / 32) {
                float* dst = out_tile + (size_t)r * p.ldc + 4 * lane;
                const float4 f = *reinterpret_cast<const float4*>(&Ct[r][4 * lane]);
                const float e[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (4 * lane + i < n_valid) dst[i] -= e[i];
            }
        }
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" :: "r"(tmem_d) : "memory");
}


// The same product on TWO column tiles a block (128 x 256 of C): a stage is Y's tile and both of Z's, so Y's tile is
// fetched once for the two (three quarters of the operand bytes of two single-tile blocks), the prologue (barriers,
// tensor memory) is paid once, and the accumulators are two runs of 128 columns of tensor memory. Two slots of 48 KB.
constexpr int NSP    = 2;                     // slots of the pair kernel
constexpr int STAGEP = 3 * HALF2;             // Y hi, lo; Z hi, lo of the first tile; of the second (48 KB)

__global__ void __launch_bounds__(T2, 2) tc_yz2_pair_kernel(const Yz2Params p) {
    dependency_wait_only();
    extern __shared__ __align__(1024) char smem[];
    __shared__ __align__(8) unsigned long long full[NSP], freed[NSP];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ct = 2 * blockIdx.x, rt = blockIdx.y, j0 = ct * 128, r0 = rt * 128;
    const bool two = j0 + 128 < p.nc;            // the second column tile exists
    if (threadIdx.x == 0) failed = *reinterpret_cast<volatile unsigned*>(p.error) != 0;
    __syncthreads();
    if (failed) return;   // an earlier block or launch gave up: do nothing (the same answer for the whole block)

    const uint32_t out_rows = min(p.mp - r0, 128u), stages = p.stages;
    float (*Ct)[CLD2] = reinterpret_cast<float (*)[CLD2]>(smem);      // takes the slots' place once the products are done
    float* out_tile = p.c + (size_t)r0 * p.ldc + j0;
    const bool aligned = (p.ldc & 3) == 0 && (reinterpret_cast<size_t>(out_tile) & 15) == 0;
    const uint32_t n_valid0 = min(p.nc - j0, 128u), n_valid1 = two ? min(p.nc - j0 - 128, 128u) : 0u;

    // The first tile of C into registers now (a warp a row, 16 bytes a lane, sixteen rows a warp in flight); the second
    // is asked into L2 and read when the first has gone out.
    float4 creg[128 / (T2 / 32)];
    if (aligned && n_valid0 == 128) {
#pragma unroll
        for (int u = 0; u < 128 / (T2 / 32); ++u) {
            const uint32_t r = warp + (T2 / 32) * u;
            creg[u] = r < out_rows ? *reinterpret_cast<const float4*>(out_tile + (size_t)r * p.ldc + 4 * lane)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (threadIdx.x / 2 < out_rows) {
        const float* line = out_tile + (size_t)(threadIdx.x / 2) * p.ldc + 128 + 64 * (threadIdx.x & 1);
        if (64 * (threadIdx.x & 1) < n_valid1) {
            asm volatile("prefetch.global.L2 [%0];" :: "l"(line));
            if (64 * (threadIdx.x & 1) + 32 < n_valid1) asm volatile("prefetch.global.L2 [%0];" :: "l"(line + 32));
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSP; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&freed[s])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {            // 2 x 128 columns of tensor memory for the two 128 x 128 float32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" :: "r"(smem_u32(&tmem_base_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    if (threadIdx.x == 0) {
        const float* ya = p.ysp + (size_t)rt * stages * kPairFloats;
        const float* zb = p.zsp + (size_t)ct * stages * kPairFloats;
        const float* zb1 = zb + (size_t)stages * kPairFloats;
        const uint32_t stage_bytes = two ? (uint32_t)STAGEP : (uint32_t)(2 * HALF2);
        auto request = [&](uint32_t s) {      // stage s into its slot: Y's hi and lo, Z's hi and lo of each tile
            const uint32_t slot = s % NSP, base = smem_u32(smem + slot * STAGEP), bar = smem_u32(&full[slot]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(stage_bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         :: "r"(base), "l"(ya + (size_t)s * kPairFloats), "r"((uint32_t)HALF2), "r"(bar) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         :: "r"(base + HALF2), "l"(zb + (size_t)s * kPairFloats), "r"((uint32_t)HALF2), "r"(bar) : "memory");
            if (two)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             :: "r"(base + 2 * HALF2), "l"(zb1 + (size_t)s * kPairFloats), "r"((uint32_t)HALF2), "r"(bar) : "memory");
        };
        int bad = 0;
        for (uint32_t s = 0; s < stages && s < (uint32_t)NSP; ++s) request(s);
        for (uint32_t s = 0; s < stages && !bad; ++s) {
            const uint32_t slot = s % NSP, parity = (s / NSP) & 1;
            if (!wait_barrier2(smem_u32(&full[slot]), parity)) { bad = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = smem_u32(smem + slot * STAGEP), a_lo = a_hi + TILE2;
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                if (tile == 1 && !two) break;
                const uint32_t b_hi = a_hi + (1 + tile) * HALF2, b_lo = b_hi + TILE2, tmem_acc = tmem_d + 128u * tile;
#pragma unroll
                for (int h = 0; h < KS2 / 8; ++h) {
                    const uint32_t koff = h * 2 * LBO2;             // two 16-byte words of K an instruction
                    const uint64_t dah = make_desc2(a_hi + koff), dal = make_desc2(a_lo + koff);
                    const uint64_t dbh = make_desc2(b_hi + koff), dbl = make_desc2(b_lo + koff);
                    const uint32_t acc0 = (s > 0 || h > 0) ? 1u : 0u;
                    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                 " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                                 :: "r"(tmem_acc), "l"(dal), "l"(dbh), "r"(kInstrDesc2), "r"(acc0) : "memory");
                    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                 " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                                 :: "r"(tmem_acc), "l"(dah), "l"(dbl), "r"(kInstrDesc2), "r"(1u) : "memory");
                    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                 " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                                 :: "r"(tmem_acc), "l"(dah), "l"(dbh), "r"(kInstrDesc2), "r"(1u) : "memory");
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(smem_u32(&freed[slot])) : "memory");
            if (s + NSP < stages) {       // the slot is free when these products have completed
                if (!wait_barrier2(smem_u32(&freed[slot]), parity)) { bad = 1; break; }
                request(s + NSP);
            }
        }
        if (bad) failed = 1;
    }
    // every product has completed when the last commit has arrived
    if (stages > 0) {
        const uint32_t last = stages - 1;
        if (!wait_barrier2(smem_u32(&freed[last % NSP]), (last / NSP) & 1)) failed = 1;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool ok = !failed;
    if (!ok && threadIdx.x == 0) atomicOr(p.error, (unsigned)kStatusTensorWait);
#pragma unroll 1
    for (int tile = 0; tile < 2; ++tile) {
        if (tile == 1 && !two) break;
        const uint32_t n_valid = tile ? n_valid1 : n_valid0;
        float* out = out_tile + 128 * tile;
        const bool out_vec = aligned && n_valid == 128;
        if (tile == 1 && out_vec) {        // the second tile of C, asked into L2 at the start
#pragma unroll
            for (int u = 0; u < 128 / (T2 / 32); ++u) {
                const uint32_t r = warp + (T2 / 32) * u;
                creg[u] = r < out_rows ? *reinterpret_cast<const float4*>(out + (size_t)r * p.ldc + 4 * lane)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        if (ok) {      // the product's tile from tensor memory into shared memory, a row per lane, 16-byte stores
            const uint32_t row = 32 * (warp & 3) + lane;
            const uint32_t c_base = 64 * (warp >> 2);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint32_t c0 = c_base + 32 * half;
                uint32_t v[32];
                const uint32_t taddr = tmem_d + 128u * tile + ((32u * (warp & 3)) << 16) + c0;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                               "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                               "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                               "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                             : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    *reinterpret_cast<uint4*>(&Ct[row][c0 + 4 * q]) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (ok) {              // C's rows minus the product's, to global memory, a warp a row, 16 bytes a lane
            if (out_vec) {
#pragma unroll
                for (int u = 0; u < 128 / (T2 / 32); ++u) {
                    const uint32_t r = warp + (T2 / 32) * u;
                    if (r < out_rows) {
                        const float4 f = *reinterpret_cast<const float4*>(&Ct[r][4 * lane]);
                        *reinterpret_cast<float4*>(out + (size_t)r * p.ldc + 4 * lane) =
                            make_float4(creg[u].x - f.x, creg[u].y - f.y, creg[u].z - f.z, creg[u].w - f.w);
                    }
                }
            } else {
                for (uint32_t r = warp; r < out_rows; r += T2 / 32) {
                    float* dst = out + (size_t)r * p.ldc + 4 * lane;
                    const float4 f = *reinterpret_cast<const float4*>(&Ct[r][4 * lane]);
                    const float e[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (4 * lane + i < n_valid) dst[i] -= e[i];
                }
            }
        }
        __syncthreads();      // the tile in shared memory has been read: the second may take its place
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" :: "r"(tmem_d) : "memory");
}

// ---------------------------------------------------------------------------
// Zp[chunk][i][j] = sum over the chunk's rows r of Y[r][i] C[r][j]
// ---------------------------------------------------------------------------
// A thread a word: column c of Y, rows 4 q ... 4 q + 3 (lanes along c: coalesced reads of Y's rows).
__global__ void __launch_bounds__(256) split_yt_kernel(const float* __restrict__ Y, size_t ldy, uint32_t mp, uint32_t kw,
                                                       float* __restrict__ ytsp) {
    dependency_wait_only();
    const uint32_t idx = blockIdx.x * 256 + threadIdx.x;
    const uint32_t c = idx & 127, q = idx >> 7;               // q: group of four rows
    if (q >= 4 * ((mp + 15) / 16)) return;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (4 * q + i < mp && c < kw) ? Y[(size_t)(4 * q + i) * ldy + c] : 0.0f;
    float4 hi, lo;
    split4(v, hi, lo);
    float* dst = ytsp + (size_t)(q / 4) * kPairFloats + word_offset(c, q % 4);
    *reinterpret_cast<float4*>(dst) = hi;
    *reinterpret_cast<float4*>(dst + TILE2 / 4) = lo;
}

// Both splits of Y in one launch (the two products of an update need one each): the first blocks_t blocks do
// split_yt_kernel's work, the rest split_y_kernel's.
__global__ void __launch_bounds__(256) split_y_both_kernel(const float* __restrict__ Y, size_t ldy, uint32_t mp, uint32_t kw,
                                                           uint32_t stages, float* __restrict__ ysp, float* __restrict__ ytsp,
                                                           uint32_t blocks_t) {
    dependency_wait_only();
    float v[4];
    if (blockIdx.x < blocks_t) {
        const uint32_t idx = blockIdx.x * 256 + threadIdx.x;
        const uint32_t c = idx & 127, q = idx >> 7;               // q: group of four rows
        if (q >= 4 * ((mp + 15) / 16)) return;
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = (4 * q + i < mp && c < kw) ? Y[(size_t)(4 * q + i) * ldy + c] : 0.0f;
        float4 hi, lo;
        split4(v, hi, lo);
        float* dst = ytsp + (size_t)(q / 4) * kPairFloats + word_offset(c, q % 4);
        *reinterpret_cast<float4*>(dst) = hi;
        *reinterpret_cast<float4*>(dst + TILE2 / 4) = lo;
    } else {
        const uint32_t idx = (blockIdx.x - blocks_t) * 256 + threadIdx.x;
        const uint32_t q = idx % (4 * stages), r = idx / (4 * stages);
        if (r >= (mp + 127) / 128 * 128) return;
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = (r < mp && 4 * q + i < kw) ? Y[(size_t)r * ldy + 4 * q + i] : 0.0f;
        tcsplit::store_word(ysp, stages, r, q, v);
    }
}

// B tiles written by threads: padded one word per K column so that the stores do not collide
constexpr int LBOB  = 16 * 128 + 16;
constexpr int TILEB = (KS2 / 4) * LBOB;           // bytes of one 128 x 16 thread-written tile
constexpr int NA2   = 3;                          // slots of A
constexpr int BOFF  = NA2 * HALF2;                // B's two stages follow A's ring
constexpr size_t kYtc2Smem = (size_t)BOFF + 2 * 2 * TILEB + 1024 > 128 * CLD2 * sizeof(float) + 1024
                                 ? (size_t)BOFF + 2 * 2 * TILEB + 1024 : 128 * CLD2 * sizeof(float) + 1024;

__device__ __forceinline__ uint64_t make_desc_b(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (((uint32_t)(LBOB >> 4) & 0x3FFFu) << 16);
    const uint32_t hi = ((uint32_t)(SBO2 >> 4) & 0x3FFFu) | (1u << 14);
    return ((uint64_t)hi << 32) | lo;
}

struct Ytc2Params {
    const float* ytsp;     // Y^T split, a (hi | lo) pair per 16 rows of Y
    const float* c;
    float*       zp;       // [chunks][128][ncp]
    size_t       ldc;
    uint32_t     mp, nc, ncp, chunk_rows;
    uint32_t     sub_tiles;      // 16-row tiles per accumulator: the chunk's first sub_tiles tiles go to the first, the rest to the second
    unsigned*    error;
};

__global__ void __launch_bounds__(T2, 2) tc_ytc2_kernel(const Ytc2Params p) {
    dependency_wait_only();
    extern __shared__ __align__(1024) char smem[];
    __shared__ __align__(8) unsigned long long fullA[NA2], freed[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t j0 = blockIdx.x * 128, chunk = blockIdx.y;
    if (threadIdx.x == 0) failed = *reinterpret_cast<volatile unsigned*>(p.error) != 0;
    __syncthreads();
    if (failed) return;

    const uint32_t k_begin = chunk * p.chunk_rows, k_end = min(p.mp, k_begin + p.chunk_rows);
    const uint32_t k_len = k_end - k_begin, tiles = (k_len + KS2 - 1) / KS2;
    const uint32_t n_valid = min(p.nc - j0, 128u);
    const float* b_src = p.c + (size_t)k_begin * p.ldc + j0;
    const float* a_src = p.ytsp + (size_t)(k_begin / KS2) * kPairFloats;
    float (*Ct)[CLD2] = reinterpret_cast<float (*)[CLD2]>(smem);
    float* out_tile = p.zp + (size_t)chunk * 128 * p.ncp + j0;
    const bool out_vec = (p.ncp & 3) == 0 && (reinterpret_cast<size_t>(out_tile) & 15) == 0 && n_valid == 128;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NA2; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&fullA[s])));
        for (int s = 0; s < 2; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&freed[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        // two accumulators of 128 columns: a chunk's rows are summed in two halves (the tensor core accumulates with
        // truncation, so a chain is kept to sub_tiles tiles) and the halves are added once, in the epilogue
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" :: "r"(smem_u32(&tmem_base_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    auto request_a = [&](uint32_t kt) {       // thread 0: Y^T's hi and lo of tile kt into its slot of the ring
        const uint32_t slot = kt % NA2, bar = smem_u32(&fullA[slot]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"((uint32_t)HALF2) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(smem_u32(smem + slot * HALF2)), "l"(a_src + (size_t)kt * kPairFloats), "r"((uint32_t)HALF2), "r"(bar)
                     : "memory");
    };
    // C's rows of a tile: lanes along the columns (coalesced), four rows a thread and word
    float rb[8];
    auto fetch_b = [&](uint32_t kt) {
        const uint32_t k0 = kt * KS2, kv = min(k_len - k0, (uint32_t)KS2);
        const uint32_t n = threadIdx.x & 127;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t kq = (threadIdx.x >> 7) + 2 * e;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t k = 4 * kq + i;
                rb[4 * e + i] = (n < n_valid && k < kv) ? b_src[(size_t)(k0 + k) * p.ldc + n] : 0.0f;
            }
        }
    };
    auto put_b = [&](char* hi_tile, char* lo_tile) {
        const uint32_t n = threadIdx.x & 127;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const uint32_t kq = (threadIdx.x >> 7) + 2 * e;
            const float v[4] = {rb[4 * e], rb[4 * e + 1], rb[4 * e + 2], rb[4 * e + 3]};
            float4 hi, lo;
            split4(v, hi, lo);
            const uint32_t off = kq * LBOB + (n >> 3) * SBO2 + (n & 7) * 16;
            *reinterpret_cast<float4*>(hi_tile + off) = hi;
            *reinterpret_cast<float4*>(lo_tile + off) = lo;
        }
    };

    if (threadIdx.x == 0) {
        if (tiles > 0) request_a(0);
        if (tiles > 1) request_a(1);
    }
    if (tiles > 0) fetch_b(0);
    for (uint32_t kt = 0; kt < tiles; ++kt) {
        const int stage = kt & 1;
        char* bbase = smem + BOFF + stage * 2 * TILEB;
        // B's stage, and A's slot of tile kt + 1, are free once the products of tile kt - 2 have completed
        if (kt >= 2 && !failed) {
            if (!wait_barrier2(smem_u32(&freed[stage]), ((kt >> 1) - 1) & 1)) failed = 1;
        }
        if (threadIdx.x == 0 && kt >= 1 && kt + 1 < tiles && !failed) request_a(kt + 1);
        put_b(bbase, bbase + TILEB);
        if (kt + 1 < tiles) fetch_b(kt + 1);                           // in flight while the tensor core works
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the writes above, visible to the tensor core
        __syncthreads();
        if (threadIdx.x == 0 && !failed) {
            if (!wait_barrier2(smem_u32(&fullA[kt % NA2]), (kt / NA2) & 1)) {
                failed = 1;
            } else {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_hi = smem_u32(smem + (kt % NA2) * HALF2), a_lo = a_hi + TILE2;
                const uint32_t b_hi = smem_u32(bbase), b_lo = b_hi + TILEB;
#pragma unroll
                for (int h = 0; h < KS2 / 8; ++h) {
                    const uint64_t dah = make_desc2(a_hi + h * 2 * LBO2), dal = make_desc2(a_lo + h * 2 * LBO2);
                    const uint64_t dbh = make_desc_b(b_hi + h * 2 * LBOB), dbl = make_desc_b(b_lo + h * 2 * LBOB);
                    const bool second = kt >= p.sub_tiles;
                    const uint32_t tmem_acc = tmem_d + (second ? 128u : 0u);
                    const uint32_t acc0 = ((second ? kt - p.sub_tiles : kt) > 0 || h > 0) ? 1u : 0u;
                    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                 " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                                 :: "r"(tmem_acc), "l"(dal), "l"(dbh), "r"(kInstrDesc2), "r"(acc0) : "memory");
                    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                 " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                                 :: "r"(tmem_acc), "l"(dah), "l"(dbl), "r"(kInstrDesc2), "r"(1u) : "memory");
                    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                                 " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
                                 :: "r"(tmem_acc), "l"(dah), "l"(dbh), "r"(kInstrDesc2), "r"(1u) : "memory");
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                         :: "r"(smem_u32(&freed[stage])) : "memory");
        }
    }
    if (tiles > 0 && !failed) {
        const uint32_t last = tiles - 1;
        if (!wait_barrier2(smem_u32(&freed[last & 1]), (last >> 1) & 1)) failed = 1;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool ok = !failed;
    if (!ok && threadIdx.x == 0) atomicOr(p.error, (unsigned)kStatusTensorWait);
    if (ok && tiles > 0) {
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
            if (tiles > p.sub_tiles) {      // the second half's sums
                uint32_t w[32];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                             : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]),
                               "=r"(w[8]), "=r"(w[9]), "=r"(w[10]), "=r"(w[11]), "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15]),
                               "=r"(w[16]), "=r"(w[17]), "=r"(w[18]), "=r"(w[19]), "=r"(w[20]), "=r"(w[21]), "=r"(w[22]), "=r"(w[23]),
                               "=r"(w[24]), "=r"(w[25]), "=r"(w[26]), "=r"(w[27]), "=r"(w[28]), "=r"(w[29]), "=r"(w[30]), "=r"(w[31])
                             : "r"(taddr + 128u) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(w[c]));
            }
#pragma unroll
            for (int q = 0; q < 8; ++q)      // 16-byte words: entry by entry the lanes' rows collide four ways
                *reinterpret_cast<uint4*>(&Ct[row][c0 + 4 * q]) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (ok) {              // the chunk's 128 rows of partial sums to global memory (zeros for an empty chunk)
        for (uint32_t r = warp; r < 128; r += T2 / 32) {
            float* dst = out_tile + (size_t)r * p.ncp + 4 * lane;
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tiles > 0) f = *reinterpret_cast<const float4*>(&Ct[r][4 * lane]);
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
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" :: "r"(tmem_d) : "memory");
}

constexpr size_t kYz2Smem = (size_t)NS2 * STAGE2 + 1024;
constexpr size_t kYz2PairSmem = (size_t)NSP * STAGEP + 1024;

} // namespace

size_t tc_split_floats(uint32_t extent) { return (size_t)((extent + 127) / 128) * 8 * kPairFloats; }

// C[r][j] -= sum_k Y[r][k] Z[k][j], k < kw <= 128, with Y and Z split first into ysp and zsp (scratch
// of tc_split_floats(mp) and tc_split_floats(nc) floats). Z null: zsp holds Z's split already (its
// producer wrote it: tc_split.cuh), for the stages of kw; Y null: ysp holds Y's (launch_tc_ytc_split made it).
void launch_tc_yz_split(cudaStream_t stream, const float* Y, size_t ldy, const float* Z, uint32_t ncp, float* C, size_t ldc,
                        uint32_t mp, uint32_t kw, uint32_t nc, float* ysp, float* zsp, unsigned* error) {
    static PerDeviceOnce once;      // the opt-in is recorded per GPU
    if (const int device = current_device(); once.first(device)) {
        cuda_check(cudaFuncSetAttribute(tc_yz2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kYz2Smem),
                   "tc_yz2 shared memory");
        cuda_check(cudaFuncSetAttribute(tc_yz2_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kYz2PairSmem),
                   "tc_yz2_pair shared memory");
        once.mark(device);
    }
    const uint32_t stages = (kw + KS2 - 1) / KS2, rtiles = (mp + 127) / 128, ctiles = (nc + 127) / 128;
    if (Y) launch_dependent(split_y_kernel, (rtiles * 128 * 4 * stages + 255) / 256, 256, 0, stream, Y, ldy, mp, kw, stages, ysp);
    if (Z) launch_dependent(split_z_kernel, (ctiles * 128 * 4 * stages + 255) / 256, 256, 0, stream, Z, (size_t)ncp, kw, nc, stages, zsp);
    Yz2Params p{ysp, zsp, C, ldc, mp, nc, stages, error};
    // two column tiles a block where that still leaves two waves of blocks (QR_TC_YZ_PAIR=0/1: never / always)
    const char* pair_env = std::getenv("QR_TC_YZ_PAIR");
    const bool pair = pair_env ? pair_env[0] != '0' : (uint64_t)((ctiles + 1) / 2) * rtiles >= 4 * 148;
    if (pair) launch_dependent(tc_yz2_pair_kernel, dim3((ctiles + 1) / 2, rtiles), T2, kYz2PairSmem, stream, p);
    else launch_dependent(tc_yz2_kernel, dim3(ctiles, rtiles), T2, kYz2Smem, stream, p);
    cuda_check(cudaGetLastError(), "tc_yz2 launch");
}

size_t tc_split_t_floats(uint32_t rows) { return (size_t)((rows + 15) / 16) * kPairFloats; }

// Zp[chunk][i][j] = sum over the chunk's rows of Y[r][i] C[r][j] with Y^T split first into ytsp
// (tc_split_t_floats(mp) floats); chunk_rows a multiple of 16, at most twice sub_rows (a multiple of 16 too): a block
// sums its chunk's first sub_rows rows in one accumulator of tensor memory, the rest in a second, and adds the two.
void launch_tc_ytc_split(cudaStream_t stream, const float* Y, size_t ldy, const float* C, size_t ldc, uint32_t mp,
                         uint32_t kw, uint32_t nc, float* zp, uint32_t ncp, uint32_t chunk_rows, uint32_t sub_rows, float* ytsp,
                         unsigned* error, float* ysp) {
    static PerDeviceOnce once;
    if (const int device = current_device(); once.first(device)) {
        cuda_check(cudaFuncSetAttribute(tc_ytc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kYtc2Smem),
                   "tc_ytc2 shared memory");
        once.mark(device);
    }
    const uint32_t words = 128 * 4 * ((mp + 15) / 16), blocks_t = (words + 255) / 256;
    if (ysp) {      // the second product's split of Y in the same launch
        const uint32_t stages = (kw + KS2 - 1) / KS2, rtiles = (mp + 127) / 128;
        launch_dependent(split_y_both_kernel, blocks_t + (rtiles * 128 * 4 * stages + 255) / 256, 256, 0, stream, Y, ldy, mp, kw,
                         stages, ysp, ytsp, blocks_t);
    } else {
        launch_dependent(split_yt_kernel, blocks_t, 256, 0, stream, Y, ldy, mp, kw, ytsp);
    }
    Ytc2Params p{ytsp, C, zp, ldc, mp, nc, ncp, chunk_rows, sub_rows / KS2, error};
    launch_dependent(tc_ytc2_kernel, dim3((nc + 127) / 128, (mp + chunk_rows - 1) / chunk_rows), T2, kYtc2Smem, stream, p);
    cuda_check(cudaGetLastError(), "tc_ytc2 launch");
}

} // namespace mlb
