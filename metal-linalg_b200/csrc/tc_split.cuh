#pragma once
// The layout of an operand of the 3xTF32 products split once into hi and lo tf32 parts (tc_gemm2.cu): per (128-wide
// tile, 16-deep K stage) 8 KB of hi then 8 KB of lo, K-major unswizzled canonical layout (16-byte words of four K
// values; eight rows 128 bytes apart; the four words of a stage 2 KB apart). Shared by the kernels that read it
// (tc_gemm2.cu) and those that write it as they produce the operand (qr_blocked.cu's reduce_t_wide_kernel).
#include <cuda_runtime.h>

#include <cstdint>

namespace mlb {
namespace tcsplit {

constexpr int      kStageK     = 16;                    // K values a stage
constexpr int      kTileBytes  = 128 * kStageK * 4;     // bytes of a 128 x 16 tf32 operand tile (8 KB)
constexpr int      kLbo        = 128 * 16;              // bytes between the 16-byte K words of a tile
constexpr int      kSbo        = 128;                   // bytes between groups of eight rows
constexpr uint32_t kPairFloats = 2 * kTileBytes / 4;    // floats of a (tile, stage): hi then lo

__device__ __forceinline__ void split4(const float (&v)[4], float4& hi, float4& lo) {
    float h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t b;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(b) : "f"(v[i]));
        h[i] = __uint_as_float(b);
        l[i] = v[i] - h[i];
    }
    hi = make_float4(h[0], h[1], h[2], h[3]);
    lo = make_float4(l[0], l[1], l[2], l[3]);
}
// float offset of the word (mn, four K values from 4 * kq) inside a (tile, stage)'s hi part
__device__ __forceinline__ uint32_t word_offset(uint32_t mn, uint32_t kq) {
    return kq * (kLbo / 4) + (mn >> 3) * (kSbo / 4) + (mn & 7) * 4;
}
// v = four consecutive K values (from 4 * q) of row or column mn of an operand of `stages` stages: split and stored
__device__ __forceinline__ void store_word(float* sp, uint32_t stages, uint32_t mn, uint32_t q, const float (&v)[4]) {
    float4 hi, lo;
    split4(v, hi, lo);
    float* dst = sp + ((size_t)(mn / 128) * stages + q / 4) * kPairFloats + word_offset(mn % 128, q % 4);
    *reinterpret_cast<float4*>(dst) = hi;
    *reinterpret_cast<float4*>(dst + kTileBytes / 4) = lo;
}

} // namespace tcsplit
} // namespace mlb
