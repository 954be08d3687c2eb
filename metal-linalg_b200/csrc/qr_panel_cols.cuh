#pragma once
// Householder QR of a block of 8 * RW rows x 32 columns by one thread block of
// eight warps, a COLUMN per lane: warp w holds rows w * RW ... of every column,
// lane l column l, two rows to a 64-bit register (RW = 32 or 64 rows a lane).
//
// With a column per lane a reflector's dot products with the 32 columns are each
// lane's own packed FMAs; what a step needs across the block is one sum of eight
// partial products per lane, through shared memory and ONE barrier. (With a row
// per thread, the layout of factor_rows in qr_panel.cu, the same step reduces 32
// numbers per thread across the lanes first: 31 shuffles and selects a thread,
// which made a step four times as long.)
//
// Step j: lane j of every warp publishes its rows of column j to shared memory
// (warp 0, which holds the triangle, with zeros in the rows <= j); every lane
// reads them back as broadcast 16-byte words and takes the product with its own
// column; the block sums the eight partial products per column. Lane j's sum is
// the tail's sum of squares, so the norm costs nothing extra. Every warp forms the
// reflector for itself (unnormalised, H = I - g u u^T with u = (v1; tail), as in
// qr_small_steps.cuh) and updates the columns right of j. The columns left of j
// are not touched: below the diagonal they keep their reflector's tail, so their
// sums in later steps are the reflectors' products with one another, the Gram
// matrix that T is built from (slarft's recurrence).
//
// The step loops are not unrolled (a panel kernel runs on a few multiprocessors,
// once: unrolled, every instruction would be fetched from memory for a single
// use, and the fetches took longer than the arithmetic). Warp 0, which holds the
// triangle, keeps the pivot row at a constant register index by rotating its
// first rows (step_warp0 below); the other warps' steps do not depend on j at all.
//
// Afterwards: the block's first 32 rows in s.rows (R on and above the diagonal,
// the reflectors' tails, unnormalised, below it), the tails of the other rows in
// the registers, in `my_sc` of lane l the scale 1 / v1 that gives column l's
// reflector a unit diagonal (0 for a reflector that is the identity), s.taus,
// s.sc, s.G set.
#include "qr_small_steps.cuh"

namespace mlb {
namespace cols {

using namespace small;

constexpr int kWarps = 8;

struct Smem {
    float red[2][kWarps][32];    // each warp's partial products per column, by step parity
    float prow[2][32];           // the pivot row, by step parity
    float taus[32], sc[32];
    float G[32][33];             // G[k][j] = v_k^T v_j for k < j (unit-diagonal reflectors)
    float T[32][33];
    float rows[32][32];          // the block's first 32 rows as they finish: R, and the reflectors' tails below the diagonal
    // the two-column steps (factor_cols2): partial products with columns j and j + 1, and the two pivot rows, by pair parity
    float redp[2][kWarps][32], redq[2][kWarps][32];
    float prow0[2][32], prow1[2][32];
};

// 1 / x to an ulp or so (x normal)
__device__ __forceinline__ float recip(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r * fmaf(-x, r, 2.0f);
}

// The step barrier: the `threads` threads of the warps that hold rows, from wherever they are in
// the code (warp 0 runs a different loop from the others, so this is a named barrier, not
// __syncthreads()).
__device__ __forceinline__ void step_barrier(int threads) { asm volatile("bar.sync 1, %0;" :: "r"(threads) : "memory"); }

// How the partial products of a step become the sums over all rows.
//
// BlockSync: the rows are held by the first nw warps of ONE block: a named barrier, then every warp
// adds up the nw partial products.
struct BlockSync {
    int nw;
    __device__ __forceinline__ bool pivot(int warp) const { return warp == 0; }      // the warp that holds the triangle
    __device__ __forceinline__ bool leader(int warp) const { return warp == 0; }     // the warp that records tau, sc and G
    __device__ __forceinline__ void exchange(Smem& s, int buf, int lane, int warp) const {
        (void)s; (void)buf; (void)lane; (void)warp;
        step_barrier(32 * nw);
    }
    __device__ __forceinline__ float total(const Smem& s, int buf, int lane) const {
        float d = s.red[buf][0][lane];
        for (int w = 1; w < nw; ++w) d += s.red[buf][w][lane];
        return d;
    }
    // the same for the two sums of a two-column step
    __device__ __forceinline__ void exchange2(Smem& s, int buf, int lane, int warp) const {
        (void)s; (void)buf; (void)lane; (void)warp;
        step_barrier(32 * nw);
    }
    __device__ __forceinline__ void total2(const Smem& s, int buf, int lane, float& p, float& q) const {
        p = s.redp[buf][0][lane];
        q = s.redq[buf][0][lane];
        for (int w = 1; w < nw; ++w) {
            p += s.redp[buf][w][lane];
            q += s.redq[buf][w][lane];
        }
    }
};

// ClusterSync: the rows are held by the eight warps of each block of a thread-block CLUSTER (block
// `rank` of `ncta` holds rows rank * 8 RW ...). After the block's barrier every warp adds up the
// block's eight partial products and stores the sum into the shared memory of two of the blocks
// (distributed shared memory: mapa + st.shared::cluster); block 0 sends the pivot row along. One
// cluster barrier (a hardware barrier: arrive.release / wait.acquire) makes them visible, and every
// warp adds up the ncta block sums. The buffers alternate with the step's parity, and a block reads
// a step's sums before it arrives at the next step's cluster barrier, so nothing is overwritten early.
constexpr int kMaxCluster = 16;
struct ClusterShared {
    float cred[2][kMaxCluster][32];      // the blocks' sums, by step parity
    float credp[2][kMaxCluster][32], credq[2][kMaxCluster][32];      // and of the two-column steps, by pair parity
};
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a float into the same place of block `rank`'s shared memory
__device__ __forceinline__ void store_to_block(const float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(remote), "f"(v) : "memory");
}
// For the steps of FOUR columns a reduction (factor_cols4): each warp's four partial products per lane as one 16-byte
// word, the four pivot rows of every column, and the blocks' sums, all by quad parity.
struct QuadShared {
    float red4[2][kWarps][32][4];
    float prow4[2][32][4];
    float cred4[2][kMaxCluster][32][4];
    unsigned long long arrived[2];      // mbarriers, by quad parity: a quad's words have all arrived (ClusterSync::post)
};
__device__ __forceinline__ void store4_to_block(const float* local, uint32_t rank, float4 v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// The same store as an asynchronous one that counts its 16 bytes on the mbarrier at `bar` of the receiving block
__device__ __forceinline__ void post4_to_block(const float* local, const unsigned long long* bar, uint32_t rank, float4 v) {
    uint32_t remote, rbar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(rbar) : "r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];"
                 :: "r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(rbar) : "memory");
}
constexpr unsigned kPostPolls = 1u << 18;       // polls of a quad's mbarrier before the block gives up on it
struct ClusterSync {
    uint32_t       rank, ncta;
    ClusterShared* cs;
    QuadShared*    qs = nullptr;
    // post: a quad's sums travel as asynchronous stores that count their bytes on an mbarrier of the receiving block,
    // and every block waits on its own mbarrier instead of the cluster's barrier (whose round trip was a third of a
    // quad's time with sixteen blocks). A block sends quad q + 1 only after all its threads have read quad q, and
    // nobody sends quad q + 2 before it has that, so two buffers are enough. A wait that runs out sets `bad`.
    int            post = 0;
    unsigned*      bad = nullptr;
    // the mbarriers, before the cluster barrier that opens the kernel (one thread of the block)
    __device__ __forceinline__ static void init_posts(QuadShared* q) {
        for (int b = 0; b < 2; ++b)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"((uint32_t)__cvta_generic_to_shared(&q->arrived[b])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the four sums of a four-column step: the block's sums to every block (16 bytes a store), block 0's pivot rows along
    __device__ __forceinline__ void exchange4(int buf, int lane, int warp, int it) const {
        step_barrier(32 * kWarps);
        float4 d = *reinterpret_cast<const float4*>(qs->red4[buf][0][lane]);
#pragma unroll
        for (int w = 1; w < kWarps; ++w) {
            const float4 e = *reinterpret_cast<const float4*>(qs->red4[buf][w][lane]);
            d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
        }
        if (post) {
            const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&qs->arrived[buf]);
            if (warp == 0 && lane == 0) {      // what this block will receive: 512 bytes a block, and block 0's pivot rows
                const uint32_t bytes = ncta * 512u + (rank != 0 ? 512u : 0u);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
            }
            for (uint32_t r = warp; r < ncta; r += kWarps) {
                post4_to_block(qs->cred4[buf][rank][lane], &qs->arrived[buf], r, d);
                if (rank == 0 && r != 0)
                    post4_to_block(qs->prow4[buf][lane], &qs->arrived[buf], r, *reinterpret_cast<const float4*>(qs->prow4[buf][lane]));
            }
            const uint32_t parity = (uint32_t)(it >> 1) & 1u;
            uint32_t ok = 0;
            for (unsigned polls = 0; polls < kPostPolls && !ok; ++polls) {
                asm volatile("{\n\t.reg .pred p;\n\t"
                             "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                             "selp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
                // once a wait has run out somewhere, the others give up soon: the factorisation is lost already
                if (!ok && (polls & 1023u) == 1023u && bad && (*reinterpret_cast<volatile unsigned*>(bad) & 2u)) break;
            }
            if (!ok && bad && lane == 0) atomicOr(bad, 2u);      // kStatusTensorWait: the outputs become NaN, the status word says why
            return;
        }
        for (uint32_t r = warp; r < ncta; r += kWarps) {
            store4_to_block(qs->cred4[buf][rank][lane], r, d);
            if (rank == 0 && r != 0)
                store4_to_block(qs->prow4[buf][lane], r, *reinterpret_cast<const float4*>(qs->prow4[buf][lane]));
        }
        cluster_barrier();
    }
    __device__ __forceinline__ float4 total4(int buf, int lane) const {
        // every block's word asked for before the first is added (the loads of a loop over ncta would go one by one);
        // the order of the additions is the ranks' in every block
        float4 e[kMaxCluster];
#pragma unroll
        for (uint32_t r = 0; r < (uint32_t)kMaxCluster; ++r)
            e[r] = r < ncta ? *reinterpret_cast<const float4*>(qs->cred4[buf][r][lane]) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 d = e[0];
#pragma unroll
        for (uint32_t r = 1; r < (uint32_t)kMaxCluster; ++r) {
            if (r < ncta) { d.x += e[r].x; d.y += e[r].y; d.z += e[r].z; d.w += e[r].w; }
        }
        return d;
    }
    __device__ __forceinline__ bool pivot(int warp) const { return rank == 0 && warp == 0; }
    // every warp of the cluster holds the same sums: the one that records tau, sc and G (and builds T from them at the
    // end) is the last warp of the last block, which has no pivot rows to look after and none of R to write
    __device__ __forceinline__ bool leader(int warp) const { return rank + 1 == ncta && warp == kWarps - 1; }
    __device__ __forceinline__ void exchange(Smem& s, int buf, int lane, int warp) const {
        step_barrier(32 * kWarps);
        float d = s.red[buf][0][lane];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) d += s.red[buf][w][lane];
        for (uint32_t r = warp; r < ncta; r += kWarps) {
            store_to_block(&cs->cred[buf][rank][lane], r, d);
            if (rank == 0 && r != 0) store_to_block(&s.prow[buf][lane], r, s.prow[buf][lane]);
        }
        cluster_barrier();
    }
    __device__ __forceinline__ float total(const Smem& s, int buf, int lane) const {
        (void)s;
        float d = cs->cred[buf][0][lane];
        for (uint32_t r = 1; r < ncta; ++r) d += cs->cred[buf][r][lane];
        return d;
    }
    __device__ __forceinline__ void exchange2(Smem& s, int buf, int lane, int warp) const {
        step_barrier(32 * kWarps);
        float dp = s.redp[buf][0][lane], dq = s.redq[buf][0][lane];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) {
            dp += s.redp[buf][w][lane];
            dq += s.redq[buf][w][lane];
        }
        for (uint32_t r = warp; r < ncta; r += kWarps) {
            store_to_block(&cs->credp[buf][rank][lane], r, dp);
            store_to_block(&cs->credq[buf][rank][lane], r, dq);
            if (rank == 0 && r != 0) {
                store_to_block(&s.prow0[buf][lane], r, s.prow0[buf][lane]);
                store_to_block(&s.prow1[buf][lane], r, s.prow1[buf][lane]);
            }
        }
        cluster_barrier();
    }
    __device__ __forceinline__ void total2(const Smem& s, int buf, int lane, float& p, float& q) const {
        (void)s;
        p = cs->credp[buf][0][lane];
        q = cs->credq[buf][0][lane];
        for (uint32_t r = 1; r < ncta; ++r) {
            p += cs->credp[buf][r][lane];
            q += cs->credq[buf][r][lane];
        }
    }
};

// What every warp does after the step barrier: the block's sums, the reflector (the same numbers
// in every warp), the Gram entries and tau. Returns t, the coefficient of this lane's update
// (0 for the columns left of j, which keep their reflectors), and v1, alpha.
template <typename Sync>
__device__ __forceinline__ float step_reflector(Smem& s, int j, int buf, int lane, int warp, const Sync& sync,
                                                float& my_sc, float& v1, float& alpha) {
    const float d = sync.total(s, buf, lane);
    const float xj = s.prow[buf][lane];
    alpha = s.prow[buf][j];
    const float ss = __shfl_sync(0xffffffffu, d, j);
    float gneg;
    fast_reflector(alpha, ss, v1, gneg);
    const float sv  = fmaf(v1, xj, d);                    // u^T (this lane's column), u = (v1; tail)
    const float scj = gneg != 0.0f ? recip(v1) : 0.0f;
    if (sync.leader(warp)) {
        if (lane < j) s.G[lane][j] = sv * my_sc * scj;
        if (lane == 0) {
            s.taus[j] = -gneg * v1 * v1;
            s.sc[j]   = scj;
        }
    }
    if (lane == j) my_sc = scj;
    return lane > j ? sv * gneg : 0.0f;
}

// One step of warp 0, which holds the block's first rows. Its first 16 pairs of rows rotate: the
// pivot row is always in pair 0 (its low half in the even step P = 0, its high half in the odd
// one), and after the odd step the two finished rows leave for s.rows and the pairs move up one
// place (zeros come in at the end), so the step loop is not unrolled, every register index is a
// constant and the code stays small enough to be fetched once and run from the instruction cache.
template <int RW, int P, typename Sync>
__device__ __forceinline__ void step_warp0(pair_t (&x2)[RW / 2], Smem& s, ulonglong2* pj, int it, int lane,
                                           const Sync& sync, float& my_sc) {
    constexpr int NQ = RW / 4, NP = RW / 2;
    const int j = 2 * it + P, buf = P;
    const pair_t zero2 = pack(0.0f, 0.0f);
    if (lane == j) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            pair_t a = x2[2 * q], b = x2[2 * q + 1];
            if (q == 0) a = P == 0 ? pack(0.0f, hi_of(a)) : zero2;      // zeros in the rows up to the pivot's
            pj[q] = make_ulonglong2(a, b);
        }
    }
    __syncwarp();
    ulonglong2 u[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) u[q] = pj[q];
    {
        pair_t s2 = P == 0 ? mul2(u[0].x, x2[0]) : zero2, s2b = mul2(u[0].y, x2[1]);
#pragma unroll
        for (int q = 1; q < NQ; ++q) {
            s2  = fma2(u[q].x, x2[2 * q], s2);
            s2b = fma2(u[q].y, x2[2 * q + 1], s2b);
        }
        s.red[buf][0][lane] = hsum2(s2, s2b);
    }
    s.prow[buf][lane] = P == 0 ? lo_of(x2[0]) : hi_of(x2[0]);
    sync.exchange(s, buf, lane, 0);
    float v1, alpha;
    const float  t  = step_reflector(s, j, buf, lane, 0, sync, my_sc, v1, alpha);
    const pair_t t2 = pack(t, t);
    const pair_t w0 = P == 0 ? pack(v1, hi_of(u[0].x)) : pack(0.0f, v1);    // the reflector's first pair: v1 in the pivot's row
    pair_t head = fma2(t2, w0, x2[0]);
    if (lane == j) head = P == 0 ? pack(alpha - v1, hi_of(head)) : pack(lo_of(head), alpha - v1);   // the owner's pivot becomes beta
    if (P == 0) {
        x2[0] = head;
#pragma unroll
        for (int i = 1; i < NP; ++i) x2[i] = fma2(t2, (i & 1) ? u[i / 2].y : u[i / 2].x, x2[i]);
    } else {
        s.rows[2 * it][lane]     = lo_of(head);
        s.rows[2 * it + 1][lane] = hi_of(head);
#pragma unroll
        for (int i = 1; i < 16; ++i) x2[i - 1] = fma2(t2, (i & 1) ? u[i / 2].y : u[i / 2].x, x2[i]);
        x2[15] = zero2;
#pragma unroll
        for (int i = 16; i < NP; ++i) x2[i] = fma2(t2, (i & 1) ? u[i / 2].y : u[i / 2].x, x2[i]);
    }
}

// Keep: the other warps' published rows stay in shared memory, vector j's at keep + j * (8 RW) +
// (block row); else they go through `pub` like warp 0's (8 RW floats, reused every step).
// Afterwards: s.rows[r][c] holds the block's first 32 rows, R on and above the diagonal and the
// reflectors' tails below it; warp 0's rotating pairs are zero, its other rows (RW = 64) and every
// other warp's hold the tails of their rows; my_sc of lane l is s.sc[l].
// sync: BlockSync{nw} (the first nw warps of the block hold rows; the others do not take part and may
// not call) or ClusterSync (all eight warps of every block of the cluster).
template <int RW, bool Keep, typename Sync>
__device__ __forceinline__ void factor_cols(pair_t (&x2)[RW / 2], Smem& s, float* pub, float* keep, float& my_sc,
                                            const Sync& sync) {
    constexpr int NQ = RW / 4;           // 16-byte words of a warp's piece of a column
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    my_sc = 0.0f;
    if (sync.pivot(warp)) {
        ulonglong2* pj = reinterpret_cast<ulonglong2*>(pub);
#pragma unroll 1
        for (int it = 0; it < 16; ++it) {
            step_warp0<RW, 0>(x2, s, pj, it, lane, sync, my_sc);
            step_warp0<RW, 1>(x2, s, pj, it, lane, sync, my_sc);
        }
    } else {
#pragma unroll 1
        for (int j = 0; j < 32; ++j) {
            const int buf = j & 1;
            ulonglong2* pj = Keep ? reinterpret_cast<ulonglong2*>(keep + (size_t)j * kWarps * RW) + (size_t)warp * NQ
                                  : reinterpret_cast<ulonglong2*>(pub) + (size_t)warp * NQ;
            if (lane == j) {
#pragma unroll
                for (int q = 0; q < NQ; ++q) pj[q] = make_ulonglong2(x2[2 * q], x2[2 * q + 1]);
            }
            __syncwarp();
            ulonglong2 u[NQ];
#pragma unroll
            for (int q = 0; q < NQ; ++q) u[q] = pj[q];
            {
                pair_t s2 = mul2(u[0].x, x2[0]), s2b = mul2(u[0].y, x2[1]);
#pragma unroll
                for (int q = 1; q < NQ; ++q) {
                    s2  = fma2(u[q].x, x2[2 * q], s2);
                    s2b = fma2(u[q].y, x2[2 * q + 1], s2b);
                }
                s.red[buf][warp][lane] = hsum2(s2, s2b);
            }
            sync.exchange(s, buf, lane, warp);
            float v1, alpha;
            const float  t  = step_reflector(s, j, buf, lane, warp, sync, my_sc, v1, alpha);
            const pair_t t2 = pack(t, t);
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                x2[2 * q]     = fma2(t2, u[q].x, x2[2 * q]);
                x2[2 * q + 1] = fma2(t2, u[q].y, x2[2 * q + 1]);
            }
        }
    }
}

template <int RW, bool Keep>
__device__ __forceinline__ void factor_cols(pair_t (&x2)[RW / 2], Smem& s, float* pub, float* keep, float& my_sc,
                                            int nw = kWarps) {
    factor_cols<RW, Keep>(x2, s, pub, keep, my_sc, BlockSync{nw});
}

// One step of a warp that holds ordinary rows (the body of factor_cols' loop for such warps, without Keep).
template <int RW, typename Sync>
__device__ __forceinline__ void step_other(pair_t (&x2)[RW / 2], Smem& s, ulonglong2* pj, int j, int lane, int warp,
                                           const Sync& sync, float& my_sc) {
    constexpr int NQ = RW / 4;
    const int buf = j & 1;
    if (lane == j) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) pj[q] = make_ulonglong2(x2[2 * q], x2[2 * q + 1]);
    }
    __syncwarp();
    ulonglong2 u[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) u[q] = pj[q];
    {
        pair_t s2 = mul2(u[0].x, x2[0]), s2b = mul2(u[0].y, x2[1]);
#pragma unroll
        for (int q = 1; q < NQ; ++q) {
            s2  = fma2(u[q].x, x2[2 * q], s2);
            s2b = fma2(u[q].y, x2[2 * q + 1], s2b);
        }
        s.red[buf][warp][lane] = hsum2(s2, s2b);
    }
    sync.exchange(s, buf, lane, warp);
    float v1, alpha;
    const float  t  = step_reflector(s, j, buf, lane, warp, sync, my_sc, v1, alpha);
    const pair_t t2 = pack(t, t);
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        x2[2 * q]     = fma2(t2, u[q].x, x2[2 * q]);
        x2[2 * q + 1] = fma2(t2, u[q].y, x2[2 * q + 1]);
    }
}

// The same factorisation with TWO columns a reduction. Before the pair of steps (j, j + 1), lanes j and
// j + 1 publish their columns below the two pivot rows, every lane takes both products with its own
// column, and ONE exchange returns, per column k, p_k = a_j^T a_k and q_k = a_(j+1)^T a_k over the rows
// below the pair; the pivot rows j and j + 1 of every column go round with it. Step j is then what it always
// was. Step j + 1 acts on columns already changed by step j, a'_k = a_k + t_k u_j, and what it needs of
// them follows from the same sums: below the pair a'_(j+1)^T a'_k = q_k + t_k p_(j+1) + t_(j+1) p_k +
// t_(j+1) t_k p_j. Both reflectors are applied as one rank-2 update with the two published columns,
// a_k += (t_k + t'_k t_(j+1)) a_j + t'_k a_(j+1). A panel is a chain of exchanges (a barrier, or a
// cluster barrier, and the trips through shared memory around it); this halves the chain.
//
// The second column's norm comes out of that formula as a difference, q - (what step j removed): where
// step j removes nearly all of column j + 1 (the two columns nearly parallel below the diagonal) the
// difference loses digits, and the reflector built on it would not be orthogonal to rounding. So the pair
// is taken only where the updated norm keeps at least kPairKeep of the old one; otherwise step j is
// applied alone and step j + 1 runs as an ordinary step with an exchange of its own. Every thread decides
// alike: all of them hold the same sums.
constexpr float kPairKeep = 1.0f / 16.0f;

// KeepU: the two published columns stay in registers from the products to the update (4 * RW / 4 more registers) instead
// of being read from shared memory a second time; the path from shared memory is what bounds a step.
template <int RW, typename Sync, bool KeepU = false>
__device__ __forceinline__ void factor_cols2(pair_t (&x2)[RW / 2], Smem& s, float* pub, float& my_sc, const Sync& sync) {
    constexpr int NQ = RW / 4, NP = RW / 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool piv = sync.pivot(warp);
    const bool lead = sync.leader(warp);
    ulonglong2* pA = reinterpret_cast<ulonglong2*>(pub) + (size_t)warp * 2 * NQ;      // this warp's pieces of columns j and j + 1
    ulonglong2* pB = pA + NQ;
    const pair_t zero2 = pack(0.0f, 0.0f);
    my_sc = 0.0f;
#pragma unroll 1
    for (int it = 0; it < 16; ++it) {
        const int j = 2 * it, buf = it & 1;
        ulonglong2 ka[KeepU ? NQ : 1], kb[KeepU ? NQ : 1];
        // 1. columns j and j + 1 below the pivot pair (the pivot warp's pair 0 holds rows j and j + 1 themselves)
        if (lane == j || lane == j + 1) {
            ulonglong2* dst = lane == j ? pA : pB;
#pragma unroll
            for (int q = 0; q < NQ; ++q) dst[q] = make_ulonglong2((piv && q == 0) ? zero2 : x2[2 * q], x2[2 * q + 1]);
        }
        __syncwarp();
        // 2. both products with this lane's column
        {
            pair_t sa = zero2, sa2 = zero2, sb = zero2, sb2 = zero2;
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const ulonglong2 ua = pA[q], ub = pB[q];
                if (KeepU) {
                    ka[q] = ua;
                    kb[q] = ub;
                }
                sa  = fma2(ua.x, x2[2 * q], sa);
                sa2 = fma2(ua.y, x2[2 * q + 1], sa2);
                sb  = fma2(ub.x, x2[2 * q], sb);
                sb2 = fma2(ub.y, x2[2 * q + 1], sb2);
            }
            s.redp[buf][warp][lane] = hsum2(sa, sa2);
            s.redq[buf][warp][lane] = hsum2(sb, sb2);
        }
        if (piv) {
            s.prow0[buf][lane] = lo_of(x2[0]);
            s.prow1[buf][lane] = hi_of(x2[0]);
        }
        sync.exchange2(s, buf, lane, warp);
        float p, q;
        sync.total2(s, buf, lane, p, q);
        // 3. step j, and what step j + 1 will see
        const float r0 = s.prow0[buf][lane], r1 = s.prow1[buf][lane];              // rows j and j + 1 of this lane's column
        const float alpha = s.prow0[buf][j], e = s.prow1[buf][j];                  // column j's
        const float f0 = s.prow0[buf][j + 1], f1 = s.prow1[buf][j + 1];            // column j + 1's
        const float pj = __shfl_sync(0xffffffffu, p, j), pj1 = __shfl_sync(0xffffffffu, p, j + 1);
        const float qj1 = __shfl_sync(0xffffffffu, q, j + 1);
        float v1, gneg;
        fast_reflector(alpha, fmaf(e, e, pj), v1, gneg);
        const float sv  = fmaf(v1, r0, fmaf(e, r1, p));                            // u_j^T (this lane's column)
        const float tk  = lane > j ? sv * gneg : 0.0f;
        const float tj1 = fmaf(v1, f0, fmaf(e, f1, pj1)) * gneg;                   // column j + 1's coefficient, in every lane
        const float scj = gneg != 0.0f ? recip(v1) : 0.0f;
        if (lead) {
            if (lane < j) s.G[lane][j] = sv * my_sc * scj;
            if (lane == 0) {
                s.taus[j] = -gneg * v1 * v1;
                s.sc[j]   = scj;
            }
        }
        if (lane == j) my_sc = scj;
        const float m1 = fmaf(tk, e, r1);                                          // row j + 1 of this column after step j
        const float rj = lane > j ? fmaf(tk, v1, r0) : (lane == j ? alpha - v1 : r0);      // row j: final
        const float alpha1 = fmaf(tj1, e, f1);
        const float ss1 = fmaf(tj1, fmaf(tj1, pj, 2.0f * pj1), qj1);               // column j + 1's norm below the pair, after step j
        if (!(ss1 < kPairKeep * qj1)) {
            // 4a. step j + 1 from the same sums, and both reflectors in one update
            float v1b, gnegb;
            fast_reflector(alpha1, ss1, v1b, gnegb);
            const float s1  = fmaf(tj1 * tk, pj, fmaf(tj1, p, fmaf(tk, pj1, q)));  // a'_(j+1)^T a'_k below the pair
            const float sv1 = fmaf(v1b, m1, s1);
            const float t1  = lane > j + 1 ? sv1 * gnegb : 0.0f;
            const float scj1 = gnegb != 0.0f ? recip(v1b) : 0.0f;
            if (lead) {
                if (lane < j + 1) s.G[lane][j + 1] = sv1 * my_sc * scj1;
                if (lane == 0) {
                    s.taus[j + 1] = -gnegb * v1b * v1b;
                    s.sc[j + 1]   = scj1;
                }
            }
            if (lane == j + 1) my_sc = scj1;
            const float ca = fmaf(t1, tj1, tk);
            const pair_t a2 = pack(ca, ca), b2 = pack(t1, t1);
            if (piv) {
                const float rj1 = lane > j + 1 ? fmaf(t1, v1b, m1) : (lane == j + 1 ? alpha1 - v1b : m1);
                s.rows[j][lane]     = rj;
                s.rows[j + 1][lane] = rj1;
                // the pairs move up one place as the two finished rows leave
#pragma unroll
                for (int i = 1; i < 16; ++i) {
                    const ulonglong2 ua = KeepU ? ka[i / 2] : pA[i / 2], ub = KeepU ? kb[i / 2] : pB[i / 2];
                    x2[i - 1] = fma2(a2, (i & 1) ? ua.y : ua.x, fma2(b2, (i & 1) ? ub.y : ub.x, x2[i]));
                }
                x2[15] = zero2;
#pragma unroll
                for (int i = 16; i < NP; ++i) {
                    const ulonglong2 ua = KeepU ? ka[i / 2] : pA[i / 2], ub = KeepU ? kb[i / 2] : pB[i / 2];
                    x2[i] = fma2(a2, (i & 1) ? ua.y : ua.x, fma2(b2, (i & 1) ? ub.y : ub.x, x2[i]));
                }
            } else {
#pragma unroll
                for (int qq = 0; qq < NQ; ++qq) {
                    const ulonglong2 ua = KeepU ? ka[qq] : pA[qq], ub = KeepU ? kb[qq] : pB[qq];
                    x2[2 * qq]     = fma2(a2, ua.x, fma2(b2, ub.x, x2[2 * qq]));
                    x2[2 * qq + 1] = fma2(a2, ua.y, fma2(b2, ub.y, x2[2 * qq + 1]));
                }
            }
        } else {
            // 4b. step j alone; step j + 1 as an ordinary step with its own exchange
            const pair_t a2 = pack(tk, tk);
            if (piv) {
#pragma unroll
                for (int i = 1; i < NP; ++i) {
                    const ulonglong2 ua = KeepU ? ka[i / 2] : pA[i / 2];
                    x2[i] = fma2(a2, (i & 1) ? ua.y : ua.x, x2[i]);
                }
                x2[0] = pack(rj, m1);          // row j finished (it leaves with row j + 1), row j + 1 the next pivot row
                step_warp0<RW, 1>(x2, s, pA, it, lane, sync, my_sc);
            } else {
#pragma unroll
                for (int qq = 0; qq < NQ; ++qq) {
                    const ulonglong2 ua = KeepU ? ka[qq] : pA[qq];
                    x2[2 * qq]     = fma2(a2, ua.x, x2[2 * qq]);
                    x2[2 * qq + 1] = fma2(a2, ua.y, x2[2 * qq + 1]);
                }
                step_other<RW>(x2, s, pA, j + 1, lane, warp, sync, my_sc);
            }
        }
    }
}

// The same factorisation with FOUR columns a reduction. Lanes j .. j + 3 publish their columns below the four pivot
// rows (w_0 .. w_3), every lane takes the four products P_a = w_a^T y with its own column's tail y, and ONE exchange
// returns them together with the four pivot rows of every column. From then on a column's tail is y + sum_a c_a w_a
// with four coefficients c (all zero at first), and its entries in the four pivot rows are four numbers b, both held by
// every thread for its lane's column. Step s (column j + s, whose tail is sum_a d_a w_a, d = e_s + its c) needs only
//   its norm              d^T G d                       with G = the Gram matrix of the w's (the P's of lanes j .. j + 3)
//   its product with y'   d^T P + c^T (G d)             for every column
// and the pivot rows' part, which is explicit; it changes b and c, not the tails. After the four steps the tails take
// all four reflectors at once, y += sum_a c_a w_a. A panel is a chain of exchanges; this halves it again.
//
// As with two columns, a norm that comes out of the Gram matrix as a difference loses digits where the earlier steps
// of the group removed most of the column: a step is taken from the sums only where its tail keeps at least
// kQuadKeep of what it was; otherwise the tails are brought up to date with the steps done so far and the rest of the
// group runs as single steps with an exchange of their own. Every thread of the cluster decides alike.
constexpr float kQuadKeep = 1.0f / 16.0f;

template <int RW, typename Sync>
__device__ __forceinline__ void factor_cols4(pair_t (&x2)[RW / 2], Smem& s, float* pub4, float& my_sc, const Sync& sync) {
    constexpr int NQ = RW / 4, NP = RW / 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool piv = sync.pivot(warp), lead = sync.leader(warp);
    QuadShared& qs = *sync.qs;
    ulonglong2* pw = reinterpret_cast<ulonglong2*>(pub4) + (size_t)warp * 4 * NQ;      // this warp's pieces of w_0 .. w_3
    const pair_t zero2 = pack(0.0f, 0.0f);
    my_sc = 0.0f;
#pragma unroll 1
    for (int it = 0; it < 8; ++it) {
        const int j = 4 * it, buf = it & 1;
        // 1. the four columns below the pivot rows (the pivot warp's pairs 0 and 1 hold rows j .. j + 3 themselves)
        __syncwarp();
        if (lane >= j && lane < j + 4) {
            ulonglong2* dst = pw + (lane - j) * NQ;
#pragma unroll
            for (int q = 0; q < NQ; ++q)
                dst[q] = (piv && q == 0) ? make_ulonglong2(zero2, zero2) : make_ulonglong2(x2[2 * q], x2[2 * q + 1]);
        }
        __syncwarp();
        // 2. the four products with this lane's column
        {
            pair_t a0 = zero2, a1 = zero2, a2 = zero2, a3 = zero2, e0 = zero2, e1 = zero2, e2 = zero2, e3 = zero2;
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const ulonglong2 u0 = pw[q], u1 = pw[NQ + q], u2 = pw[2 * NQ + q], u3 = pw[3 * NQ + q];
                a0 = fma2(u0.x, x2[2 * q], a0); e0 = fma2(u0.y, x2[2 * q + 1], e0);
                a1 = fma2(u1.x, x2[2 * q], a1); e1 = fma2(u1.y, x2[2 * q + 1], e1);
                a2 = fma2(u2.x, x2[2 * q], a2); e2 = fma2(u2.y, x2[2 * q + 1], e2);
                a3 = fma2(u3.x, x2[2 * q], a3); e3 = fma2(u3.y, x2[2 * q + 1], e3);
            }
            *reinterpret_cast<float4*>(qs.red4[buf][warp][lane]) = make_float4(hsum2(a0, e0), hsum2(a1, e1), hsum2(a2, e2), hsum2(a3, e3));
        }
        if (piv) *reinterpret_cast<float4*>(qs.prow4[buf][lane]) = make_float4(lo_of(x2[0]), hi_of(x2[0]), lo_of(x2[1]), hi_of(x2[1]));
        sync.exchange4(buf, lane, warp, it);
        float P[4], b[4], c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        {
            const float4 t4 = sync.total4(buf, lane);
            P[0] = t4.x; P[1] = t4.y; P[2] = t4.z; P[3] = t4.w;
            const float4 b4 = *reinterpret_cast<const float4*>(qs.prow4[buf][lane]);
            b[0] = b4.x; b[1] = b4.y; b[2] = b4.z; b[3] = b4.w;
        }
        float G[4][4];      // G[a][k] = w_a^T w_k
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int k = a; k < 4; ++k) G[a][k] = G[k][a] = __shfl_sync(0xffffffffu, P[a], j + k);
        // 3. the four steps, from the sums
        int done = 4;
        static_for<4>([&](auto sc_) {
            constexpr int st = decltype(sc_)::value;
            if (done != 4) return;
            const int J = j + st;
            float d[4], bb[4], g[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) d[a] = __shfl_sync(0xffffffffu, c[a], J) + (a == st ? 1.0f : 0.0f);
#pragma unroll
            for (int r = st; r < 4; ++r) bb[r] = __shfl_sync(0xffffffffu, b[r], J);
            float vv = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                g[k] = fmaf(d[0], G[0][k], fmaf(d[1], G[1][k], fmaf(d[2], G[2][k], d[3] * G[3][k])));
                vv = fmaf(g[k], d[k], vv);
            }
            if (st > 0 && !(vv >= kQuadKeep * G[st][st])) {
                done = st;
                return;
            }
            const float alpha = bb[st];
            float ssum = fmaxf(vv, 0.0f);
#pragma unroll
            for (int r = st + 1; r < 4; ++r) ssum = fmaf(bb[r], bb[r], ssum);
            float v1, gneg;
            fast_reflector(alpha, ssum, v1, gneg);
            float dot = v1 * b[st];
#pragma unroll
            for (int r = st + 1; r < 4; ++r) dot = fmaf(bb[r], b[r], dot);
#pragma unroll
            for (int a = 0; a < 4; ++a) dot = fmaf(d[a], P[a], fmaf(c[a], g[a], dot));
            const float t   = lane > J ? dot * gneg : 0.0f;
            const float scj = gneg != 0.0f ? recip(v1) : 0.0f;
            if (lead) {
                if (lane < J) s.G[lane][J] = dot * my_sc * scj;
                if (lane == 0) {
                    s.taus[J] = -gneg * v1 * v1;
                    s.sc[J]   = scj;
                }
            }
            if (lane == J) my_sc = scj;
            b[st] = lane > J ? fmaf(t, v1, b[st]) : (lane == J ? alpha - v1 : b[st]);
#pragma unroll
            for (int r = st + 1; r < 4; ++r) b[r] = fmaf(t, bb[r], b[r]);
#pragma unroll
            for (int a = 0; a < 4; ++a) c[a] = fmaf(t, d[a], c[a]);
        });
        // 4. the tails take the steps done: y += sum_a c_a w_a (zeros were published for the pivot rows)
        {
            const pair_t c0 = pack(c[0], c[0]), c1 = pack(c[1], c[1]), c2 = pack(c[2], c[2]), c3 = pack(c[3], c[3]);
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const ulonglong2 u0 = pw[q], u1 = pw[NQ + q], u2 = pw[2 * NQ + q], u3 = pw[3 * NQ + q];
                x2[2 * q]     = fma2(c0, u0.x, fma2(c1, u1.x, fma2(c2, u2.x, fma2(c3, u3.x, x2[2 * q]))));
                x2[2 * q + 1] = fma2(c0, u0.y, fma2(c1, u1.y, fma2(c2, u2.y, fma2(c3, u3.y, x2[2 * q + 1]))));
            }
        }
        // 5. what is left of the group as single steps, each with its own exchange
        if (done != 4) {
            static_for<3>([&](auto sc_) {
                constexpr int st = decltype(sc_)::value + 1;
                if (st < done) return;
                const int J = j + st, sb = st & 1;
                __syncwarp();
                if (lane == J) {
#pragma unroll
                    for (int q = 0; q < NQ; ++q)
                        pw[q] = (piv && q == 0) ? make_ulonglong2(zero2, zero2) : make_ulonglong2(x2[2 * q], x2[2 * q + 1]);
                }
                __syncwarp();
                {
                    pair_t a0 = zero2, e0 = zero2;
#pragma unroll
                    for (int q = 0; q < NQ; ++q) {
                        const ulonglong2 u0 = pw[q];
                        a0 = fma2(u0.x, x2[2 * q], a0);
                        e0 = fma2(u0.y, x2[2 * q + 1], e0);
                    }
                    s.red[sb][warp][lane] = hsum2(a0, e0);
                }
                if (piv) s.prow[sb][lane] = 0.0f;      // the exchange sends it along; the pivot rows are in b here
                sync.exchange(s, sb, lane, warp);
                const float p = sync.total(s, sb, lane);
                float bb[4];
#pragma unroll
                for (int r = st; r < 4; ++r) bb[r] = __shfl_sync(0xffffffffu, b[r], J);
                const float alpha = bb[st];
                float ssum = __shfl_sync(0xffffffffu, p, J);
#pragma unroll
                for (int r = st + 1; r < 4; ++r) ssum = fmaf(bb[r], bb[r], ssum);
                float v1, gneg;
                fast_reflector(alpha, ssum, v1, gneg);
                float dot = fmaf(v1, b[st], p);
#pragma unroll
                for (int r = st + 1; r < 4; ++r) dot = fmaf(bb[r], b[r], dot);
                const float t   = lane > J ? dot * gneg : 0.0f;
                const float scj = gneg != 0.0f ? recip(v1) : 0.0f;
                if (lead) {
                    if (lane < J) s.G[lane][J] = dot * my_sc * scj;
                    if (lane == 0) {
                        s.taus[J] = -gneg * v1 * v1;
                        s.sc[J]   = scj;
                    }
                }
                if (lane == J) my_sc = scj;
                b[st] = lane > J ? fmaf(t, v1, b[st]) : (lane == J ? alpha - v1 : b[st]);
#pragma unroll
                for (int r = st + 1; r < 4; ++r) b[r] = fmaf(t, bb[r], b[r]);
                const pair_t t2 = pack(t, t);
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    const ulonglong2 u0 = pw[q];
                    x2[2 * q]     = fma2(t2, u0.x, x2[2 * q]);
                    x2[2 * q + 1] = fma2(t2, u0.y, x2[2 * q + 1]);
                }
            });
        }
        // 6. the four finished rows leave; the pivot warp's pairs move up two places
        if (piv) {
#pragma unroll
            for (int r = 0; r < 4; ++r) s.rows[j + r][lane] = b[r];
#pragma unroll
            for (int i = 2; i < 16; ++i) x2[i - 2] = x2[i];
            x2[14] = zero2;
            x2[15] = zero2;
        }
    }
}

// T from s.G and s.taus (slarft's forward recurrence) by one warp, a row of T per lane, to
// T[i * ldt + j].
__device__ __forceinline__ void build_t_to(const Smem& s, float* T, int ldt) {
    const int i = threadIdx.x & 31;
    float tr[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const float tau = s.taus[j];
        float a = 0.0f;
#pragma unroll
        for (int k = 0; k < j; ++k) a = fmaf(tr[k], s.G[k][j], a);
        tr[j] = i < j ? -tau * a : (i == j ? tau : 0.0f);
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) T[i * ldt + j] = tr[j];
}

// row r of this lane's column
template <int RW>
__device__ __forceinline__ float row_of(const pair_t (&x2)[RW / 2], int r) {
    return (r & 1) ? hi_of(x2[r / 2]) : lo_of(x2[r / 2]);
}

} // namespace cols
} // namespace mlb
