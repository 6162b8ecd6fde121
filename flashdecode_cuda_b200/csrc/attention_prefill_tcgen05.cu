// Prompt attention on the 5th-generation tensor cores (head size 128, bfloat16):
// causal, grouped-query, paged, variable lengths, optional window, continuing a
// cached prefix.  A CTA takes 256 consecutive query tokens of one sequence and
// one query head as two query tiles of 128 rows, and walks the keys in tiles of
// 64 that both query tiles share (each is fetched once):
//
//   S[128 q, 64 keys] = Q K^T      tcgen05.mma, both operands K-major in shared memory,
//                                  accumulator S in tensor memory (per query tile two buffers
//                                  of 64 columns: the next scores are computed while the
//                                  softmax works on these)
//   softmax                        4 warps per query tile, one thread per query row:
//                                  tcgen05.ld of its S row, running max / sum in float (base
//                                  2), P written to shared memory as bfloat16 in the
//                                  128-byte-swizzled K-major layout
//   O[128 q, 128 d] += P V         tcgen05.mma with V as an MN-major operand (V rows are keys,
//                                  the head dimension is contiguous), accumulator O in tensor
//                                  memory (128 columns per query tile), rescaled in place when
//                                  a row's maximum grew by more than 2^8
//
// The two query tiles run the same steps out of phase: while one's softmax warps
// are in their exp phase (bound by the special-function units), the other's are
// waiting, packing or storing, and the tensor cores serve both.  All 512 columns
// of tensor memory are in use (2 x 2 x 64 for S, 2 x 128 for O).
//
// Keys and values come straight from the paged pools by TMA: one 2-D box of
// (block_size keys x 64 dims) per cache block and half head, placed so that a
// tile of 64 keys forms the canonical swizzled layout; three tiles are in
// flight (four in the short-prompt form below).  Roles: warp 0 issues TMA (the copies of a tile from as many lanes at
// once, the block numbers fetched 32 at a time ahead of use), warp 1 issues
// Q K^T and owns the tensor-memory allocation, warps 2-9 do the softmax and the
// epilogue, warp 10 issues P V.  Every mbarrier wait is bounded in time; a wait
// that runs out sets a status bit and the CTA winds down (see gemm_tcgen05.cu).
//
// CTAs start in the order of their work: the head is the grid's fastest index
// and the query tiles run from the last (most keys) to the first, over all
// heads, so no long tile starts in a late wave.  A prompt so short that this
// grid leaves SMs empty runs a second form of the kernel (SPLIT below): 128
// queries per CTA, their key tiles dealt to the two groups of softmax warps.
#include <cuda.h>
#include <math.h>

#include <map>
#include <mutex>
#include <tuple>

#include "attention.cuh"
#include "tcgen05.cuh"        // g_tc_wait_ns, g_tc_skip_last: the limit of the bounded waits and the tests' hook

namespace fd {

constexpr int TA_D = 128;                 // head size
constexpr int TA_BM = 128;                // queries per query tile (the M of the MMAs)
constexpr int TA_BN = 64;                 // keys per tile
constexpr int TA_STAGES = 3;              // key/value tiles in flight
constexpr int TA_NQ = 2;                  // query tiles per CTA
constexpr int TA_ROWS = TA_NQ * TA_BM;    // queries per CTA
constexpr int TA_PV_WARP = 2 + 4 * TA_NQ;  // warps: 0 TMA, 1 issuer of Q K^T, 2-9 softmax (four per query tile), 10 issuer of P V
constexpr int TA_THREADS = (TA_PV_WARP + 1) * 32;
constexpr int TA_QSLAB = TA_BM * 128;     // bytes of a [128 queries][64 bf16] slab (Q: two of them; P: one)
constexpr int TA_KSLAB = TA_BN * 128;     // bytes of a [64 keys][64 bf16] slab (K and V: two each)
constexpr int TA_QTILE = 2 * TA_QSLAB;    // Q [128][128]
constexpr int TA_PTILE = TA_QSLAB;        // P [128][64]
constexpr int TA_KTILE = 2 * TA_KSLAB;    // K or V [64][128]
// 192 KB + barriers, one CTA per SM: two query tiles (Q 32 KB and P 16 KB each) and three key/value tiles
// in flight (32 KB each); with one query tile per CTA (see the kernel), one Q and four key/value tiles
constexpr int TA_SMEM = TA_NQ * (TA_QTILE + TA_PTILE) + TA_STAGES * 2 * TA_KTILE + 256;

__device__ __forceinline__ uint32_t ta_saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long ta_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool ta_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                        unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t spins = 0;; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((spins & 63) != 63) continue;                    // the clock and the flag only now and then
        if (*abort_flag) return false;
        if (t0 == 0) t0 = ta_ns();
        else if (ta_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            set_status(status, STATUS_WAIT_TIMEOUT);
            return false;
        }
    }
}
__device__ __forceinline__ void ta_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ta_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ta_tma(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void ta_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ta_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void ta_ld32(uint32_t taddr, uint32_t v[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void ta_st32(uint32_t taddr, const uint32_t v[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

// K-major operand, rows of 128 bytes, 128-byte swizzle: 8-row groups 1024 bytes apart.
// 2^x by the special function unit (two units in the last place; 2^-inf = 0)
__device__ __forceinline__ float ta_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint64_t ta_desc_k(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (rows are the contraction index, 64 contiguous elements of the N side per
// 128-byte row, 128-byte swizzle): slabs of 64 N-elements `slab_bytes` apart (leading offset),
// 8-row groups along K 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t ta_desc_mn(uint32_t addr, uint32_t slab_bytes) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(slab_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// SPLIT: the CTA takes 128 query tokens only, and its two groups of softmax warps work on the SAME query tile:
// the first on the even key tiles of its range, the second on the odd ones, each with its own running maximum,
// sum and O; at the end the second group hands its state over through shared memory and the first adds the two
// up.  A query tile's chain of key tiles - what bounds the time of a short prompt, whose few CTAs do not fill
// the GPU - is half as long this way; every key tile is then used by one group only, which a long prompt pays
// for in shared-memory and L2 traffic, so the launcher picks this form only while the other leaves SMs idle.
template <bool SPLIT>
__global__ void __launch_bounds__(TA_THREADS, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const AttnParams p,
                            const unsigned long long wait_ns, const int skip_last) {
    // SPLIT: one copy of the one query tile, and the 32 KB that saves as a fourth key/value tile in flight
    constexpr int STAGES = SPLIT ? TA_STAGES + 1 : TA_STAGES;
    constexpr int NQB = SPLIT ? 1 : TA_NQ;
    static_assert(NQB * TA_QTILE + TA_NQ * TA_PTILE + STAGES * 2 * TA_KTILE + 256 <= TA_SMEM, "shared memory layout");
    static_assert(STAGES * 2 * TA_KTILE >= (TA_D + 2) * TA_BM * 4, "the ring takes the second group's O, maxima and sums");
    extern __shared__ __align__(1024) unsigned char ta_raw[];
    unsigned char* q_s = ta_raw;                             // per query tile: [2 slabs][128 q][64 d]
    unsigned char* p_s = q_s + NQB * TA_QTILE;             // per query tile: [128 q][64 keys]
    unsigned char* kv_s = p_s + TA_NQ * TA_PTILE;            // per stage: K [2 slabs][64 keys][64 d], V the same
    uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + STAGES * 2 * TA_KTILE);
    // bars: [0] q_full, kv_full[S], kv_empty[S]; per query tile: s_full[2], s_free[2], p_ready, o_done
    uint64_t* kv_full = bars + 1;
    uint64_t* kv_empty = kv_full + STAGES;
    uint64_t* s_full = kv_empty + STAGES;                 // [qt][2]
    uint64_t* s_free = s_full + 2 * TA_NQ;                   // [qt][2]
    uint64_t* p_ready = s_free + 2 * TA_NQ;                  // [qt]
    uint64_t* o_done = p_ready + TA_NQ;                      // [qt]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + TA_NQ);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The head is the fastest grid index and the query tiles run from the last to the first: CTAs start in the
    // order of their work (a causal tile's key range grows with its position), the longest of every head
    // first, and the heads of a group walk the same keys at the same time.
    const int tile = gridDim.y - 1 - blockIdx.y, h = blockIdx.x, b = blockIdx.z;
    const int slot = p.row_slot[b];
    const int q_len = slot >= 0 ? p.row_q_len[b] : 0;
    constexpr int CTA_ROWS = SPLIT ? TA_BM : TA_ROWS;        // query tokens of a CTA
    if (tile * CTA_ROWS >= q_len) return;                    // uniform for the CTA; nothing allocated yet
    if ((ta_saddr(ta_raw) & 1023u) != 0) {                   // the swizzled tiles need a 1024-byte-aligned base
        if (threadIdx.x == 0) set_status(p.status, STATUS_WAIT_TIMEOUT);
        return;
    }
    const int ctx = p.row_ctx_len[b];
    const int tok0 = p.row_q_start[b] + tile * CTA_ROWS;     // first token of the CTA
    const int kvh = h / p.G;
    const int bs = p.block_size;
    // The CTA's two query tiles (128 rows each; the second may be empty) share every key tile.  Of the key
    // tiles t_begin + 64 it, it = 0 .. n_tiles - 1, query tile qt takes it_lo[qt] .. it_hi[qt] - 1: causality
    // ends the first tile's range two key tiles early, a window starts the second's two key tiles late.
    int nq[TA_NQ], p_first[TA_NQ], q_lo[TA_NQ], q_hi[TA_NQ], it_lo[TA_NQ], it_hi[TA_NQ];
#pragma unroll
    for (int qt = 0; qt < TA_NQ; ++qt) {
        const int first = tile * CTA_ROWS + (SPLIT ? 0 : qt * TA_BM);   // the group's first query in the step
        nq[qt] = max(0, min(TA_BM, q_len - first));
        p_first[qt] = ctx + first;
        q_hi[qt] = p_first[qt] + nq[qt];
        q_lo[qt] = p.window > 0 ? max(0, p_first[qt] - p.window + 1) : 0;
    }
    const int lo = q_lo[0];
    const int hi = !SPLIT && nq[1] > 0 ? q_hi[1] : q_hi[0];
    const int t_begin = (lo / TA_BN) * TA_BN;
    const int n_tiles = (hi - t_begin + TA_BN - 1) / TA_BN;
#pragma unroll
    for (int qt = 0; qt < TA_NQ; ++qt) {
        it_lo[qt] = (q_lo[qt] / TA_BN * TA_BN - t_begin) / TA_BN;
        it_hi[qt] = nq[qt] > 0 ? (q_hi[qt] - t_begin + TA_BN - 1) / TA_BN : it_lo[qt];
    }
    // whether group qt works on key tile `it`, and which of its own tiles (0, 1, ...) that is
    auto mine = [&](int qt, int it, int& j) -> bool {
        if (it < it_lo[qt] || it >= it_hi[qt]) return false;
        j = it - it_lo[qt];
        if (SPLIT) {
            if ((j & 1) != qt) return false;
            j >>= 1;
        }
        return true;
    };

    if (threadIdx.x == 0) {
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        auto init = [](uint64_t* bar, int count) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ta_saddr(bar)), "r"(count) : "memory");
        };
        init(&bars[0], 1);
        for (int s = 0; s < STAGES; ++s) { init(&kv_full[s], 1); init(&kv_empty[s], 1); }
        for (int i = 0; i < 2 * TA_NQ; ++i) { init(&s_full[i], 1); init(&s_free[i], 128); }   // s_free, p_ready: every softmax thread arrives
        for (int qt = 0; qt < TA_NQ; ++qt) { init(&p_ready[qt], 128); init(&o_done[qt], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ta_saddr(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // columns: S of query tile qt, buffer j at 128 qt + 64 j; O of query tile qt at 256 + 128 qt
    const uint32_t tmem_s = tmem, tmem_o = tmem + 256;

    if (warp == 0) {
        // ---- TMA producer: the warp's lanes fetch the block numbers of the
        // next 32 copies together, one chunk ahead, so that no copy waits for a table entry ----
        if (lane == 0) {
            // rows beyond the last token of the step are zero-filled; rows of a following sequence are computed and dropped
            ta_expect(ta_saddr(&bars[0]), NQB * TA_QTILE);
#pragma unroll
            for (int qt = 0; qt < NQB; ++qt) {
                const int row = tok0 + qt * TA_BM;
                ta_tma(ta_saddr(q_s + qt * TA_QTILE), &map_q, ta_saddr(&bars[0]), h * TA_D, row);
                ta_tma(ta_saddr(q_s + qt * TA_QTILE + TA_QSLAB), &map_q, ta_saddr(&bars[0]), h * TA_D + 64, row);
            }
        }
        const int first_col = lo / bs;                        // blocks behind a window may have been given back
        const int last_col = (hi - 1) / bs;                   // last block column that holds a key of this CTA
        const int box = min(bs, TA_BN);                       // keys of one copy
        const int per_tile = TA_BN / box;                     // 1, 2, 4 or 8 copies: chunks of 32 end with a tile
        const int n_boxes = n_tiles * per_tile;
        // block of the g-th copy of this CTA; one outside [first key, last key] is replaced by a valid one:
        // its data is masked, and the softmax warps zero its rows of V
        auto fetch = [&](int g) -> int {
            if (g >= n_boxes) return 0;
            const int col = max(first_col, min((t_begin + g * box) / bs, last_col));
            int blk = p.block_table[(size_t)slot * p.max_blocks + col];
            if (blk < 0 || blk >= p.num_blocks) { set_status(p.status, STATUS_BAD_BLOCK); blk = 0; }
            return blk;
        };
        int blk_cur = 0, blk_next = fetch(lane);
        int issued = 0;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % STAGES;
            bool ok = true;
            if (it >= STAGES) ok = ta_wait(ta_saddr(&kv_empty[s]), ((it / STAGES) - 1) & 1, abort_flag, p.status, wait_ns);
            if (!__all_sync(0xffffffffu, ok && *abort_flag == 0)) break;
            const uint32_t full = ta_saddr(&kv_full[s]);
            if (lane == 0) ta_expect(full, 2 * TA_KTILE);
            unsigned char* ks = kv_s + s * 2 * TA_KTILE;
            unsigned char* vs = ks + TA_KTILE;
            const int t0 = t_begin + it * TA_BN;
            // The tile's copies (4 per cache block: K and V, each in two halves of the head) are issued by as
            // many lanes at once: one lane issuing them one after another took longer than the tile's tensor work.
            const int g0 = it * per_tile;                      // the tile's first copy group; chunks of 32 start on a tile
            if ((g0 & 31) == 0) { blk_cur = blk_next; blk_next = fetch(g0 + 32 + lane); }
            __syncwarp();                                      // the expectation is set before any copy can complete
            const int j = lane >> 2, part = lane & 3;
            const int blk = __shfl_sync(0xffffffffu, blk_cur, (g0 + j) & 31);
            if (j < per_tile && !(skip_last && it == n_tiles - 1 && lane == 0)) {      // tests: one copy of the last tile never leaves
                // row of the pool seen as [rows, d]: the (block, head) slab, and the tile's place in a larger block
                const int r0 = j * box;
                const int row = (blk * p.n_kv + kvh) * bs + (t0 + r0) % bs;
                unsigned char* dst = ((part & 2) ? vs : ks) + (part & 1) * TA_KSLAB + r0 * 128;
                ta_tma(ta_saddr(dst), (part & 2) ? &map_v : &map_k, full, (part & 1) * 64, row);
            }
            issued = it + 1;
        }
        // giving up: the copies in flight must land before the CTA's shared memory is released
        if (lane == 0 && *abort_flag)
            for (int it = max(0, issued - STAGES); it < issued; ++it)
                ta_wait(ta_saddr(&kv_full[it % STAGES]), (it / STAGES) & 1, abort_flag + 1, nullptr, wait_ns);
    } else if (warp == 1 && lane == 0) {
        // ---- issuer of S = Q K^T ----
        // D float, A and B bf16, M 128, N = 64 keys, both operands K-major.  S of a query tile's j-th key tile
        // goes into its S buffer j & 1 as soon as the softmax warps have taken the scores before last out of it
        // (s_free) - long before they are done with them - so the next scores are always ready; P V has an
        // issuer of its own (below): one thread issuing both took 0.6 us per tile, between two softmax steps.
        const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TA_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        bool ok = ta_wait(ta_saddr(&bars[0]), 0, abort_flag, p.status, wait_ns);
        for (int it = 0; ok && it < n_tiles; ++it) {
            const int s = it % STAGES;
            ok = ta_wait(ta_saddr(&kv_full[s]), (it / STAGES) & 1, abort_flag, p.status, wait_ns);
            const uint32_t ks = ta_saddr(kv_s + s * 2 * TA_KTILE);
#pragma unroll
            for (int qt = 0; qt < TA_NQ; ++qt) {
                int j;
                if (!ok || !mine(qt, it, j)) continue;
                if (j >= 2) ok = ta_wait(ta_saddr(&s_free[qt * 2 + (j & 1)]), ((j >> 1) - 1) & 1, abort_flag, p.status, wait_ns);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t qa = ta_saddr(q_s + (SPLIT ? 0 : qt) * TA_QTILE);
#pragma unroll
                for (int kk = 0; kk < TA_D / 16; ++kk) {       // 8 steps over the head dimension
                    const uint32_t inner = (kk & 3) * 32;
                    ta_mma(tmem_s + qt * 128 + (j & 1) * TA_BN, ta_desc_k(qa + (kk >> 2) * TA_QSLAB + inner),
                           ta_desc_k(ks + (kk >> 2) * TA_KSLAB + inner), idesc_qk, kk != 0);
                }
                ta_commit(ta_saddr(&s_full[qt * 2 + (j & 1)]));
            }
        }
        if (!ok) for (int i = 0; i < 2 * TA_NQ; ++i) ta_commit(ta_saddr(&s_full[i]));
    } else if (warp == TA_PV_WARP) {
        if (lane == 0) {
            // ---- issuer of O += P V: N = 128 dims, B (= V) MN-major ----
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(TA_D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            bool ok = true;
            for (int it = 0; ok && it < n_tiles; ++it) {
                const int s = it % STAGES;
                // the tile's copies have landed (the other issuer saw it long ago; this thread must see it too)
                ok = ta_wait(ta_saddr(&kv_full[s]), (it / STAGES) & 1, abort_flag, p.status, wait_ns);
                const uint32_t vs = ta_saddr(kv_s + s * 2 * TA_KTILE + TA_KTILE);
#pragma unroll
                for (int qt = 0; qt < TA_NQ; ++qt) {
                    int j;
                    if (!ok || !mine(qt, it, j)) continue;
                    ok = ta_wait(ta_saddr(&p_ready[qt]), j & 1, abort_flag, p.status, wait_ns);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t pa = ta_saddr(p_s + qt * TA_PTILE);
#pragma unroll
                    for (int kk = 0; kk < TA_BN / 16; ++kk)    // 4 steps over the keys
                        ta_mma(tmem_o + qt * TA_D, ta_desc_k(pa + kk * 32), ta_desc_mn(vs + kk * 2048, TA_KSLAB), idesc_pv,
                               (j | kk) != 0);
                    ta_commit(ta_saddr(&o_done[qt]));
                }
                // Q K^T of this key tile completed before its scores were read, so every product is done with the stage
                if (ok) ta_commit(ta_saddr(&kv_empty[s]));
            }
            if (!ok) for (int qt = 0; qt < TA_NQ; ++qt) ta_commit(ta_saddr(&o_done[qt]));
        }
    } else if (warp >= 2 && warp < 2 + 4 * TA_NQ) {
        // ---- softmax and epilogue (warps 2-5: first query tile, 6-9: second): thread = query row ----
        const int qt = (warp - 2) >> 2;
        const int quarter = warp & 3;                               // the quarter of the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pos = p_first[qt] + r;
        const int my_lo = q_lo[qt], my_hi = q_hi[qt];
        const float scale_log2 = p.scale * 1.4426950408889634f;   // > 0: the maximum is taken over raw scores
        float m_run = -INFINITY, l_run = 0.f;                      // running maximum (raw score) and sum
        bool ok = true;
        const int n_both = it_hi[qt] - it_lo[qt];
        const int n_mine = SPLIT ? (n_both + 1 - qt) >> 1 : n_both;
        unsigned char* my_p = p_s + qt * TA_PTILE;
        const uint32_t my_o = tmem_o + qt * TA_D;
        for (int j = 0; j < n_mine; ++j) {
            const int it = it_lo[qt] + (SPLIT ? 2 * j + qt : j);
            const int t0 = t_begin + it * TA_BN;
            ok = __all_sync(0xffffffffu, ta_wait(ta_saddr(&s_full[qt * 2 + (j & 1)]), (j >> 1) & 1, abort_flag, p.status, wait_ns));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float x[TA_BN];
            {
                uint32_t* v = reinterpret_cast<uint32_t*>(x);
                ta_ld32(tmem_s + qt * 128 + (j & 1) * TA_BN + lane_base, v);
                ta_ld32(tmem_s + qt * 128 + (j & 1) * TA_BN + lane_base + 32, v + 32);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            }
            // the scores are in registers: the S buffer may take the key tile after next
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            ta_arrive(ta_saddr(&s_free[qt * 2 + (j & 1)]));
            const bool need_mask = t0 + TA_BN - 1 > p_first[qt] || t0 < my_lo || t0 + TA_BN > my_hi ||
                                   (p.window > 0 && t0 < p_first[qt] + TA_BM - p.window);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < TA_BN; ++c) {
                    const int t = t0 + c;
                    if (!(t >= my_lo && t < my_hi && t <= pos && (p.window <= 0 || pos - t < p.window))) x[c] = -INFINITY;
                }
            }
            float mx4[4] = {x[0], x[1], x[2], x[3]};          // four chains instead of one of 63 dependent steps
#pragma unroll
            for (int c = 4; c < TA_BN; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], x[c]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // The maximum moves only when it grows by more than 2^8 (P stays below 256, exact enough in
            // bfloat16 and far from overflow in the 32-bit sums): most tiles then need no rescaling of O
            float m_new = fmaxf(m_run, mx);
            if (m_run != -INFINITY && (m_new - m_run) * scale_log2 <= 8.f) m_new = m_run;
            const float alpha = m_new == m_run ? 1.f : ta_ex2((m_run - m_new) * scale_log2);   // m_run = -inf: 0
            m_run = m_new;
            const float m_off = m_new == -INFINITY ? 0.f : m_new * scale_log2;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[TA_BN / 2];
#pragma unroll
            for (int c = 0; c < TA_BN; c += 2) {
                const float p0 = ta_ex2(fmaf(x[c], scale_log2, -m_off));
                const float p1 = ta_ex2(fmaf(x[c + 1], scale_log2, -m_off));
                rs4[(c >> 1) & 3] += p0 + p1;
                const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                packed[c >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
            }
            l_run = l_run * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
            // The previous P V must be complete before P is overwritten and before O is touched;
            // then O *= alpha where a maximum moved
            if (j > 0) {
                ok = __all_sync(0xffffffffu, ta_wait(ta_saddr(&o_done[qt]), (j - 1) & 1, abort_flag, p.status, wait_ns));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                    for (int c0 = 0; c0 < TA_D; c0 += 32) {
                        uint32_t v[32];
                        ta_ld32(my_o + lane_base + c0, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * alpha);
                        ta_st32(my_o + lane_base + c0, v);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            // P as bfloat16 into shared memory: K-major rows of 128 bytes, 16-byte chunks swizzled by the row
            unsigned char* prow = my_p + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) =
                    make_uint4(packed[c * 4], packed[c * 4 + 1], packed[c * 4 + 2], packed[c * 4 + 3]);
            // Rows of V that belong to no key of this CTA's range (the unused tail of the last cache block, a
            // block that stands in for one outside the range) may hold anything, even NaN, and 0 * NaN is NaN:
            // zero them.  The tile has landed (S was computed from it).  Both query tiles do it (the same zeros),
            // each before its own P V is allowed to start.
            if (r < TA_BN && (t0 + r < lo || t0 + r >= hi)) {
                unsigned char* vrow = kv_s + (it % STAGES) * 2 * TA_KTILE + TA_KTILE + r * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    *reinterpret_cast<uint4*>(vrow + c * 16) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(vrow + TA_KSLAB + c * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            // P and V (generic-proxy stores) must be visible to the tensor core's reads of shared memory
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            ta_arrive(ta_saddr(&p_ready[qt]));
        }
        if (ok && n_mine > 0) ok = __all_sync(0xffffffffu, ta_wait(ta_saddr(&o_done[qt]), (n_mine - 1) & 1, abort_flag, p.status, wait_ns));
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float w_own = l_run > 0.f ? 1.f / l_run : 0.f;          // what this thread's O is multiplied by
        float w_other = 0.f;                                    // SPLIT: and the other group's
        const float* o_other = nullptr;
        bool writes = ok && n_mine > 0;
        if (SPLIT) {
            // Both groups are past their last product and every copy of the ring was consumed, once all 256
            // threads have met: the ring is free, and takes the second group's O (float, [dim][row], so that
            // a warp's rows are neighbours) with its maxima and sums behind it.
            float* o_x = reinterpret_cast<float*>(kv_s);
            float* m_x = o_x + TA_D * TA_BM;
            float* l_x = m_x + TA_BM;
            const bool has_other = (n_both >> 1) > 0;           // the second group had a key tile at all
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const bool fine = ok && *abort_flag == 0;
            if (qt == 1 && fine && n_mine > 0) {
                m_x[r] = m_run == -INFINITY ? -INFINITY : m_run * scale_log2;
                l_x[r] = l_run;
#pragma unroll 1
                for (int c0 = 0; c0 < TA_D; c0 += 32) {
                    uint32_t v[32];
                    ta_ld32(my_o + lane_base + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < 32; ++c) o_x[(c0 + c) * TA_BM + r] = __uint_as_float(v[c]);
                }
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            writes = qt == 0 && fine && n_mine > 0;
            if (writes) {
                const float m0 = m_run == -INFINITY ? -INFINITY : m_run * scale_log2;
                const float m1 = has_other ? m_x[r] : -INFINITY;
                const float l1 = has_other ? l_x[r] : 0.f;
                const float m = fmaxf(m0, m1);
                const float a0 = m0 == -INFINITY ? 0.f : ta_ex2(m0 - m);
                const float a1 = m1 == -INFINITY ? 0.f : ta_ex2(m1 - m);
                const float l = l_run * a0 + l1 * a1;
                const float inv = l > 0.f ? 1.f / l : 0.f;
                w_own = a0 * inv;
                w_other = a1 * inv;
                if (has_other) o_other = o_x + r;
            }
        }
        if (writes) {
            __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(p.out) + ((size_t)(tok0 + (SPLIT ? 0 : qt * TA_BM) + r) * p.n_q + h) * TA_D;
#pragma unroll 1
            for (int c0 = 0; c0 < TA_D; c0 += 32) {
                uint32_t v[32];
                ta_ld32(my_o + lane_base + c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (SPLIT && o_other != nullptr) {
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        v[c] = __float_as_uint(fmaf(o_other[(c0 + c) * TA_BM], w_other, __uint_as_float(v[c]) * w_own));
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * w_own);
                }
                if (r < nq[qt]) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(v[c + 2 * e]), __uint_as_float(v[c + 2 * e + 1]));
                            w[e] = *reinterpret_cast<const uint32_t*>(&pk);
                        }
                        *reinterpret_cast<uint4*>(orow + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- host side ------------------------------------------------------------
typedef CUresult (*TaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TaEncodeFn ta_encode_fn() {
    static TaEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TaEncodeFn>(sym);
    }
    return fn;
}

// bf16 matrix [rows, cols] read in boxes of box_rows x 64 columns with the 128-byte swizzle
static int ta_map(const void* ptr, long long rows, int cols, int box_rows, CUtensorMap* out) {
    static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(ptr, rows, cols, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    TaEncodeFn fn = ta_encode_fn();
    if (fn == nullptr) return 1;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return 0;
}

static int g_ta_form = 0;

static int ta_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

// Returns 1 when it does not take the sizes (the caller falls back to the mma.sync kernel):
// head size 128, block size a multiple of 8 that divides 128, no split of the keys.
int launch_attn_prefill_tcgen05(const AttnParams& p, int n_rows, int T, int max_q_len, cudaStream_t stream) {
    if (p.d != TA_D || p.n_splits != 1) return 1;
    const int bs = p.block_size;
    if (bs < 8 || bs > 128 || bs % 8 != 0 || 128 % bs != 0) return 1;
    if ((max_q_len + TA_BM - 1) / TA_BM > 65535 || n_rows > 65535) return 1;
    CUtensorMap mq, mk, mv;
    if (ta_map(p.q, T, p.n_q * TA_D, TA_BM, &mq) != 0) return 1;
    const long long pool_rows = (long long)p.num_blocks * p.n_kv * bs;
    const int box = bs < TA_BN ? bs : TA_BN;
    if (ta_map(p.k_pool, pool_rows, TA_D, box, &mk) != 0) return 1;
    if (ta_map(p.v_pool, pool_rows, TA_D, box, &mv) != 0) return 1;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM);
        if (e != cudaSuccess) return fail(-3, "attention: cannot get %d bytes of shared memory: %s", TA_SMEM, cudaGetErrorString(e));
        configured = true;
    }
    // Two query tiles per CTA share every key tile; while that leaves SMs without a CTA, one query tile per
    // CTA with its key tiles dealt to the two softmax groups finishes sooner.
    const int shared_ctas = ((max_q_len + TA_ROWS - 1) / TA_ROWS) * p.n_q * n_rows;
    const bool split = g_ta_form == 2 || (g_ta_form == 0 && shared_ctas < ta_sm_count());
    if (split) {
        dim3 grid(p.n_q, (max_q_len + TA_BM - 1) / TA_BM, n_rows);
        attn_prefill_tcgen05_kernel<true><<<grid, TA_THREADS, TA_SMEM, stream>>>(mq, mk, mv, p, g_tc_wait_ns, g_tc_skip_last);
    } else {
        dim3 grid(p.n_q, (max_q_len + TA_ROWS - 1) / TA_ROWS, n_rows);
        attn_prefill_tcgen05_kernel<false><<<grid, TA_THREADS, TA_SMEM, stream>>>(mq, mk, mv, p, g_tc_wait_ns, g_tc_skip_last);
    }
    return check_launch("attention_prefill_tcgen05");
}

}  // namespace fd

// 0: the launcher chooses; 1: two query tiles per CTA; 2: one query tile, its key tiles dealt to the two groups
extern "C" void fd_attn_prefill_set_form(int form) { fd::g_ta_form = form; }

