// Matrix product for prompt steps on the 5th-generation tensor cores:
//     out[M, N] = x[M, K] W[N, K]^T (+ bias | gated SiLU)      bfloat16 in, float accumulate
//
// One CTA computes one 128 x 128 tile of the output.
//  * warp 0 (one lane): TMA producer.  `cp.async.bulk.tensor.2d` brings 128 x 64
//    tiles of x and of W into shared memory in the 128-byte-swizzled layout, three
//    stages deep, each stage announced on an mbarrier (expect_tx / complete_tx).
//    Three stages (97 KB) let two CTAs share an SM, so one CTA's epilogue runs
//    under the other's main loop; each takes 128 of the 512 tensor-memory columns.
//  * warp 1 (one lane): MMA issuer.  For every stage it issues four
//    `tcgen05.mma.cta_group::1.kind::f16` (M 128, N 128, K 16) whose operands are
//    shared-memory descriptors and whose accumulator lives in tensor memory
//    (128 lanes x 128 columns of float); `tcgen05.commit` hands the stage back to
//    the producer and, after the last one, tells the epilogue the tile is done.
//  * warps 2-5: epilogue.  Each reads its quarter of the accumulator with
//    `tcgen05.ld.32x32b` (a thread gets 32 consecutive columns of one row), adds
//    the bias or applies silu(gate) * up, rounds once and stores.
// Rows of x beyond M, rows of W beyond N and columns beyond K are zero-filled by
// the TMA unit, so any M, N and any K that is a multiple of 8 are taken.
//
// Every wait on an mbarrier is bounded in time: if one runs out, the CTA sets
// a bit in the status word, every role leaves its loop, tensor memory is freed
// and the kernel returns (wrong output, a reported error, no hang).
#include "tcgen05.cuh"

namespace fd {

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64, TC_STAGES = 3;
constexpr int TC_THREADS = 192;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;          // 16 KB
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;          // 16 KB
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_SMEM = TC_STAGES * TC_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

struct TcParams {
    const void* bias;      // [N] or null
    void* out;
    int* status;
    int M, N, K;
    int mode;              // 1: bf16 [M, N]; 2: float [M, N]; 3: gated, bf16 [M, N / 2];
                           // 4: q/k/v projection with rotary encoding and cache append (TcRope)
    int bias_f32;
    unsigned long long wait_ns;   // limit of every bounded wait
    int skip_last;                // tests only: the producer leaves out its very last copy, so that a wait runs out
};

// Mode 4: where the token of an output row lives in the cache.
struct TcToken {
    int slot, pos;
    size_t kv_off;
    bool kv_ok;
};

__device__ __forceinline__ TcToken tc_token(const TcParams& p, const TcRope& ra, int m) {
    TcToken t;
    t.slot = -1; t.pos = 0; t.kv_off = 0; t.kv_ok = false;
    if (p.mode == 4 && m < p.M) {
        t.slot = ra.row_slot[ra.tok_row[m]];
        t.pos = ra.tok_pos[m];
        if (t.slot >= 0) {
            if (t.pos < 0 || t.pos >= ra.table_len) {
                set_status(p.status, STATUS_BAD_POSITION);
                t.slot = -1;
            } else if (ra.write_kv) {
                const int blk = ra.block_table[(size_t)t.slot * ra.max_blocks + t.pos / ra.block_size];
                if (blk < 0 || blk >= ra.num_blocks) {
                    set_status(p.status, STATUS_BAD_BLOCK);
                } else {
                    t.kv_off = ((size_t)blk * ra.n_kv * ra.block_size + t.pos % ra.block_size) * ra.d;
                    t.kv_ok = true;
                }
            }
        }
    }
    return t;
}

// The epilogue of 32 consecutive columns n .. n + 31 of output row m, whose float sums are v[0..31].
__device__ __forceinline__ void tc_store32(const TcParams& p, const TcRope& ra, const TcToken& tk, const uint32_t (&v)[32],
                                           const int m, const int n) {
    const int tok_slot = tk.slot, tok_pos = tk.pos;
    const size_t kv_off = tk.kv_off;
    const bool kv_ok = tk.kv_ok;
    if (m >= p.M || n >= p.N) return;
    if (p.mode == 4) {
        if (tok_slot < 0) return;                         // padding row or bad position
        const int d = ra.d, half = d >> 1;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int col = n + t * 16;                      // first column of this tile of 16
            if (col >= p.N) break;
            const int head = col / d, in_head = col - head * d;
            float lo8[8], hi8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                lo8[j] = __uint_as_float(v[t * 16 + j]);
                hi8[j] = __uint_as_float(v[t * 16 + 8 + j]);
            }
            if (p.bias != nullptr) {
                // the 16 bias values of the tile with vector loads (col is a multiple of 16, the launcher checks the base)
                if (p.bias_f32) {
                    const float4* b4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.bias) + col);
                    const float4 b0 = b4[0], b1 = b4[1], b2 = b4[2], b3 = b4[3];
                    lo8[0] += b0.x; lo8[1] += b0.y; lo8[2] += b0.z; lo8[3] += b0.w;
                    lo8[4] += b1.x; lo8[5] += b1.y; lo8[6] += b1.z; lo8[7] += b1.w;
                    hi8[0] += b2.x; hi8[1] += b2.y; hi8[2] += b2.z; hi8[3] += b2.w;
                    hi8[4] += b3.x; hi8[5] += b3.y; hi8[6] += b3.z; hi8[7] += b3.w;
                } else {
                    const uint4* b4 = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.bias) + col);
                    const uint4 bl = b4[0], bh = b4[1];
                    const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&bl);
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&bh);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        lo8[2 * j] += __low2float(l2[j]); lo8[2 * j + 1] += __high2float(l2[j]);
                        hi8[2 * j] += __low2float(h2[j]); hi8[2 * j + 1] += __high2float(h2[j]);
                    }
                }
            }
            const bool is_v = head >= ra.n_q + ra.n_kv;
            int j_lo, j_hi;                                   // dims of the two groups of 8 inside the head
            if (is_v) {
                j_lo = in_head; j_hi = in_head + 8;
            } else {
                j_lo = (in_head >> 4) * 8; j_hi = j_lo + half;
                const float4* c4 = reinterpret_cast<const float4*>(ra.cos_t + (size_t)tok_pos * half + j_lo);
                const float4* s4 = reinterpret_cast<const float4*>(ra.sin_t + (size_t)tok_pos * half + j_lo);
                const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
                const float cs[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
                const float sn[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float x1 = lo8[j], x2 = hi8[j];
                    lo8[j] = x1 * cs[j] - x2 * sn[j];
                    hi8[j] = x2 * cs[j] + x1 * sn[j];
                }
            }
            uint32_t pl[4], ph[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 a = __floats2bfloat162_rn(lo8[2 * j], lo8[2 * j + 1]);
                const __nv_bfloat162 b = __floats2bfloat162_rn(hi8[2 * j], hi8[2 * j + 1]);
                pl[j] = *reinterpret_cast<const uint32_t*>(&a);
                ph[j] = *reinterpret_cast<const uint32_t*>(&b);
            }
            __nv_bfloat16* dst;
            if (head < ra.n_q) {
                dst = static_cast<__nv_bfloat16*>(p.out) + ((size_t)m * ra.n_q + head) * d;
            } else {
                if (!kv_ok) continue;
                const int kvh = is_v ? head - ra.n_q - ra.n_kv : head - ra.n_q;
                dst = (is_v ? ra.v_pool : ra.k_pool) + kv_off + (size_t)kvh * ra.block_size * d;
            }
            *reinterpret_cast<uint4*>(dst + j_lo) = make_uint4(pl[0], pl[1], pl[2], pl[3]);
            *reinterpret_cast<uint4*>(dst + j_hi) = make_uint4(ph[0], ph[1], ph[2], ph[3]);
        }
        return;
    }
    if (p.mode == 3) {
        // 32 columns = two tiles of 8 gate + 8 up values -> 16 outputs (N is a multiple of 16)
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)m * (p.N >> 1) + (n >> 1);
        uint32_t packed[8];
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const float g0 = __uint_as_float(v[t * 16 + j]), u0 = __uint_as_float(v[t * 16 + 8 + j]);
                const float g1 = __uint_as_float(v[t * 16 + j + 1]), u1 = __uint_as_float(v[t * 16 + 9 + j]);
                const __nv_bfloat162 r = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0,
                                                               g1 / (1.f + __expf(-g1)) * u1);
                packed[t * 4 + (j >> 1)] = *reinterpret_cast<const uint32_t*>(&r);
            }
        *reinterpret_cast<uint4*>(o) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        if (n + 16 < p.N) *reinterpret_cast<uint4*>(o + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        return;
    }
    const int cols = min(32, p.N - n);
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
    if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int nn = min(n + j, p.N - 1);
            f[j] += p.bias_f32 ? static_cast<const float*>(p.bias)[nn]
                               : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[nn]);
        }
    }
    if (p.mode == 1) {
        __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.N + n;
        if (cols == 32 && (p.N & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                const __nv_bfloat162 r0 = __floats2bfloat162_rn(f[j], f[j + 1]), r1 = __floats2bfloat162_rn(f[j + 2], f[j + 3]);
                const __nv_bfloat162 r2 = __floats2bfloat162_rn(f[j + 4], f[j + 5]), r3 = __floats2bfloat162_rn(f[j + 6], f[j + 7]);
                *reinterpret_cast<uint4*>(o + j) = make_uint4(*reinterpret_cast<const uint32_t*>(&r0), *reinterpret_cast<const uint32_t*>(&r1),
                                                              *reinterpret_cast<const uint32_t*>(&r2), *reinterpret_cast<const uint32_t*>(&r3));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < cols) o[j] = __float2bfloat16_rn(f[j]);
        }
    } else {
        float* o = static_cast<float*>(p.out) + (size_t)m * p.N + n;
        if (cols == 32 && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(o + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < cols) o[j] = f[j];
        }
    }
}

__global__ void __launch_bounds__(TC_THREADS, 2)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const TcParams p, const TcRope ra) {
    extern __shared__ unsigned char tc_smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);
    // bars[0..S): full, bars[S..2S): empty, bars[2S]: accumulator ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN;
    const int k_iters = (p.K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        abort_flag[0] = 0;
        abort_flag[1] = 0;        // private flag of the producer's drain loop
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(s_addr(&bars[s]), 1);
            mbar_init(s_addr(&bars[TC_STAGES + s]), 1);
        }
        mbar_init(s_addr(&bars[2 * TC_STAGES]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // 128 columns of tensor memory for the float accumulator (power of two >= 32)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(TC_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer ----
        int issued = 0;
        for (int it = 0; it < k_iters; ++it) {
            const int s = it % TC_STAGES;
            if (it >= TC_STAGES &&
                !mbar_wait(s_addr(&bars[TC_STAGES + s]), ((it / TC_STAGES) - 1) & 1, abort_flag, p.status, p.wait_ns)) break;
            if (*abort_flag) break;
            const uint32_t full = s_addr(&bars[s]);
            mbar_expect_tx(full, TC_STAGE_BYTES);
            unsigned char* a = tiles + s * TC_STAGE_BYTES;
            tma_load_2d(s_addr(a), &map_x, full, it * TC_BK, m0);
            if (!(p.skip_last && it == k_iters - 1)) tma_load_2d(s_addr(a + TC_A_BYTES), &map_w, full, it * TC_BK, n0);
            issued = it + 1;
        }
        if (*abort_flag) {
            // let the copies already under way land before the CTA goes away
            for (int it = max(0, issued - TC_STAGES); it < issued; ++it)
                mbar_wait(s_addr(&bars[it % TC_STAGES]), (it / TC_STAGES) & 1, abort_flag + 1, nullptr, p.wait_ns);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        // instruction descriptor: D float, A and B bf16, both K-major, N / 8, M / 16
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        for (int it = 0; it < k_iters; ++it) {
            const int s = it % TC_STAGES;
            if (!mbar_wait(s_addr(&bars[s]), (it / TC_STAGES) & 1, abort_flag, p.status, p.wait_ns)) break;
            tc_fence_after();
            const uint32_t a = s_addr(tiles + s * TC_STAGE_BYTES);
            const uint64_t adesc = smem_desc_sw128(a), bdesc = smem_desc_sw128(a + TC_A_BYTES);
#pragma unroll
            for (int kk = 0; kk < TC_BK / 16; ++kk)        // 32 bytes further along the swizzled row per K = 16
                tc_mma(tmem, adesc + 2 * kk, bdesc + 2 * kk, idesc, (it | kk) != 0);
            tc_commit(s_addr(&bars[TC_STAGES + s]));        // the stage is free once these MMAs have read it
        }
        tc_commit(s_addr(&bars[2 * TC_STAGES]));            // the accumulator is complete
    } else if (warp >= 2) {
        // ---- epilogue: warp w may touch lanes 32 (w % 4) .. + 32 of tensor memory ----
        const int quarter = warp & 3;
        const int m = m0 + quarter * 32 + lane;
        // all lanes of a warp must agree before the warp-wide tensor-memory loads
        const bool ok = __all_sync(0xffffffffu, mbar_wait(s_addr(&bars[2 * TC_STAGES]), 0, abort_flag, p.status, p.wait_ns));
        tc_fence_after();
        const TcToken tk = tc_token(p, ra, m);
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < TC_BN; c0 += 32) {
                uint32_t v[32];
                tc_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + c0, v);
                tc_wait_ld();
                tc_store32(p, ra, tk, v, m, n0 + c0);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_BN) : "memory");
    }
}

// ---- the wide, persistent form --------------------------------------------
// 128 x 256 tiles, one CTA per SM that walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...:
//  * a 128 x 128 tile reads 32 KB of shared memory for every 2 MFLOP, which is the whole
//    shared-memory bandwidth of an SM at the tensor cores' rate; 128 x 256 reads 48 KB for 4 MFLOP;
//  * the accumulator is double-buffered in tensor memory (2 x 256 of the 512 columns): the
//    epilogue warps drain one tile while the MMA warp fills the next, and the TMA warp runs
//    ahead across tile boundaries, four stages of 48 KB deep;
//  * consecutive tiles share their W panel (tile index = n_tile * tiles_m + m_tile), so the CTAs
//    running at one time read the same few panels of W through L2.
constexpr int TW_BN = 256, TW_STAGES = 4;
constexpr int TW_B_BYTES = TW_BN * TC_BK * 2;                 // 32 KB
constexpr int TW_STAGE_BYTES = TC_A_BYTES + TW_B_BYTES;       // 48 KB
constexpr int TW_SMEM = TW_STAGES * TW_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
// The same kernel with 128 x 128 tiles and six stages of 32 KB, for products so small that even these tiles number no
// more than the SMs (prompts of up to about 1,000 tokens at these widths): twice the CTAs at work, each with half the
// chain of copies and MMAs (q/k/v with its epilogue at 512 and 1,024 tokens: 16 against 22 us).
constexpr int TN_BN = 128, TN_STAGES = 6;
constexpr int TN_SMEM = TN_STAGES * (TC_A_BYTES + TN_BN * TC_BK * 2) + 1024 + 256;
constexpr int TW_EPI_WARPS = 8;               // two per quarter of the tensor-memory lanes, half of the columns each
constexpr int TW_THREADS = (2 + TW_EPI_WARPS) * 32;

template <int BN, int STAGES>
__global__ void __launch_bounds__(TW_THREADS, 1)
gemm_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const TcParams p, const TcRope ra, const int tiles_m, const int tiles_n) {
    constexpr int STAGE_BYTES = TC_A_BYTES + BN * TC_BK * 2;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                       // [S] a stage has landed
    uint64_t* empty = bars + STAGES;          // [S] the MMAs that read a stage are done
    uint64_t* acc_full = bars + 2 * STAGES;   // [2] an accumulator is complete
    uint64_t* acc_empty = acc_full + 2;          // [2] the epilogue has read it (one arrival per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_iters = (p.K + TC_BK - 1) / TC_BK;
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(s_addr(&full[s]), 1);
            mbar_init(s_addr(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_addr(&acc_full[b]), 1);
            mbar_init(s_addr(&acc_empty[b]), TW_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer ----
        int it = 0;                                    // k-blocks issued so far, over all tiles
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(s_addr(&empty[s]), ((it / STAGES) - 1) & 1, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
                if (*abort_flag) { ok = false; break; }
                const uint32_t fb = s_addr(&full[s]);
                mbar_expect_tx(fb, STAGE_BYTES);
                unsigned char* a = tiles + s * STAGE_BYTES;
                tma_load_2d(s_addr(a), &map_x, fb, k * TC_BK, m0);
                if (p.skip_last && k == k_iters - 1 && tile + (int)gridDim.x >= n_tiles) continue;       // tests: this CTA's very last copy
                tma_load_2d(s_addr(a + TC_A_BYTES), &map_w, fb, k * TC_BK, n0);     // BN rows of W in one box
            }
        }
        if (*abort_flag) {
            for (int j = max(0, it - STAGES); j < it; ++j)
                mbar_wait(s_addr(&full[j % STAGES]), (j / STAGES) & 1, abort_flag + 1, nullptr, p.wait_ns);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        int it = 0, t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            if (t >= 2 && !mbar_wait(s_addr(&acc_empty[buf]), ((t >> 1) - 1) & 1, abort_flag, p.status, p.wait_ns)) break;
            tc_fence_after();
            const uint32_t acc = tmem + buf * BN;
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(s_addr(&full[s]), (it / STAGES) & 1, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a = s_addr(tiles + s * STAGE_BYTES);
                const uint64_t adesc = smem_desc_sw128(a), bdesc = smem_desc_sw128(a + TC_A_BYTES);
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)
                    tc_mma(acc, adesc + 2 * kk, bdesc + 2 * kk, idesc, (k | kk) != 0);
                tc_commit(s_addr(&empty[s]));
            }
            if (ok) tc_commit(s_addr(&acc_full[buf]));
        }
        if (!ok || *abort_flag) { tc_commit(s_addr(&acc_full[0])); tc_commit(s_addr(&acc_full[1])); }
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads lanes 32 (w % 4) .. + 32; warps 2-5 take columns 0..127, 6-9 the rest ----
        const int quarter = warp & 3;
        const int col_half = (warp - 2) >> 2;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        int t = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
            const int m = m0 + quarter * 32 + lane;
            const TcToken tk = tc_token(p, ra, m);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(s_addr(&acc_full[buf]), (t >> 1) & 1, abort_flag, p.status, p.wait_ns)) &&
                            *abort_flag == 0;
            if (!__all_sync(0xffffffffu, ok)) break;
            tc_fence_after();
#pragma unroll 1
            for (int c0 = col_half * (BN / 2); c0 < (col_half + 1) * (BN / 2); c0 += 32) {
                uint32_t v[32];
                tc_ld32(tmem + lane_base + buf * BN + c0, v);
                tc_wait_ld();
                tc_store32(p, ra, tk, v, m, n0 + c0);
            }
            // the accumulator may be overwritten once all epilogue warps have read it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(&acc_empty[buf])) : "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}

// ---- the two-SM form ---------------------------------------------------------
// A cluster of two CTAs (two SMs) computes one 256 x 256 tile with tcgen05.mma.cta_group::2: each CTA holds
// 128 rows of x and HALF of the W tile (128 of its 256 rows) in its own shared memory and gets 128 rows of the
// accumulator in its own tensor memory; the tensor cores of both SMs read both halves of W.  A stage is then
// 32 KB per CTA instead of 48 KB for the same 4 MFLOP per CTA, so six stages fit and the copies from L2 keep up
// (the wide one-SM form above waits for data more than half of the time).
//  * both CTAs run a TMA thread; every copy signals the LEADER's (rank 0) `full` barrier, which expects the
//    bytes of both CTAs (cp.async.bulk.tensor with .cta_group::2 may signal the peer's barrier);
//  * the leader's MMA thread issues for the pair; tcgen05.commit with a CTA mask hands a stage back to both
//    TMA threads and an accumulator to both CTAs' epilogue warps;
//  * both CTAs' epilogue warps read their own tensor memory and arrive (the peer remotely) on the leader's
//    `acc_empty` barrier; tensor memory is allocated and freed by one warp of each CTA together.
// A stage holds KB k-blocks of 64 (KB = 2 where K is a multiple of 64: each operand's k-blocks then come as ONE copy
// through a three-dimensional tensor map, 32 KB instead of 16 KB - an SM keeps only a few bulk copies in flight,
// whatever their size, and with 16 KB copies that bounds the pair at about 70 GB/s per SM, below what its tensor
// cores consume).  Three stages of 64 KB, or six of 32 KB.
constexpr int TP_RING_KBLOCKS = 6;
constexpr int TP_B_BYTES = 128 * TC_BK * 2;                   // this CTA's half of the W tile, one k-block: 16 KB
constexpr int TP_KBLOCK_BYTES = TC_A_BYTES + TP_B_BYTES;      // 32 KB
constexpr int TP_SMEM = TP_RING_KBLOCKS * TP_KBLOCK_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
template <int KB>
__global__ void __launch_bounds__(TW_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const TcParams p, const TcRope ra, const int tiles_m, const int tiles_n) {
    constexpr int TP_STAGES = TP_RING_KBLOCKS / KB;
    constexpr int TP_STAGE_BYTES = KB * TP_KBLOCK_BYTES;      // x: KB tiles of 16 KB, then W: KB tiles of 16 KB
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TP_STAGES * TP_STAGE_BYTES);
    uint64_t* full = bars;                       // [S] used in the leader: both CTAs' copies of a stage have landed
    uint64_t* empty = bars + TP_STAGES;          // [S] in each CTA: the MMAs that read the stage are done
    uint64_t* acc_full = bars + 2 * TP_STAGES;   // [2] in each CTA: an accumulator is complete
    uint64_t* acc_empty = acc_full + 2;          // [2] used in the leader: both CTAs' epilogue warps have read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int k_iters = ((p.K + TC_BK - 1) / TC_BK + KB - 1) / KB;       // stages of KB k-blocks (a last one may reach beyond K: zeros)
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        abort_flag[0] = 0;
        abort_flag[1] = 0;
        for (int s = 0; s < TP_STAGES; ++s) {
            mbar_init(s_addr(&full[s]), 1);
            mbar_init(s_addr(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_addr(&acc_full[b]), 1);
            mbar_init(s_addr(&acc_empty[b]), 2 * TW_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // one warp of each CTA, together: the same 512 columns in both tensor memories
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();              // the peer's barriers exist before anything of this CTA signals them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer (in both CTAs): this CTA's 128 rows of x and its half of the W tile ----
        int it = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < n_tiles; tile += n_pairs) {
            const int m0 = (tile % tiles_m) * (2 * TC_BM) + (int)rank * TC_BM;
            const int n0 = (tile / tiles_m) * TW_BN + (int)rank * TC_BN;
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % TP_STAGES;
                if (it >= TP_STAGES && !mbar_wait(s_addr(&empty[s]), ((it / TP_STAGES) - 1) & 1, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
                if (*abort_flag) { ok = false; break; }
                if (leader) mbar_expect_tx(s_addr(&full[s]), 2 * TP_STAGE_BYTES);
                const uint32_t fb = map_to_rank(s_addr(&full[s]), 0);
                unsigned char* a = tiles + s * TP_STAGE_BYTES;
                if (KB == 1) tma_load_2d_pair(s_addr(a), &map_x, fb, k * TC_BK, m0);
                else tma_load_3d_pair(s_addr(a), &map_x, fb, 0, m0, k * KB);
                if (p.skip_last && k == k_iters - 1 && tile + n_pairs >= n_tiles) continue;              // tests: this CTA's very last copy
                if (KB == 1) tma_load_2d_pair(s_addr(a + TC_A_BYTES), &map_w, fb, k * TC_BK, n0);
                else tma_load_3d_pair(s_addr(a + KB * TC_A_BYTES), &map_w, fb, 0, n0, k * KB);
            }
        }
        // Giving up: the copies in flight must land before this CTA's shared memory goes away.  The leader sees
        // them on its own barriers; the peer cannot wait on the leader's, so it waits out the copies' time.
        if (*abort_flag) {
            if (leader) {
                for (int j = max(0, it - TP_STAGES); j < it; ++j)
                    mbar_wait(s_addr(&full[j % TP_STAGES]), (j / TP_STAGES) & 1, abort_flag + 1, nullptr, p.wait_ns);
            } else {
                const unsigned long long t0 = global_ns();
                while (global_ns() - t0 < 1000000ull) { }
            }
        }
    } else if (warp == 1 && lane == 0 && leader) {
        // ---- MMA issuer, for the pair: M 256 (128 rows in each CTA), N 256 ----
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TW_BN >> 3) << 17) | ((uint32_t)((2 * TC_BM) >> 4) << 24);
        int it = 0, t = 0;
        bool ok = true;
        for (int tile = pair; ok && tile < n_tiles; tile += n_pairs, ++t) {
            const int buf = t & 1;
            if (t >= 2 && !mbar_wait(s_addr(&acc_empty[buf]), ((t >> 1) - 1) & 1, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
            tc_fence_after();
            const uint32_t acc = tmem + buf * TW_BN;
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % TP_STAGES;
                if (!mbar_wait(s_addr(&full[s]), (it / TP_STAGES) & 1, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a = s_addr(tiles + s * TP_STAGE_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    const uint64_t adesc = smem_desc_sw128(a + kb * TC_A_BYTES), bdesc = smem_desc_sw128(a + KB * TC_A_BYTES + kb * TP_B_BYTES);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk)
                        tc_mma_pair(acc, adesc + 2 * kk, bdesc + 2 * kk, idesc, (k | kb | kk) != 0);
                }
                tc_commit_pair(s_addr(&empty[s]), 3);          // the stage is free in both CTAs
            }
            if (ok) tc_commit_pair(s_addr(&acc_full[buf]), 3); // the accumulator is complete in both CTAs
        }
        if (!ok || *abort_flag) { tc_commit_pair(s_addr(&acc_full[0]), 3); tc_commit_pair(s_addr(&acc_full[1]), 3); }
    } else if (warp >= 2) {
        // ---- epilogue (in both CTAs): this CTA's 128 rows of the tile ----
        const int quarter = warp & 3;
        const int col_half = (warp - 2) >> 2;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        int t = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++t) {
            const int buf = t & 1;
            const int m0 = (tile % tiles_m) * (2 * TC_BM) + (int)rank * TC_BM, n0 = (tile / tiles_m) * TW_BN;
            const int m = m0 + quarter * 32 + lane;
            const TcToken tk = tc_token(p, ra, m);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(s_addr(&acc_full[buf]), (t >> 1) & 1, abort_flag, p.status, p.wait_ns)) &&
                            *abort_flag == 0;
            if (!__all_sync(0xffffffffu, ok)) break;
            tc_fence_after();
#pragma unroll 1
            for (int c0 = col_half * (TW_BN / 2); c0 < (col_half + 1) * (TW_BN / 2); c0 += 32) {
                uint32_t v[32];
                tc_ld32(tmem + lane_base + buf * TW_BN + c0, v);
                tc_wait_ld();
                tc_store32(p, ra, tk, v, m, n0 + c0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(s_addr(&acc_empty[buf]), 0));
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();              // neither CTA leaves (or frees tensor memory) while the other may still touch it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- host side ------------------------------------------------------------
int g_tc_wide = 1;      // 2: the two-SM kernel where N >= 256; 1: the persistent one-SM kernel (128 x 256 tiles, or 128 x 128
                        // where those number no more than the SMs); 3: the same with 128 x 256 tiles always; 0: 128 x 128 tiles, one per CTA

static int launch_tc(const void* x, const void* w, const TcParams& p, const TcRope& ra, cudaStream_t stream,
                     const char* what) {
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_wide_kernel<TW_BN, TW_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, TW_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_wide_kernel<TN_BN, TN_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, TN_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TP_SMEM);
        if (e != cudaSuccess) return fail(-3, "gemm_tcgen05: cannot get %d bytes of shared memory: %s", TW_SMEM, cudaGetErrorString(e));
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int tiles_m = (p.M + TC_BM - 1) / TC_BM;
    const bool wide = g_tc_wide && p.N >= TW_BN;
    const bool pair = wide && g_tc_wide == 2;
    // 128 x 128 tiles where even those give no CTA a second tile: twice the CTAs at work.  (Where CTAs would take two
    // of them in a row, the wider tile is faster: q/k/v of 2,048 tokens 22.5 against 25.3 us.)
    const bool narrow = wide && !pair && g_tc_wide != 3 && (long long)tiles_m * ((p.N + TN_BN - 1) / TN_BN) <= sms;
    CUtensorMap mx, mw;
    if (pair) {
        const int tiles_m2 = (p.M + 2 * TC_BM - 1) / (2 * TC_BM), tiles_n = (p.N + TW_BN - 1) / TW_BN;
        const long long n_tiles = (long long)tiles_m2 * tiles_n;
        FD_REQUIRE(n_tiles < (1ll << 30), -2, "gemm_tcgen05: %lld tiles", n_tiles);
        const int pairs = (int)(n_tiles < sms / 2 ? n_tiles : sms / 2);
        // two k-blocks per copy where the three-dimensional view of the operands exists
        if (p.K % 64 == 0 && p.K >= 128 && tensor_map_blocks(x, p.M, p.K, &mx, TC_BM, 2) == 0 &&
            tensor_map_blocks(w, p.N, p.K, &mw, TC_BM, 2) == 0)
            return launch(what, gemm_tcgen05_pair_kernel<2>, dim3(2 * pairs), dim3(TW_THREADS), TP_SMEM, stream, dim3(2, 1, 1), mx, mw,
                          p, ra, tiles_m2, tiles_n);
        int rc = tensor_map(x, p.M, p.K, &mx, TC_BM);
        if (rc == 0) rc = tensor_map(w, p.N, p.K, &mw, TC_BM);
        if (rc != 0) return rc;
        return launch(what, gemm_tcgen05_pair_kernel<1>, dim3(2 * pairs), dim3(TW_THREADS), TP_SMEM, stream, dim3(2, 1, 1), mx, mw, p, ra,
                      tiles_m2, tiles_n);
    }
    int rc = tensor_map(x, p.M, p.K, &mx, TC_BM);
    if (rc != 0) return rc;
    rc = tensor_map(w, p.N, p.K, &mw, (wide && !narrow) ? TW_BN : TC_BM);
    if (rc != 0) return rc;
    if (wide) {
        const int bn = narrow ? TN_BN : TW_BN;
        const int tiles_n = (p.N + bn - 1) / bn;
        const long long n_tiles = (long long)tiles_m * tiles_n;
        FD_REQUIRE(n_tiles < (1ll << 30), -2, "gemm_tcgen05: %lld tiles", n_tiles);
        const int grid = (int)(n_tiles < sms ? n_tiles : sms);
        if (narrow) gemm_tcgen05_wide_kernel<TN_BN, TN_STAGES><<<grid, TW_THREADS, TN_SMEM, stream>>>(mx, mw, p, ra, tiles_m, tiles_n);
        else gemm_tcgen05_wide_kernel<TW_BN, TW_STAGES><<<grid, TW_THREADS, TW_SMEM, stream>>>(mx, mw, p, ra, tiles_m, tiles_n);
        return check_launch(what);
    }
    dim3 grid((p.N + TC_BN - 1) / TC_BN, tiles_m);
    FD_REQUIRE(grid.y <= 65535, -2, "gemm_tcgen05: M=%d too large for one launch", p.M);
    gemm_tcgen05_kernel<<<grid, TC_THREADS, TC_SMEM, stream>>>(mx, mw, p, ra);
    return check_launch(what);
}

}  // namespace fd

using namespace fd;

// Which tiling the products use from now on where N >= 256 (1, the default: persistent CTAs with 128 x 256 tiles, or
// with 128 x 128 tiles where those number no more than the SMs; 3: persistent CTAs with 128 x 256 tiles always; 2: two
// SMs per 256 x 256 tile; 0: 128 x 128 tiles, one per CTA, everywhere).  For tests and measurements.
extern "C" int fd_gemm_tc_set_wide(int on) {
    g_tc_wide = on < 0 ? 0 : (on > 3 ? 3 : on);
    return 0;
}

// 1 if the tensor-core product takes these sizes (K a multiple of 8, enough rows to be worth a
// 128-row tile), else 0.
extern "C" int fd_gemm_tc_supported(int M, int N, int K) {
    return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && encode_fn() != nullptr;
}

// mode 1: out bf16 [M, N] (+ bias); 2: out float [M, N] (+ bias); 3: W rows in tiles of 8 gate +
// 8 up rows, out bf16 [M, N / 2] = silu(gate) * up (N a multiple of 16).
extern "C" int fd_gemm_tc(const void* x, const void* w, const void* bias, int bias_f32, void* out, int mode,
                          int M, int N, int K, int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    FD_REQUIRE(K >= 8 && K % 8 == 0, -2, "gemm_tcgen05: K=%d must be a multiple of 8 (16-byte rows for TMA)", K);
    FD_REQUIRE(mode >= 1 && mode <= 3, -2, "gemm_tcgen05: mode %d", mode);
    FD_REQUIRE(mode != 3 || N % 16 == 0, -2, "gemm_tcgen05: the gated form needs N (= 2 x outputs) to be a multiple of 16, got %d", N);
    FD_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0, -2,
               "gemm_tcgen05: x, W and out must be 16-byte aligned");
    TcParams p;
    p.bias = bias; p.out = out; p.status = status; p.M = M; p.N = N; p.K = K; p.mode = mode; p.bias_f32 = bias_f32;
    p.wait_ns = g_tc_wait_ns; p.skip_last = g_tc_skip_last;
    TcRope ra = {};
    return launch_tc(x, w, p, ra, stream, "gemm_tcgen05");
}

// The q/k/v projection of a prompt step with bias, rotary encoding and the append to the
// paged cache in its epilogue (mode 4; see TcRope for the row order W and bias must have).
extern "C" int fd_gemm_tc_qkv_rope(const void* x, const void* w, const void* bias, int bias_f32, void* q_out,
                                   int M, int K, const float* cos_t, const float* sin_t, int table_len,
                                   const int* tok_row, const int* tok_pos, const int* row_slot, void* k_pool,
                                   void* v_pool, const int* block_table, int max_blocks, int num_blocks,
                                   int block_size, int n_q, int n_kv, int d, int write_kv, int* status,
                                   cudaStream_t stream) {
    if (M == 0) return 0;
    const int N = (n_q + 2 * n_kv) * d;
    FD_REQUIRE(K >= 8 && K % 8 == 0, -2, "gemm_tcgen05: K=%d must be a multiple of 8 (16-byte rows for TMA)", K);
    FD_REQUIRE(d >= 16 && d % 16 == 0, -2, "gemm_tc_qkv_rope: head size %d must be a multiple of 16", d);
    FD_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)q_out % 16 == 0 &&
               (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0 && (uintptr_t)cos_t % 16 == 0 &&
               (uintptr_t)sin_t % 16 == 0 && (uintptr_t)bias % 16 == 0, -2, "gemm_tc_qkv_rope: all arrays must be 16-byte aligned");
    TcParams p;
    p.bias = bias; p.out = q_out; p.status = status; p.M = M; p.N = N; p.K = K; p.mode = 4; p.bias_f32 = bias_f32;
    p.wait_ns = g_tc_wait_ns; p.skip_last = g_tc_skip_last;
    TcRope ra;
    ra.cos_t = cos_t; ra.sin_t = sin_t; ra.tok_row = tok_row; ra.tok_pos = tok_pos; ra.row_slot = row_slot;
    ra.k_pool = (__nv_bfloat16*)k_pool; ra.v_pool = (__nv_bfloat16*)v_pool; ra.block_table = block_table;
    ra.table_len = table_len; ra.max_blocks = max_blocks; ra.num_blocks = num_blocks; ra.block_size = block_size;
    ra.n_q = n_q; ra.n_kv = n_kv; ra.d = d; ra.write_kv = write_kv;
    return launch_tc(x, w, p, ra, stream, "gemm_tc_qkv_rope");
}

// Tests only: the limit of every bounded wait in the TMA + tcgen05 kernels (nanoseconds; 0 restores the
// default of 0.2 s), and whether their TMA producers leave out their very last copy, so that a wait runs
// out, the kernel reports STATUS_WAIT_TIMEOUT and returns.  Nothing faults or hangs.
extern "C" int fd_tc_test_hook(long long wait_ns, int skip_last) {
    g_tc_wait_ns = wait_ns > 0 ? (unsigned long long)wait_ns : TC_WAIT_NS;
    g_tc_skip_last = skip_last ? 1 : 0;
    return 0;
}
