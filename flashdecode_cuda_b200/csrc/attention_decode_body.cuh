// The body of the split-KV decode attention kernel on the tensor cores (attention_decode_mma.cu), as a
// function of a CTA of W warps (4 or 8).
//
// Two arrangements of the tensor work per 16-key tile of a warp:
//  * TR (groups of up to 8 query heads per KV head): the 16 KEYS are the M rows of mma.m16n8k16 and the
//    heads its 8 columns: S^T[16 keys, 8 heads] = K Q^T, O^T[D, 8 heads] += V^T P^T.  8 + 8 MMAs per tile
//    and 32 accumulator registers for O; P^T reaches the second product through `movmatrix` (a transpose
//    of 8 x 8 tiles across the warp).
//  * otherwise (groups of up to 16): the heads are the M rows: S[16 heads, 16 keys] = Q K^T, O[16 heads, D]
//    += P V; 16 + 16 MMAs per tile and 64 registers for O.
// With 6 heads in 16 rows the second form spends most of its tensor work on padding; the first halves the
// MMAs and ldmatrix traffic of a tile, which at batch 64 was what the warps waited for.
#pragma once

#include <math.h>

#include "attention.cuh"
#include "mma_utils.cuh"

namespace fd {

constexpr int DM_TILE = 16;       // keys per warp tile
constexpr int DM_STAGES = 3;     // tiles of a warp under way or in use: two loads always in flight


// 2^x by the special function unit (two units in the last place; 2^-inf = 0)
__device__ __forceinline__ float dm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// transpose of an 8 x 8 tile of 16-bit values held across the warp in the fragment layout of mma
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// shared memory of a CTA of W warps: queries, the warps' staging areas, their softmax state, one flag
template <int D, int W>
__host__ __device__ constexpr size_t dm_smem_bytes() {
    return 16 * D * 2 + (size_t)W * DM_STAGES * 2 * DM_TILE * D * 2 + 2 * W * 16 * sizeof(float) + 16;
}

// One (sequence, KV head, split) by a CTA of W warps.  `smem`: dm_smem_bytes<D, W>() of shared memory.
// TR: the arrangement with the keys as the M rows (G <= 8).  Every thread returns together.
template <int D, int W, bool TR>
__device__ __forceinline__ void attn_decode_item(const AttnParams& p, const int split, const int kvh, const int b,
                                                 unsigned char* smem, const int tid) {
    constexpr int DM_WARPS = W, DM_THREADS = W * 32;
    auto sync = [] { __syncthreads(); };
    constexpr int CPR = D / 8;                 // 16-byte chunks per row
    constexpr int TILE_BYTES = DM_TILE * D * 2;
    constexpr int WARP_BYTES = DM_STAGES * 2 * TILE_BYTES;   // K and V, every stage
    const int slot = p.row_slot[b];
    const int tok = p.row_q_start[b];
    const int G = p.G;
    if (slot < 0) {
        // padding row: zeros, written here when no merge kernel follows
        if (p.counters != nullptr && split == 0)
            for (int e = tid; e < G * D; e += DM_THREADS)
                static_cast<__nv_bfloat16*>(p.out)[((size_t)tok * p.n_q + kvh * G) * D + e] = __float2bfloat16_rn(0.f);
        return;
    }
    const int ctx = p.row_ctx_len[b];
    int lo = p.window > 0 ? max(0, ctx - p.window + 1) : 0;
    int hi = ctx + 1;                           // the new token's own key is already in the cache
    if (p.n_splits > 1) {
        lo = max(lo, split * p.split_len);
        hi = min(hi, (split + 1) * p.split_len);
    }

    unsigned char* q_s = smem;                                  // [16][D] bf16, swizzled
    unsigned char* kv_s = smem + 16 * D * 2;                    // per warp: [stage][K|V][16][D]
    float* m_s = reinterpret_cast<float*>(kv_s + DM_WARPS * WARP_BYTES);   // [warps][16]
    float* l_s = m_s + DM_WARPS * 16;
    int* is_last = reinterpret_cast<int*>(l_s + DM_WARPS * 16);

    const int lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* qg = static_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(p.k_pool);
    const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(p.v_pool);

    // queries: rows 0..G-1 are the heads of this KV head, the rest zero.  Their loads are issued here
    // and land in shared memory after the first key tiles have been asked for.
    constexpr int Q_PER_THREAD = (16 * CPR + DM_THREADS - 1) / DM_THREADS;
    uint4 q_regs[Q_PER_THREAD];
#pragma unroll
    for (int i = 0; i < Q_PER_THREAD; ++i) {
        const int c = tid + i * DM_THREADS;
        const int r = c / CPR, cc = c - r * CPR;
        q_regs[i] = make_uint4(0, 0, 0, 0);
        // L2 load: in the persistent kernel another CTA wrote the queries just before
        if (c < 16 * CPR && r < G)
            q_regs[i] = __ldcg(reinterpret_cast<const uint4*>(qg + ((size_t)tok * p.n_q + kvh * G + r) * D + cc * 8));
    }

    // O: heads as rows [16 heads][D] (two rows per thread), or TR: dims as rows [D][8 heads] (two heads per thread)
    constexpr int NO = TR ? D / 16 : D / 8;
    float o[NO][4];
#pragma unroll
    for (int i = 0; i < NO; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};   // heads lane/4 and lane/4 + 8; TR: heads 2 (lane%4) and + 1
    float l_run[2] = {0.f, 0.f};               // per-thread partial sums (its share of each tile's keys)
    const float scale_log2 = p.scale * 1.4426950408889634f;

    unsigned char* my = kv_s + warp * WARP_BYTES;
    const int bs = p.block_size;
    const int bs_shift = (bs & (bs - 1)) == 0 ? __ffs(bs) - 1 : -1;     // powers of two: shift and mask
    const bool tile_in_block = bs_shift >= 4;                           // a 16-key tile then lies in one block
    const int first_tile = lo / DM_TILE;
    const int n_tiles = hi > lo ? (hi - 1) / DM_TILE - first_tile + 1 : 0;

    int n_mine = 0;
    for (int j = warp; j < n_tiles; j += DM_WARPS) ++n_mine;
    // Blocks of this warp's tiles, 32 at a time, one per lane: fetched together and ahead of use, so that
    // no tile's copies wait for a table entry of their own.
    int blk_base = 0, blk_reg = -1;
    auto fetch_blocks = [&](int base) {
        blk_base = base;
        blk_reg = -1;
        const int i = base + lane;
        if (tile_in_block && i < n_mine)
            blk_reg = p.block_table[(size_t)slot * p.max_blocks + (((first_tile + warp + i * DM_WARPS) * DM_TILE) >> bs_shift)];
    };
    fetch_blocks(0);

    // Per-lane constants of the main loop (an address then costs one add): where this lane's 16-byte chunks of
    // a tile go in shared memory, and where its ldmatrix rows of K and of V start.
    uint32_t chunk_off[DM_TILE * CPR / 32];
#pragma unroll
    for (int u = 0; u < DM_TILE * CPR / 32; ++u) {
        const int c = u * 32 + lane;
        chunk_off[u] = (uint32_t)swz<D>(c / CPR, c % CPR);
    }
    uint32_t k_off[D / 16], v_off[D / 16];
    {
        const int mi = lane >> 3;
        // K as the B operand (keys 0-7: dims lo, hi; keys 8-15: dims lo, hi) or, TR, as the A operand (dims lo:
        // keys 0-7, 8-15; dims hi: keys 0-7, 8-15); V the other way round
        const int rk = (TR ? (mi & 1) : (mi >> 1)) * 8 + (lane & 7), rv = (TR ? (mi >> 1) : (mi & 1)) * 8 + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            k_off[kk] = (uint32_t)swz<D>(rk, kk * 2 + (TR ? (mi >> 1) : (mi & 1)));
            v_off[kk] = (uint32_t)swz<D>(rv, kk * 2 + (TR ? (mi & 1) : (mi >> 1)));
        }
    }
    const uint32_t my_u32 = smem_u32(my);

    // stage the warp's i-th 16-key tile (keys and values); called with i ascending
    auto issue = [&](int i, int stage) {
        const int j = warp + i * DM_WARPS;
        const int t0 = (first_tile + j) * DM_TILE;
        unsigned char* ks = my + stage * 2 * TILE_BYTES;
        unsigned char* vs = ks + TILE_BYTES;
        int tile_blk = -1, tile_off = 0;
        if (tile_in_block) {
            if (i >= blk_base + 32) fetch_blocks(i);
            tile_blk = __shfl_sync(0xffffffffu, blk_reg, i - blk_base);
            tile_off = t0 & (bs - 1);
            if (t0 >= lo && t0 + DM_TILE <= hi && tile_blk >= 0 && tile_blk < p.num_blocks) {
                // the usual case, a whole tile inside one block: one base address, constant offsets per lane
                // (the address arithmetic of the general path below cost more than the tile's tensor work)
                // the tile is DM_TILE * D contiguous elements in each pool: chunk c of the tile lies 16 c bytes in
                const size_t base = (((size_t)tile_blk * p.n_kv + kvh) * bs + tile_off) * D + lane * 8;
                const __nv_bfloat16* kb = kp + base;
                const __nv_bfloat16* vb = vp + base;
                const uint32_t ks32 = my_u32 + stage * 2 * TILE_BYTES, vs32 = ks32 + TILE_BYTES;
#pragma unroll
                for (int u = 0; u < DM_TILE * CPR / 32; ++u) {
                    cp_async16(ks32 + chunk_off[u], kb + u * 256, 16);
                    cp_async16(vs32 + chunk_off[u], vb + u * 256, 16);
                }
                cp_async_commit();
                return;
            }
        }
        // tiles at the edges of the range, small or odd block sizes, bad table entries: chunk by chunk
#pragma unroll
        for (int u = 0; u < DM_TILE * CPR / 32; ++u) {
            const int c = u * 32 + lane;
            const int r = c / CPR, cc = c - r * CPR;
            const int t = t0 + r;
            const __nv_bfloat16* ksrc = kp;
            const __nv_bfloat16* vsrc = vp;
            int bytes = 0;
            if (t >= lo && t < hi) {
                int blk, in_blk;
                if (tile_in_block) { blk = tile_blk; in_blk = tile_off + r; }
                else if (bs_shift >= 0) { blk = p.block_table[(size_t)slot * p.max_blocks + (t >> bs_shift)]; in_blk = t & (bs - 1); }
                else { const int col = t / bs; blk = p.block_table[(size_t)slot * p.max_blocks + col]; in_blk = t - col * bs; }
                if (blk < 0 || blk >= p.num_blocks) {
                    set_status(p.status, STATUS_BAD_BLOCK);
                } else {
                    const size_t off = (((size_t)blk * p.n_kv + kvh) * bs + in_blk) * D + cc * 8;
                    ksrc = kp + off;
                    vsrc = vp + off;
                    bytes = 16;
                }
            }
            cp_async16(smem_u32(ks + swz<D>(r, cc)), ksrc, bytes);     // 0 bytes: the chunk is zero-filled
            cp_async16(smem_u32(vs + swz<D>(r, cc)), vsrc, bytes);
        }
        cp_async_commit();
    };

    // prologue: the first DM_STAGES - 1 tiles (an empty group keeps the count uniform)
#pragma unroll
    for (int st = 0; st < DM_STAGES - 1; ++st) {
        if (st < n_mine) issue(st, st);
        else cp_async_commit();
    }
    // now the queries: to shared memory, and from there as tensor-core fragments
#pragma unroll
    for (int i = 0; i < Q_PER_THREAD; ++i) {
        const int c = tid + i * DM_THREADS;
        const int r = c / CPR, cc = c - r * CPR;
        if (c < 16 * CPR) *reinterpret_cast<uint4*>(q_s + swz<D>(r, cc)) = q_regs[i];
    }
    sync();
    // queries as tensor-core fragments, kept in registers: the A operand [16 heads][16 dims] per k-step, or, TR,
    // the B operand Q^T [16 dims][8 heads] (rows 0-7 of the query tile only: half the registers)
    uint32_t qf[TR ? D / 32 : D / 16][4];
    const int q_mi = lane >> 3;
    if (TR) {
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks)        // four 8 x 8 tiles: heads 0-7, dims 32 ks + 8 mi ..
            ldmatrix_x4(smem_u32(q_s + swz<D>(lane & 7, ks * 4 + q_mi)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    } else {
        const int q_r = (q_mi & 1) * 8 + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
            ldmatrix_x4(smem_u32(q_s + swz<D>(q_r, ks * 2 + (q_mi >> 1))), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    for (int i = 0; i < n_mine; ++i) {
        const int j = warp + i * DM_WARPS;
        cp_async_wait<DM_STAGES - 2>();       // tile i has landed
        __syncwarp();
        // refill the stage that iteration i - 1 finished with
        if (i + DM_STAGES - 1 < n_mine) issue(i + DM_STAGES - 1, (i + DM_STAGES - 1) % DM_STAGES);
        else cp_async_commit();
        const uint32_t ks32 = my_u32 + (i % DM_STAGES) * 2 * TILE_BYTES, vs32 = ks32 + TILE_BYTES;

        const int t0 = (first_tile + j) * DM_TILE;
        if constexpr (TR) {
            // S^T = K Q^T: rows = the 16 keys, columns = 8 heads.  This thread: keys lane/4 and lane/4 + 8,
            // heads 2 (lane%4) and 2 (lane%4) + 1.
            float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};     // two chains of MMAs, added up below
#pragma unroll
            for (int kk = 0; kk < D / 16; kk += 2) {
                uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
                ldmatrix_x4(ks32 + k_off[kk], a0, a1, a2, a3);
                ldmatrix_x4(ks32 + k_off[kk + 1], c0, c1, c2, c3);
                mma_bf16(s, a0, a1, a2, a3, qf[kk >> 1][0], qf[kk >> 1][1]);
                mma_bf16(s2, c0, c1, c2, c3, qf[kk >> 1][2], qf[kk >> 1][3]);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] += s2[e];
            // mask (only a split's first and last tile can hold keys outside [lo, hi)) and online softmax, base 2,
            // the maximum kept in units of the raw scores (scale > 0)
            if (t0 < lo || t0 + DM_TILE > hi) {
                const int ka = t0 + (lane >> 2), kb = ka + 8;
                if (ka < lo || ka >= hi) s[0] = s[1] = -INFINITY;
                if (kb < lo || kb >= hi) s[2] = s[3] = -INFINITY;
            }
            float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
            float alpha[2], m_off[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
                const float m_new = fmaxf(m_run[h], mx[h]);
                alpha[h] = m_new == -INFINITY ? 1.f : dm_ex2((m_run[h] - m_new) * scale_log2);   // m_run = -inf: 0
                m_run[h] = m_new;
                m_off[h] = m_new == -INFINITY ? 0.f : m_new * scale_log2;                        // all masked so far: P = 2^-inf = 0
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] = dm_ex2(fmaf(s[e], scale_log2, -m_off[e & 1]));
            l_run[0] = l_run[0] * alpha[0] + s[0] + s[2];
            l_run[1] = l_run[1] * alpha[1] + s[1] + s[3];
            // P^T as the B operand [16 keys][8 heads] of the second product: the two 8 x 8 tiles transposed
            const uint32_t pb0 = movmatrix_trans(pack_bf16(s[0], s[1])), pb1 = movmatrix_trans(pack_bf16(s[2], s[3]));
            // O^T = O^T * alpha + V^T P^T: rows = dims (16 per MMA), columns = heads
            const bool rescale = __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f);
#pragma unroll
            for (int np = 0; np < D / 16; ++np) {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4_trans(vs32 + v_off[np], a0, a1, a2, a3);
                if (rescale) {       // most tiles leave every running maximum as it was
                    o[np][0] *= alpha[0]; o[np][1] *= alpha[1]; o[np][2] *= alpha[0]; o[np][3] *= alpha[1];
                }
                mma_bf16(o[np], a0, a1, a2, a3, pb0, pb1);
            }
        } else {
            // S = Q K^T for 16 keys: two n-tiles of 8 keys
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    #pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(ks32 + k_off[kk], b0, b1, b2, b3);
                mma_bf16(s[0], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
                mma_bf16(s[1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
            }
            // mask and online softmax (base 2, the maximum kept in units of the raw scores: scale > 0);
            // this thread's keys: t0 + (lane%4)*2 + {0,1} (+8).  Only a split's first and last tile can hold
            // keys outside [lo, hi).
            if (t0 < lo || t0 + DM_TILE > hi) {
    #pragma unroll
                for (int nt = 0; nt < 2; ++nt)
    #pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int t = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        if (t < lo || t >= hi) s[nt][e] = -INFINITY;
                    }
            }
            float mx[2];
            mx[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
            mx[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
            float alpha[2], m_off[2];
    #pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                alpha[h] = m_new == -INFINITY ? 1.f : dm_ex2((m_run[h] - m_new) * scale_log2);   // m_run = -inf: 0
                m_run[h] = m_new;
                m_off[h] = m_new == -INFINITY ? 0.f : m_new * scale_log2;                        // all masked so far: P = 2^-inf = 0
            }
            float rs[2] = {0.f, 0.f};
    #pragma unroll
            for (int nt = 0; nt < 2; ++nt)
    #pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = dm_ex2(fmaf(s[nt][e], scale_log2, -m_off[e >> 1]));
                    s[nt][e] = pv;
                    rs[e >> 1] += pv;
                }
            l_run[0] = l_run[0] * alpha[0] + rs[0];
            l_run[1] = l_run[1] * alpha[1] + rs[1];
            const uint32_t pa0 = pack_bf16(s[0][0], s[0][1]), pa1 = pack_bf16(s[0][2], s[0][3]);
            const uint32_t pa2 = pack_bf16(s[1][0], s[1][1]), pa3 = pack_bf16(s[1][2], s[1][3]);
            // O = O * alpha + P V
            const bool rescale = __any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f);
    #pragma unroll
            for (int np = 0; np < D / 16; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(vs32 + v_off[np], b0, b1, b2, b3);
                float* oa = o[np * 2];
                float* ob = o[np * 2 + 1];
                if (rescale) {       // most tiles leave every running maximum as it was
                    oa[0] *= alpha[0]; oa[1] *= alpha[0]; oa[2] *= alpha[1]; oa[3] *= alpha[1];
                    ob[0] *= alpha[0]; ob[1] *= alpha[0]; ob[2] *= alpha[1]; ob[3] *= alpha[1];
                }
                mma_bf16(oa, pa0, pa1, pa2, pa3, b0, b1);
                mma_bf16(ob, pa0, pa1, pa2, pa3, b2, b3);
            }
        }
        __syncwarp();      // every lane is done with this stage before it is refilled
    }

    cp_async_wait<0>();
    if (p.pf_bytes != 0 && tid == DM_THREADS - 1) l2_prefetch_share(p.pf_ptr, p.pf_bytes);
    // per-warp results to shared memory: O as float [16][D] in the warp's own staging area
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if constexpr (TR) {            // the lanes that share a head hold different keys: lane/4
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
        } else {
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
            l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
        }
    }
    float* o_w = reinterpret_cast<float*>(my);
    if constexpr (TR) {
        const int h0 = (lane & 3) * 2, d0 = lane >> 2;        // this thread's heads h0, h0 + 1 and dims 16 np + d0 (+ 8)
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
            o_w[h0 * D + np * 16 + d0] = o[np][0];
            o_w[(h0 + 1) * D + np * 16 + d0] = o[np][1];
            o_w[h0 * D + np * 16 + d0 + 8] = o[np][2];
            o_w[(h0 + 1) * D + np * 16 + d0 + 8] = o[np][3];
        }
        if (d0 == 0) {
            m_s[warp * 16 + h0] = m_run[0];  m_s[warp * 16 + h0 + 1] = m_run[1];
            l_s[warp * 16 + h0] = l_run[0];  l_s[warp * 16 + h0 + 1] = l_run[1];
        }
    } else {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            *reinterpret_cast<float2*>(o_w + r0 * D + nt * 8 + c0) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(o_w + (r0 + 8) * D + nt * 8 + c0) = make_float2(o[nt][2], o[nt][3]);
        }
        if ((lane & 3) == 0) {
            m_s[warp * 16 + r0] = m_run[0];  m_s[warp * 16 + r0 + 8] = m_run[1];
            l_s[warp * 16 + r0] = l_run[0];  l_s[warp * 16 + r0 + 8] = l_run[1];
        }
    }
    sync();

    // merge the warps; one (head, dim) pair per thread step
    constexpr float LN2 = 0.6931471805599453f;
    for (int e = tid; e < G * D; e += DM_THREADS) {
        const int r = e / D, j = e - r * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w) m = fmaxf(m, m_s[w * 16 + r]);
        float l = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < DM_WARPS; ++w) {
            const float mw = m_s[w * 16 + r];
            const float f = mw == -INFINITY ? 0.f : exp2f((mw - m) * scale_log2);      // the maxima are raw scores
            l += l_s[w * 16 + r] * f;
            a += reinterpret_cast<const float*>(kv_s + w * WARP_BYTES)[r * D + j] * f;
        }
        const size_t row = (size_t)tok * p.n_q + kvh * G + r;
        if (p.n_splits > 1) {
            const size_t pi = row * p.n_splits + split;
            p.part_acc[pi * D + j] = a;
            if (j == 0) { p.part_m[pi] = m * scale_log2 * LN2; p.part_l[pi] = l; }   // natural-log units for the merge
        } else {
            static_cast<__nv_bfloat16*>(p.out)[row * D + j] = __float2bfloat16_rn(l > 0.f ? a / l : 0.f);
        }
    }
    if (p.n_splits == 1 || p.counters == nullptr) return;

    // The CTA that finishes last for this (sequence, KV head) merges the splits: no CTA waits for
    // another.  Its partial results are made visible device-wide before it announces itself.
    __threadfence();
    sync();
    if (tid == 0) {
        int* cnt = p.counters + (size_t)b * p.n_kv + kvh;
        const int old = atomicAdd(cnt, 1);
        *is_last = old == p.n_splits - 1;
        if (*is_last) *cnt = 0;                      // ready for the next launch
    }
    sync();
    if (!*is_last) return;
    __threadfence();
    // The staging area is free now.  First every (head, split)'s maximum and sum, fetched in one round trip;
    // then the weights e^(m_s - m) / l, one warp per head; then the weighted sum of the splits' outputs.
    const int ns = p.n_splits;
    float* wgt = reinterpret_cast<float*>(kv_s);     // [G][ns]: the sums, then the weights
    float* mx_s = wgt + G * ns;                      // [G][ns]: the maxima (-inf for an empty split)
    // four output dims per thread and pass; the loads of up to MB splits are in flight together.  Those of this
    // thread's first pass are asked for now, before the weights exist: they need none, and so the round trip
    // for the splits' outputs passes under the one for their maxima and sums.
    // (Only in the eight-warp form, which exists for many splits: the registers this takes made the four-warp
    // form, whose merges are short, slower.)
    constexpr bool AHEAD = W == 8;
    constexpr int MB = 16;
    const int n_items = G * (D / 4);
    float4 v0[AHEAD ? MB : 1];
    if (AHEAD && tid < n_items) {
        const int r = tid / (D / 4), j4 = tid - r * (D / 4);
        const float4* pa = reinterpret_cast<const float4*>(p.part_acc + ((size_t)tok * p.n_q + kvh * G + r) * ns * D) + j4;
#pragma unroll
        for (int u = 0; u < MB; ++u)
            if (u < ns) v0[u] = __ldcg(pa + (size_t)u * (D / 4));
    }
    for (int e = tid; e < G * ns; e += DM_THREADS) {
        const int r = e / ns, s = e - r * ns;
        const size_t idx = ((size_t)tok * p.n_q + kvh * G + r) * ns + s;
        const float ls = __ldcg(p.part_l + idx), ms = __ldcg(p.part_m + idx);
        wgt[e] = ls;
        mx_s[e] = ls > 0.f ? ms : -INFINITY;
    }
    sync();
    for (int r = warp; r < G; r += DM_WARPS) {
        float m = -INFINITY;
        for (int s = lane; s < ns; s += 32) m = fmaxf(m, mx_s[r * ns + s]);
        m = warp_max(m);
        float lsum = 0.f;
        for (int s = lane; s < ns; s += 32) {
            const float ls = wgt[r * ns + s];
            const float w = ls > 0.f ? expf(mx_s[r * ns + s] - m) : 0.f;
            wgt[r * ns + s] = w;
            lsum += ls * w;
        }
        lsum = warp_sum(lsum);
        const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        for (int s = lane; s < ns; s += 32) wgt[r * ns + s] *= inv;
    }
    sync();
    for (int e = tid; e < n_items; e += DM_THREADS) {
        const int r = e / (D / 4), j4 = e - r * (D / 4);
        const size_t row = (size_t)tok * p.n_q + kvh * G + r;
        const float4* pa = reinterpret_cast<const float4*>(p.part_acc + row * ns * D) + j4;
        const float* w = wgt + r * ns;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < ns; s0 += MB) {
            float4 v[MB];
            if (AHEAD && e == tid && s0 == 0) {
#pragma unroll
                for (int u = 0; u < MB; ++u) v[u] = v0[u];
            } else {
#pragma unroll
                for (int u = 0; u < MB; ++u)
                    if (s0 + u < ns) v[u] = __ldcg(pa + (size_t)(s0 + u) * (D / 4));
            }
#pragma unroll
            for (int u = 0; u < MB; ++u)
                if (s0 + u < ns) {
                    const float ws = w[s0 + u];
                    a.x = fmaf(v[u].x, ws, a.x); a.y = fmaf(v[u].y, ws, a.y);
                    a.z = fmaf(v[u].z, ws, a.z); a.w = fmaf(v[u].w, ws, a.w);
                }
        }
        uint2 o2;
        *reinterpret_cast<__nv_bfloat162*>(&o2.x) = __floats2bfloat162_rn(a.x, a.y);
        *reinterpret_cast<__nv_bfloat162*>(&o2.y) = __floats2bfloat162_rn(a.z, a.w);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + row * D + j4 * 4) = o2;
    }
}

}  // namespace fd
