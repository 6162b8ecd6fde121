// Prompt attention (many new tokens per sequence) over the paged bfloat16
// cache on the tensor cores: causal, grouped-query, variable lengths, optional
// sliding window, and the new tokens may continue a cached prefix.
//
// A CTA takes 64 consecutive query tokens of one sequence and one query head;
// each of its 4 warps owns 16 query rows.  Keys and values of the head's KV
// head stream through shared memory in tiles of 64 tokens, gathered from the
// block table with cp.async (double buffered, XOR-swizzled for ldmatrix):
//     S[16, 64] = Q[16, D] K^T      O[16, D] += P[16, 64] V[64, D]
// with the online softmax (float, base 2) between the two products, as in the
// decode kernel.  Tiles start at multiples of 64 in absolute position, so a
// query's sums do not depend on what else is in the batch.
#include <math.h>

#include "attention.cuh"
#include "mma_utils.cuh"

namespace fd {

constexpr int PM_WARPS = 4;
constexpr int PM_THREADS = PM_WARPS * 32;
constexpr int PM_BM = 64;     // query rows per CTA
constexpr int PM_BN = 64;     // keys per tile

template <int D>
__global__ void __launch_bounds__(PM_THREADS)
attn_prefill_mma_kernel(const AttnParams p) {
    constexpr int CPR = D / 8;                      // 16-byte chunks per row
    constexpr int TILE_BYTES = PM_BN * D * 2;
    // the last query tiles of a sequence see the most keys: schedule them first, so that the
    // short tiles fill the tail of the launch instead of the long ones
    const int tile = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int slot = p.row_slot[b];
    if (slot < 0) return;
    const int q_len = p.row_q_len[b];
    if (tile * PM_BM >= q_len) return;
    const int ctx = p.row_ctx_len[b];
    const int tok0 = p.row_q_start[b] + tile * PM_BM;
    const int nq = min(PM_BM, q_len - tile * PM_BM);
    const int kvh = h / p.G;
    const int p_first = ctx + tile * PM_BM;          // position of this CTA's first query
    const int hi = p_first + nq;                      // keys 0 .. last query position
    const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                        // [64][D]
    unsigned char* k_s = q_s + PM_BM * D * 2;         // [2][64][D]
    unsigned char* v_s = k_s + 2 * TILE_BYTES;        // [2][64][D]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* qg = static_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(p.k_pool);
    const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(p.v_pool);
    const int bs = p.block_size;
    const int bs_shift = (bs & (bs - 1)) == 0 ? __ffs(bs) - 1 : -1;     // block sizes that are powers of two: shift and mask

    // queries of the tile (rows beyond nq as zeros)
#pragma unroll
    for (int i = 0; i < PM_BM * CPR / PM_THREADS; ++i) {
        const int c = i * PM_THREADS + tid;
        const int r = c / CPR, cc = c - r * CPR;
        const bool ok = r < nq;
        const __nv_bfloat16* src = ok ? qg + ((size_t)(tok0 + r) * p.n_q + h) * D + cc * 8 : qg;
        cp_async16(smem_u32(q_s + swz<D>(r, cc)), src, ok ? 16 : 0);
    }
    auto issue = [&](int t0, int stage) {
        unsigned char* ks = k_s + stage * TILE_BYTES;
        unsigned char* vs = v_s + stage * TILE_BYTES;
#pragma unroll
        for (int i = 0; i < PM_BN * CPR / PM_THREADS; ++i) {
            const int c = i * PM_THREADS + tid;
            const int r = c / CPR, cc = c - r * CPR;
            const int t = t0 + r;
            const __nv_bfloat16* ksrc = kp;
            const __nv_bfloat16* vsrc = vp;
            int bytes = 0;
            if (t >= lo && t < hi) {
                const int col = bs_shift >= 0 ? t >> bs_shift : t / bs;
                const int in_blk = bs_shift >= 0 ? t & (bs - 1) : t - col * bs;
                const int blk = p.block_table[(size_t)slot * p.max_blocks + col];
                if (blk < 0 || blk >= p.num_blocks) {
                    set_status(p.status, STATUS_BAD_BLOCK);
                } else {
                    const size_t off = (((size_t)blk * p.n_kv + kvh) * bs + in_blk) * D + cc * 8;
                    ksrc = kp + off;
                    vsrc = vp + off;
                    bytes = 16;
                }
            }
            cp_async16(smem_u32(ks + swz<D>(r, cc)), ksrc, bytes);
            cp_async16(smem_u32(vs + swz<D>(r, cc)), vsrc, bytes);
        }
        cp_async_commit();
    };

    const int t_begin = (lo / PM_BN) * PM_BN;
    const int n_tiles = (hi - t_begin + PM_BN - 1) / PM_BN;
    issue(t_begin, 0);                                // this group also carries the queries

    uint32_t qf[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int row_a = warp * 16 + (lane >> 2);        // this thread's rows: row_a and row_a + 8
    const int pos_a = p_first + row_a, pos_b = pos_a + 8;
    const int w_first = p_first + warp * 16, w_last = w_first + 15;     // positions of the warp's rows

    for (int it = 0; it < n_tiles; ++it) {
        const int t0 = t_begin + it * PM_BN;
        if (it + 1 < n_tiles) {
            issue(t0 + PM_BN, (it + 1) & 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
            const int mi = lane >> 3, r = warp * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(smem_u32(q_s + swz<D>(r, ks * 2 + (mi >> 1))), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        const unsigned char* ks_ = k_s + (it & 1) * TILE_BYTES;
        const unsigned char* vs_ = v_s + (it & 1) * TILE_BYTES;
        // a tile wholly in the future of all rows of this warp contributes nothing
        const bool skip = t0 > w_last || (p.window > 0 && t0 + PM_BN - 1 < w_first - p.window + 1);
        if (!skip) {
            float s[PM_BN / 8][4];
#pragma unroll
            for (int i = 0; i < PM_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            {
                const int mi = lane >> 3;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
                    for (int np = 0; np < PM_BN / 16; ++np) {
                        const int r = np * 16 + (mi >> 1) * 8 + (lane & 7);
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4(smem_u32(ks_ + swz<D>(r, kk * 2 + (mi & 1))), b0, b1, b2, b3);
                        mma_bf16(s[np * 2], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
                        mma_bf16(s[np * 2 + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
                    }
            }
            const bool need_mask = t0 + PM_BN - 1 > w_first || t0 < lo || t0 + PM_BN > hi ||
                                   (p.window > 0 && t0 < w_last - p.window + 1);
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < PM_BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[nt][e] * scale_log2;
                    if (need_mask) {
                        const int t = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int pos = (e >> 1) ? pos_b : pos_a;
                        const bool ok = t >= lo && t < hi && t <= pos && (p.window <= 0 || pos - t < p.window);
                        if (!ok) v = -INFINITY;
                    }
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
                const float m_new = fmaxf(m_run[hh], mx[hh]);
                alpha[hh] = m_new == -INFINITY ? 1.f : exp2f(m_run[hh] - m_new);
                m_run[hh] = m_new;
            }
            float rs[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < PM_BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = m_run[e >> 1] == -INFINITY ? 0.f : exp2f(s[nt][e] - m_run[e >> 1]);
                    s[nt][e] = pv;
                    rs[e >> 1] += pv;
                }
            l_run[0] = l_run[0] * alpha[0] + rs[0];
            l_run[1] = l_run[1] * alpha[1] + rs[1];
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
            {
                const int mi = lane >> 3;
#pragma unroll
                for (int k2 = 0; k2 < PM_BN / 16; ++k2) {
                    const uint32_t pa0 = pack_bf16(s[2 * k2][0], s[2 * k2][1]), pa1 = pack_bf16(s[2 * k2][2], s[2 * k2][3]);
                    const uint32_t pa2 = pack_bf16(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
                    const uint32_t pa3 = pack_bf16(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
                    const int r = k2 * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
                    for (int np = 0; np < D / 16; ++np) {
                        uint32_t b0, b1, b2, b3;
                        ldmatrix_x4_trans(smem_u32(vs_ + swz<D>(r, np * 2 + (mi >> 1))), b0, b1, b2, b3);
                        mma_bf16(o[np * 2], pa0, pa1, pa2, pa3, b0, b1);
                        mma_bf16(o[np * 2 + 1], pa0, pa1, pa2, pa3, b2, b3);
                    }
                }
            }
        }
        __syncthreads();          // everyone is done with this stage before it is refilled
    }

#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    __nv_bfloat16* og = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = row_a + hh * 8;
        if (r >= nq) continue;
        const float inv = l_run[hh] > 0.f ? 1.f / l_run[hh] : 0.f;
        __nv_bfloat16* orow = og + ((size_t)(tok0 + r) * p.n_q + h) * D + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt)
            *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8) =
                __floats2bfloat162_rn(o[nt][hh * 2] * inv, o[nt][hh * 2 + 1] * inv);
    }
}

template <int D>
static int launch_pm(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream) {
    constexpr size_t smem = (size_t)(PM_BM + 4 * PM_BN) * D * 2;
    auto k = attn_prefill_mma_kernel<D>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-3, "attention: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int q_tiles = (max_q_len + PM_BM - 1) / PM_BM;
    if (p.n_q > 65535 || n_rows > 65535) return 1;
    dim3 grid(q_tiles, p.n_q, n_rows);
    k<<<grid, PM_THREADS, smem, stream>>>(p);
    return check_launch("attention_prefill_mma");
}

int launch_attn_prefill_mma(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream) {
    if (p.n_splits != 1) return 1;
    if (p.d == 128) return launch_pm<128>(p, n_rows, max_q_len, stream);
    if (p.d == 64) return launch_pm<64>(p, n_rows, max_q_len, stream);
    return 1;
}

}  // namespace fd
