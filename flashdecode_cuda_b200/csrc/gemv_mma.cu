// Weight-streaming matrix product for decode steps (bfloat16):
//     out[m, n] = sum_k x[m, k] W[n, k]        M <= 64 rows of x, W [N, K] row-major
//
// At M <= 64 the product is bound by reading W once from HBM, so the kernel is
// built around that stream.  The roles of the operands are swapped for the
// tensor cores: 16 rows of W are the M side of mma.m16n8k16 and 8 rows of x the
// N side, so no tensor work is wasted on padding a tiny batch up to a 64- or
// 128-row tile.  Each thread loads 16 contiguous bytes of its W row straight
// from global memory into registers (W is never staged in shared memory): with
// the k index permuted identically on both operands, those 8 values ARE two A
// fragments, and 16 bytes of an x row (from global memory, which L1/L2 serve)
// are the matching B fragments.  Several such loads are in flight per thread
// before the first is used, and nothing waits at the start of the kernel.
//
// A CTA has W warps (8 or 16) arranged as WR row tiles x WK slices of K: wide
// matrices use 32 rows per CTA, narrow ones 16 rows per CTA with all warps
// slicing K (their partial sums added in shared memory in a fixed order), so
// that N / (16 WR) CTAs cover the GPU without partial sums in global memory.
// grid.y splits K across CTAs as well.  Outputs:
//   * mode 0: float partial sums [split, M, N] that a consumer adds up;
//   * modes 1, 2: out = sum (+ bias) as bfloat16 or float.  With n_splits > 1
//     the CTAs of one row block form a thread-block cluster; each leaves its
//     partial tile in its own shared memory and the cluster's first CTA adds
//     them through distributed shared memory in rank order, so no partial sum
//     ever goes to global memory;
//   * gated: W rows come in tiles of 16 = 8 gate rows then 8 up rows, so a
//     thread holds gate_i and up_i together and writes silu(gate_i) * up_i.
#include <cooperative_groups.h>

#include "gemv_common.cuh"

namespace fd {

constexpr int GV_WARPS = 8;
constexpr int GV_THREADS = GV_WARPS * 32;

// ROPE: the instantiation for mode 4, which keeps its epilogue's inputs in registers across the main loop
// (the other modes must not pay for those registers with a CTA less per SM).
template <int NT, int WK, int UNROLL, bool CLUSTER, int W, bool ROPE>
__global__ void __launch_bounds__(W * 32, (!ROPE && W == 8 && NT == 2) ? 4 : 0)     // 16 rows of x: four 8-warp CTAs per SM (at most 64 registers)
gemv_mma_kernel(const GemvParams p, const RopeArgs ra) {
    constexpr int WR = W / WK;
    __shared__ float red[WK > 1 ? W * 32 * NT * 4 : 1];
    __shared__ float ctile[CLUSTER ? WR * 32 * NT * 4 : 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wr = warp / WK, wk = warp % WK;
    const int split = blockIdx.y;
    const int k0 = split * p.k_per_split;
    const int k1 = min(p.K, k0 + p.k_per_split);
    const int n_chunks = (k1 - k0) >> 5;              // chunks of 32 k in this CTA's range

    const int r = lane >> 2, q = lane & 3;
    const int row0 = (blockIdx.x * WR + wr) * 16 + r;           // this thread's W rows: row0 and row0 + 8
    // rows beyond N (and x rows beyond M) read the last valid row; their results are never stored
    const __nv_bfloat16* w0 = p.w + (size_t)min(row0, p.N - 1) * p.K + k0 + q * 8;
    const __nv_bfloat16* w1 = p.w + (size_t)min(row0 + 8, p.N - 1) * p.K + k0 + q * 8;
    const __nv_bfloat16* xb[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xb[nt] = p.x + (size_t)min(nt * 8 + r, p.M - 1) * p.K + k0 + q * 8;

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    // this warp takes chunks wk, wk + WK, ...: at any moment the WK warps of a row tile read
    // neighbouring 64-byte pieces of the same rows
    pdl_launch_dependents();
    pdl_wait();
    RopePre<NT> pre;
    if (ROPE && wk == 0) rope_prefetch_first<NT>(p, ra, q, pre);
    bool pre_done = !ROPE || wk != 0;       // the rest of the epilogue's inputs: once, behind the first weight loads
    int kc = wk;
    for (; kc + (UNROLL - 1) * WK < n_chunks; kc += UNROLL * WK) {
        uint4 a[UNROLL], b[UNROLL], xv[UNROLL][NT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            a[u] = ldg_stream(w0 + (kc + u * WK) * 32);
            b[u] = ldg_stream(w1 + (kc + u * WK) * 32);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
                xv[u][nt] = __ldg(reinterpret_cast<const uint4*>(xb[nt] + (kc + u * WK) * 32));
        if (!pre_done) { rope_prefetch_rest<NT>(p, ra, row0, r, pre); pre_done = true; }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mma16816(acc[nt], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][nt].x, xv[u][nt].y);
                mma16816(acc[nt], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][nt].z, xv[u][nt].w);
            }
        }
    }
    // The rest of the range (fewer than UNROLL chunks for this warp) in groups of REST chunks, again with every
    // load of a group issued before the first is used: one chunk at a time, each waiting for its own load, cost
    // a trip to memory per chunk - for K = 1536 and 16 warps slicing K that was all three of a warp's chunks.
    // A group's places beyond the range read the range's last chunk once more (it is in L2) against zeros for x.
    constexpr int REST = NT > 1 ? 2 : (UNROLL > 4 ? 4 : (UNROLL > 1 ? UNROLL - 1 : 1));     // NT 2 with groups of 4: 78 registers, a CTA less per SM
    for (; kc < n_chunks; kc += REST * WK) {
        uint4 a[REST], b[REST], xv[REST][NT];
#pragma unroll
        for (int u = 0; u < REST; ++u) {
            const int c = min(kc + u * WK, n_chunks - 1);
            a[u] = ldg_stream(w0 + c * 32);
            b[u] = ldg_stream(w1 + c * 32);
        }
#pragma unroll
        for (int u = 0; u < REST; ++u) {
            const bool in = kc + u * WK < n_chunks;            // the same for all lanes of the warp
            const int c = min(kc + u * WK, n_chunks - 1);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                xv[u][nt] = __ldg(reinterpret_cast<const uint4*>(xb[nt] + c * 32));
                if (!in) xv[u][nt] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        if (!pre_done) { rope_prefetch_rest<NT>(p, ra, row0, r, pre); pre_done = true; }
#pragma unroll
        for (int u = 0; u < REST; ++u) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mma16816(acc[nt], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][nt].x, xv[u][nt].y);
                mma16816(acc[nt], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][nt].z, xv[u][nt].w);
            }
        }
    }

    if (!pre_done) rope_prefetch_rest<NT>(p, ra, row0, r, pre);       // a warp without a chunk of its own
    if (p.pf_bytes != 0 && tid == W * 32 - 1) l2_prefetch_share(p.pf_ptr, p.pf_bytes);
    if (WK > 1) {
        // add the K slices of a row tile in the order wk = 0, 1, ...
        float* mine = red + (warp * 32 + lane) * NT * 4;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) mine[nt * 4 + e] = acc[nt][e];
        __syncthreads();
        if (wk == 0) {
#pragma unroll
            for (int k = 1; k < WK; ++k) {
                const float* other = red + ((warp + k) * 32 + lane) * NT * 4;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[nt][e] += other[nt * 4 + e];
            }
        }
    }
    if (CLUSTER) {
        // the CTAs of a cluster hold the K splits of the same rows: rank 0 adds the others'
        // tiles out of their shared memory, in rank order
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        float* tile = ctile + (wr * 32 + lane) * NT * 4;
        if (wk == 0 && cluster.block_rank() != 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) tile[nt * 4 + e] = acc[nt][e];
        }
        cluster.sync();
        if (wk == 0 && cluster.block_rank() == 0) {
            const int n = cluster.num_blocks();
            for (int rk = 1; rk < n; ++rk) {
                const float* remote = cluster.map_shared_rank(tile, rk);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[nt][e] += remote[nt * 4 + e];
            }
        }
        cluster.sync();                          // the others' shared memory stays alive until it has been read
        if (cluster.block_rank() != 0) return;
    }
    if (WK > 1 && wk != 0) return;

    gemv_epilogue<NT, ROPE>(p, ra, acc, row0, split, r, q, pre);
}

template <int NT, int WK, int UNROLL, int W = GV_WARPS>
static int launch_gemv(const GemvParams& p, const RopeArgs& ra, cudaStream_t stream) {
    constexpr int rows = 16 * (W / WK);
    dim3 grid((p.N + rows - 1) / rows, p.n_splits);
    if (p.mode == 4) {
        if (p.n_splits > 1)
            return launch("gemv_mma", gemv_mma_kernel<NT, WK, UNROLL, true, W, true>, grid, dim3(W * 32), 0, stream,
                          dim3(1, p.n_splits, 1), p, ra);
        return launch("gemv_mma", gemv_mma_kernel<NT, WK, UNROLL, false, W, true>, grid, dim3(W * 32), 0, stream,
                      dim3(1, 1, 1), p, ra);
    }
    if (p.n_splits > 1 && p.mode != 0)
        return launch("gemv_mma", gemv_mma_kernel<NT, WK, UNROLL, true, W, false>, grid, dim3(W * 32), 0, stream,
                      dim3(1, p.n_splits, 1), p, ra);
    return launch("gemv_mma", gemv_mma_kernel<NT, WK, UNROLL, false, W, false>, grid, dim3(W * 32), 0, stream,
                  dim3(1, 1, 1), p, ra);
}

// Measured on B200 (graph-timed, weights beyond L2): wide matrices stream best with 32 rows
// per CTA (4 or more CTAs per SM), narrow ones with 16 rows per CTA plus a split of K.
static int gemv_slots() {            // 8-warp CTAs of at most 64 registers that the GPU holds at once
    static int slots = 0;
    if (slots == 0) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        slots = 4 * sms;
    }
    return slots;
}
// 32 rows per CTA (4 warps slicing K) for wide matrices, and for narrower ones whose 16-row CTAs times their splits
// of K would not fit the GPU at once: a second, nearly empty wave cost a fifth of the kernel's time (down projection
// of Qwen2.5-7B, 3584 x 18944: 672 CTAs of 16 rows 30.1 us, 560 CTAs of 32 rows 23.8 us; o projection of
// Qwen2.5-14B 16.8 -> 13.3 us).
static int pick_wk(int N, int n_splits) {
    if (N >= 8192) return 4;
    return (long long)((N + 15) / 16) * n_splits > gemv_slots() ? 4 : 8;
}

template <int NT, int UNROLL>
static int launch_gemv_wk(const GemvParams& p, const RopeArgs& ra, cudaStream_t stream) {
    if constexpr (NT <= 2) {
        // narrow and not split across CTAs: 16 warps share the 16 rows of a CTA (measured 4.2 us against
        // 5.2 us with 8 warps for the q/k/v and o projections of Qwen2.5-1.5B)
        if (p.n_splits == 1 && pick_wk(p.N, 1) == 8) return launch_gemv<NT, 16, (UNROLL > 4 ? 4 : UNROLL), 16>(p, ra, stream);
    }
    if (pick_wk(p.N, p.n_splits) == 4) return launch_gemv<NT, 4, UNROLL>(p, ra, stream);
    return launch_gemv<NT, 8, UNROLL>(p, ra, stream);
}

static int run_gemv(GemvParams& p, const RopeArgs& ra, cudaStream_t stream) {
    const int chunks = p.K / 32;
    p.k_per_split = ((chunks + p.n_splits - 1) / p.n_splits) * 32;
    FD_REQUIRE((long long)p.k_per_split * (p.n_splits - 1) < p.K, -2, "gemv: %d splits leave one empty for K=%d", p.n_splits, p.K);
    const int nt = p.M <= 8 ? 1 : (p.M <= 16 ? 2 : (p.M <= 32 ? 4 : 8));
    switch (nt) {
        case 1: return launch_gemv_wk<1, 8>(p, ra, stream);
        case 2: return launch_gemv_wk<2, 8>(p, ra, stream);     // 8 chunks in flight as well: 13.5 against 20.6 us for gate/up at 16 rows
        case 4: return launch_gemv_wk<4, 2>(p, ra, stream);
        default: return launch_gemv_wk<8, 1>(p, ra, stream);
    }
}

}  // namespace fd

using namespace fd;

// How many splits of K (each a multiple of 32 wide, as CTAs of their own) the
// product would use to reach about `target_ctas` CTAs; 1 when the rows alone
// give enough.  0: sizes not taken (M > 64, K not a multiple of 32): use another
// matrix product.
extern "C" int fd_gemv_splits(int M, int N, int K, int target_ctas, int allow_split) {
    if (M < 1 || M > 64 || K < 32 || K % 32 != 0 || N < 1) return 0;
    if (!allow_split) return 1;
    const int chunks = K / 32;
    // A split across CTAs costs a cluster launch and two cluster barriers (about 3 us measured on
    // B200), or partial sums for a consumer to add: worth it only while every warp of a CTA still walks 8 or more chunks.
    int cap = chunks / (8 * 8);
    if (cap > 8) cap = 8;                                 // the most CTAs a portable cluster holds
    if (cap < 1) cap = 1;
    auto splits_for = [&](int want) {                     // the splits that k ranges of a multiple of 32 give
        if (want > cap) want = cap;
        if (want < 1) want = 1;
        const int per = ((chunks + want - 1) / want) * 32;
        return (K + per - 1) / per;
    };
    const int rows = 16 * (GV_WARPS / (N >= 8192 ? 4 : 8));
    const int row_blocks = (N + rows - 1) / rows;
    int s = splits_for((target_ctas + row_blocks / 2) / row_blocks);
    // 16-row CTAs that would spill into a second wave: 32-row CTAs instead (see pick_wk), as many as fit at once
    if (N < 8192 && (long long)row_blocks * s > gemv_slots()) {
        const int rb4 = (N + 31) / 32;
        const int s4 = splits_for(gemv_slots() / rb4);
        if ((long long)rb4 * s4 <= gemv_slots() && (long long)row_blocks * s4 > gemv_slots()) s = s4;
    }
    return s;
}

// mode 0: out = float partial sums [n_splits, M, N]; 1: bf16 [M, N]; 2: float [M, N] (both with
// up to 8 splits added inside a cluster); 3: gated (rows of W in tiles of 8 gate + 8 up):
// bf16 [M, N / 2], n_splits == 1.  prefetch / prefetch_bytes (optional, 16-byte aligned): memory that a
// later kernel streams, which this kernel asks L2 for once its own loads are through.
extern "C" int fd_gemv(const void* x, const void* w, const void* bias, int bias_f32, void* out, int mode,
                       int M, int N, int K, int n_splits, const void* prefetch, unsigned long long prefetch_bytes,
                       cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    FD_REQUIRE((uintptr_t)prefetch % 16 == 0, -2, "gemv: the memory to prefetch must be 16-byte aligned");
    FD_REQUIRE(M >= 1 && M <= 64, -2, "gemv: %d rows of x; this kernel takes 1..64", M);
    FD_REQUIRE(K >= 32 && K % 32 == 0, -2, "gemv: K=%d must be a positive multiple of 32", K);
    FD_REQUIRE(n_splits >= 1 && (mode != 3 || n_splits == 1), -2, "gemv: the gated form cannot be split over K");
    FD_REQUIRE(mode == 0 || n_splits <= 8, -2, "gemv: at most 8 splits add up inside a cluster, got %d", n_splits);
    FD_REQUIRE(mode >= 0 && mode <= 3, -2, "gemv: mode %d", mode);
    FD_REQUIRE(mode != 3 || N % 16 == 0, -2, "gemv: gated output needs N (= 2 x outputs) to be a multiple of 16, got %d", N);
    FD_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0, -2, "gemv: x and W must be 16-byte aligned");
    GemvParams p;
    p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = bias; p.out = out;
    p.M = M; p.N = N; p.K = K; p.n_splits = n_splits; p.mode = mode; p.bias_f32 = bias_f32;
    p.pf_ptr = (const unsigned char*)prefetch; p.pf_bytes = prefetch ? prefetch_bytes : 0;
    RopeArgs ra = {};
    return run_gemv(p, ra, stream);
}

// The q/k/v projection of a decode step with its epilogue: bias, rotary
// encoding of q and k (float), q to q_out [M, n_q d], k and v into the paged
// cache at each token's position.  W [(n_q + 2 n_kv) d, K] and bias must have
// the rows of every q and k head in tiles of 8 dims + their 8 partners (see
// RopeArgs).  Up to 8 splits of K add up inside a cluster.  prefetch / prefetch_bytes (optional, 16-byte aligned):
// memory that a later kernel streams - the output projection's weights - which this kernel asks L2 for.
extern "C" int fd_gemv_qkv_rope(const void* x, const void* w, const void* bias, int bias_f32, void* q_out,
                                int M, int K, int n_splits, const float* cos_t, const float* sin_t, int table_len,
                                const int* tok_row, const int* tok_pos, const int* row_slot, void* k_pool,
                                void* v_pool, const int* block_table, int max_blocks, int num_blocks,
                                int block_size, int n_q, int n_kv, int d, int write_kv, int* status,
                                const void* prefetch, unsigned long long prefetch_bytes, cudaStream_t stream) {
    if (M == 0) return 0;
    FD_REQUIRE((uintptr_t)prefetch % 16 == 0, -2, "gemv_qkv_rope: the memory to prefetch must be 16-byte aligned");
    FD_REQUIRE(M >= 1 && M <= 64, -2, "gemv: %d rows of x; this kernel takes 1..64", M);
    FD_REQUIRE(K >= 32 && K % 32 == 0, -2, "gemv: K=%d must be a positive multiple of 32", K);
    FD_REQUIRE(d >= 16 && d % 16 == 0, -2, "gemv_qkv_rope: head size %d must be a multiple of 16", d);
    FD_REQUIRE(n_splits >= 1 && n_splits <= 8, -2, "gemv: at most 8 splits add up inside a cluster, got %d", n_splits);
    FD_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0, -2, "gemv: x and W must be 16-byte aligned");
    GemvParams p;
    p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.bias = bias; p.out = q_out;
    p.M = M; p.N = (n_q + 2 * n_kv) * d; p.K = K; p.n_splits = n_splits; p.mode = 4; p.bias_f32 = bias_f32;
    p.pf_ptr = (const unsigned char*)prefetch; p.pf_bytes = prefetch ? prefetch_bytes : 0;
    RopeArgs ra;
    ra.cos_t = cos_t; ra.sin_t = sin_t; ra.tok_row = tok_row; ra.tok_pos = tok_pos; ra.row_slot = row_slot;
    ra.k_pool = (__nv_bfloat16*)k_pool; ra.v_pool = (__nv_bfloat16*)v_pool; ra.block_table = block_table;
    ra.status = status; ra.table_len = table_len; ra.max_blocks = max_blocks; ra.num_blocks = num_blocks;
    ra.block_size = block_size; ra.n_q = n_q; ra.n_kv = n_kv; ra.d = d; ra.write_kv = write_kv;
    return run_gemv(p, ra, stream);
}
