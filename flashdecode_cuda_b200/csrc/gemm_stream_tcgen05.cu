// Weight-streaming matrix product for decode steps on the 5th-generation tensor cores (bfloat16):
//     out[m, n] = sum_k x[m, k] W[n, k]        M <= 128 rows of x, W [N, K] row-major
//
// With few rows of x the product is bound by reading W once from HBM, so the roles of the operands are
// swapped: 128 rows of W are the M side of `tcgen05.mma` and the rows of x (rounded up to a multiple of
// 16) its N side.  No tensor work goes into padding a small batch up to a 128-row tile, the accumulator
// [128 rows of W x rows of x] takes at most 128 of the 512 tensor-memory columns, and what an SM needs
// per byte of W is one TMA copy and a quarter of an MMA.
//
//  * warp 0 (one lane): TMA producer.  A stage holds `kb` k-blocks of 64: kb [128 x 64] tiles of W and kb
//    [rows of x x 64] tiles of x, each in the 128-byte-swizzled layout (rows of W beyond N, rows of x
//    beyond M and k-blocks beyond K read as zero).  An SM keeps only a handful of bulk copies in flight
//    whatever their size (measured on B200: 19 GB/s per SM with 4 KB copies, 73 with 16 KB, 136 with
//    32 KB), so the kb tiles of a stage come as ONE copy through a three-dimensional tensor map
//    (k inside a block, row, k-block) where K is a multiple of 64, and as kb two-dimensional copies
//    otherwise.  The W copies of the first ring-ful depend on nothing that an earlier kernel writes:
//    they are issued before anything else in the kernel and before the programmatic-dependent-launch
//    wait; x follows after it.
//  * warp 1 (one lane): MMA issuer, four `tcgen05.mma.cta_group::1.kind::f16` (M 128, N rows of x, K 16)
//    per stage; `tcgen05.commit` hands the stage back and, after a tile's last, the accumulator over.
//  * warps 2-5: epilogue.  `tcgen05.ld` (thread = row of W) -> float tile [row of x][128] in shared
//    memory -> the finishing loop below.
//
// Narrow matrices (q/k/v, o, down: a dozen tiles of 128 rows) would leave most SMs idle, so K is split
// over the CTAs of a thread-block cluster (2, 4 or 8, one tile per cluster): each CTA leaves its partial
// tile in its own shared memory, and after a cluster barrier CTA r finishes rows r * 128 / S .. of the
// tile, adding the S partial sums out of the S shared memories in rank order (distributed shared memory),
// so the order of the summation is fixed and no partial sum goes through global memory.  Wide matrices
// (gate/up, the output head) run unsplit: one persistent CTA per SM walks tiles, with the accumulator
// double-buffered in tensor memory so that the epilogue of one tile runs under the copies of the next.
//
// The finishing loop adds the bias and stores bfloat16 or float; or applies silu(gate) * up (rows of W in
// tiles of 8 gate + 8 up); or, for the q/k/v projection, adds the bias, rotates q and k by each token's
// position (float) and writes q to q_out and k, v into the paged cache (rows of W in the paired order
// of TcRope).  The per-token lookups (token -> sequence -> slot -> block) are done once per CTA by the
// epilogue warps while the weights stream.
//
// Every wait on an mbarrier is bounded in time (see tcgen05.cuh); the cluster barriers are hardware
// barriers among co-scheduled CTAs that every thread reaches, also after a wait has run out.
#include "tcgen05.cuh"

namespace fd {

constexpr int GS_BM = 128;                       // rows of W per tile (the M of the MMAs)
constexpr int GS_BK = 64;                        // k per stage
constexpr int GS_W_BYTES = GS_BM * GS_BK * 2;    // 16 KB
constexpr int GS_THREADS = 224;                  // warps: 0 copies of W, 1 MMA, 2-5 epilogue, 6 copies of x
constexpr int GS_MAX_NX = 128;                   // most rows of x
constexpr int GS_MAX_STAGES = 12;
constexpr int GS_MAX_KB = 4;                     // most k-blocks per stage
constexpr int GS_SMEM_LIMIT = 227 * 1024;
constexpr int GS_FIXED_SMEM = 1024 /* alignment slack */ + GS_MAX_NX * 12 /* per-token lookups */ + 512 /* barriers */;

struct GsParams {
    const void* bias;      // [N] or null
    void* out;
    int* status;
    int M, N, K;
    int mode;              // 1: bf16 [M, N]; 2: float [M, N]; 3: gated, bf16 [M, N / 2]; 4: q/k/v (TcRope), out = q_out
    int bias_f32;
    int nx;                // M rounded up to a multiple of 16: the N of the MMAs
    int splits;            // CTAs of a cluster; each takes a range of K
    int stages;
    int kb;                // k-blocks of 64 per stage
    int map3d;             // the tensor maps are three-dimensional: one copy per operand and stage
    int k_blocks;          // k-blocks of 64 in K
    int blocks_per_split;  // a multiple of kb
    int n_tiles;           // tiles of 128 rows of W
    unsigned long long wait_ns;
    int skip_last;         // tests only: the producer leaves out its very last copy
};

// Named barrier 1 of the 128 epilogue threads, plain and with an AND over a flag of every thread.
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool epi_bar_and(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"((uint32_t)v) : "memory");
    return r != 0;
}

// What the q/k/v epilogue needs to know of a token: its position (-1: skip the token) and where its key
// and value go in the pools (-1: nowhere).
__device__ __forceinline__ void gs_token(const GsParams& p, const TcRope& ra, int m, int* s_pos, long long* s_kv) {
    int pos = -1;
    long long kv = -1;
    if (m < p.M) {
        const int slot = ra.row_slot[ra.tok_row[m]];
        if (slot >= 0) {                                     // a padding row otherwise
            pos = ra.tok_pos[m];
            if (pos < 0 || pos >= ra.table_len) {
                set_status(p.status, STATUS_BAD_POSITION);
                pos = -1;
            } else if (ra.write_kv) {
                const int blk = ra.block_table[(size_t)slot * ra.max_blocks + pos / ra.block_size];
                if (blk < 0 || blk >= ra.num_blocks) set_status(p.status, STATUS_BAD_BLOCK);
                else kv = ((long long)blk * ra.n_kv * ra.block_size + pos % ra.block_size) * ra.d;
            }
        }
    }
    s_pos[m] = pos;
    s_kv[m] = kv;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&r);
}

// 16 consecutive bias values (bfloat16 or float) added to v; `at` is a multiple of 16 and the launcher
// checks the base address.
__device__ __forceinline__ void add_bias16(const GsParams& p, int at, float (&v)[16]) {
    if (p.bias == nullptr) return;
    if (p.bias_f32) {
        const float4* b4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.bias) + at);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 b = b4[i];
            v[4 * i] += b.x; v[4 * i + 1] += b.y; v[4 * i + 2] += b.z; v[4 * i + 3] += b.w;
        }
    } else {
        const uint4* b4 = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.bias) + at);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 b = b4[i];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[8 * i + 2 * j] += __low2float(h[j]); v[8 * i + 2 * j + 1] += __high2float(h[j]); }
        }
    }
}

// Finish rows r0 .. r0 + rows_here (rows_here = 1 << rows_shift, at least 16) of the tile that starts at row n0
// of W: add the partial sums that the cluster's CTAs have put into this CTA's shared memory (parts [CTA][row
// of x][rows_here]) in rank order, apply the epilogue and store.  Called by the 128 epilogue threads (et = 0 ..
// 127).  An item is (row of x, 16 consecutive rows of W): 64 bytes from each CTA's partial sums, and 16-byte
// stores - for the q/k/v projection a tile of 16 rows is 8 dims of a head and their 8 rotation partners, so a
// thread rotates and writes 8 + 8 neighbouring values; single bfloat16 stores into the cache, a block of which
// lies cold in HBM, took several microseconds.
__device__ __forceinline__ void gs_finish(const GsParams& p, const TcRope& ra, const float* parts, const int* s_pos,
                                          const long long* s_kv, const int n0, const int r0, const int rows_shift,
                                          const int et) {
    const int S = p.splits;
    const int part_stride = p.nx << rows_shift;
    const int ts = rows_shift - 4;                       // tiles of 16 rows per row of x: 1 << ts
    const int total = p.M << ts;
    const bool vec_ok = (p.N & 15) == 0;                 // every tile is whole and the rows of out are 16-byte aligned
    for (int idx = et; idx < total; idx += 128) {
        const int m = idx >> ts, t = idx & ((1 << ts) - 1);
        const int n_tile = n0 + r0 + t * 16;
        if (n_tile >= p.N) continue;
        float v[16];
        {
            const float4* src = reinterpret_cast<const float4*>(parts + (m << rows_shift) + t * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float4 a = src[i]; v[4 * i] = a.x; v[4 * i + 1] = a.y; v[4 * i + 2] = a.z; v[4 * i + 3] = a.w; }
#pragma unroll
            for (int k = 1; k < 8; ++k) {
                if (k >= S) break;
                const float4* sk = reinterpret_cast<const float4*>(parts + k * part_stride + (m << rows_shift) + t * 16);
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float4 a = sk[i]; v[4 * i] += a.x; v[4 * i + 1] += a.y; v[4 * i + 2] += a.z; v[4 * i + 3] += a.w; }
            }
        }
        if (p.mode == 1 || p.mode == 2) {
            if (vec_ok) {
                add_bias16(p, n_tile, v);
                if (p.mode == 1) {
                    uint4* o = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * p.N + n_tile);
                    o[0] = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
                    o[1] = make_uint4(pack_bf16(v[8], v[9]), pack_bf16(v[10], v[11]), pack_bf16(v[12], v[13]), pack_bf16(v[14], v[15]));
                } else {
                    float4* o = reinterpret_cast<float4*>(static_cast<float*>(p.out) + (size_t)m * p.N + n_tile);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int n = n_tile + j;
                    if (n >= p.N) break;
                    float a = v[j];
                    if (p.bias != nullptr)
                        a += p.bias_f32 ? static_cast<const float*>(p.bias)[n]
                                        : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
                    if (p.mode == 1) static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(a);
                    else static_cast<float*>(p.out)[(size_t)m * p.N + n] = a;
                }
            }
            continue;
        }
        if (p.mode == 3) {
            // 8 gate values, then the 8 up values of the same outputs (N is a multiple of 16)
            uint32_t o4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float g0 = v[2 * j], g1 = v[2 * j + 1];
                o4[j] = pack_bf16(__fdividef(g0, 1.f + __expf(-g0)) * v[8 + 2 * j], __fdividef(g1, 1.f + __expf(-g1)) * v[9 + 2 * j]);
            }
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + (size_t)m * (p.N >> 1) + (n_tile >> 1)) =
                make_uint4(o4[0], o4[1], o4[2], o4[3]);
            continue;
        }
        // mode 4: bias, rotation of q and k by the token's position, q to q_out, k and v into the cache
        const int pos = s_pos[m];
        if (pos < 0) continue;                                   // padding row or bad position
        const int d = ra.d, half = d >> 1;
        const int head = n_tile / d, in_head = n_tile - head * d;
        const bool is_v = head >= ra.n_q + ra.n_kv;
        add_bias16(p, n_tile, v);
        int j_lo, j_hi;                                          // dims of the two groups of 8 inside the head
        if (is_v) {
            j_lo = in_head; j_hi = in_head + 8;
        } else {
            j_lo = (in_head >> 4) * 8; j_hi = j_lo + half;
            const float4* c4 = reinterpret_cast<const float4*>(ra.cos_t + (size_t)pos * half + j_lo);
            const float4* s4 = reinterpret_cast<const float4*>(ra.sin_t + (size_t)pos * half + j_lo);
            const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
            const float cs[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
            const float sn[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float x1 = v[j], x2 = v[8 + j];
                v[j] = x1 * cs[j] - x2 * sn[j];
                v[8 + j] = x2 * cs[j] + x1 * sn[j];
            }
        }
        __nv_bfloat16* dst;
        if (head < ra.n_q) {
            dst = static_cast<__nv_bfloat16*>(p.out) + ((size_t)m * ra.n_q + head) * d;
        } else {
            const long long kv = s_kv[m];
            if (kv < 0) continue;
            const int kvh = is_v ? head - ra.n_q - ra.n_kv : head - ra.n_q;
            dst = (is_v ? ra.v_pool : ra.k_pool) + kv + (size_t)kvh * ra.block_size * d;
        }
        *reinterpret_cast<uint4*>(dst + j_lo) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        *reinterpret_cast<uint4*>(dst + j_hi) = make_uint4(pack_bf16(v[8], v[9]), pack_bf16(v[10], v[11]), pack_bf16(v[12], v[13]), pack_bf16(v[14], v[15]));
    }
}

__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           const GsParams p, const TcRope ra) {
    extern __shared__ unsigned char gs_smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)gs_smem_raw + 1023) & ~(uintptr_t)1023);
    const int x_bytes = p.nx * 128;                                        // one k-block of x
    const int stage_bytes = p.kb * (GS_W_BYTES + x_bytes);                  // kb tiles of W, then kb tiles of x
    const int x_off = p.kb * GS_W_BYTES;
    float* ftile = reinterpret_cast<float*>(tiles + p.stages * stage_bytes);       // [nx][128] partial sums of this CTA
    int* s_pos = reinterpret_cast<int*>(ftile + p.nx * GS_BM);
    long long* s_kv = reinterpret_cast<long long*>(s_pos + GS_MAX_NX);
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_kv + GS_MAX_NX);
    uint64_t* full = bars;                           // [stages] a stage has landed
    uint64_t* empty = bars + GS_MAX_STAGES;          // [stages] the MMAs that read a stage are done
    uint64_t* acc_full = bars + 2 * GS_MAX_STAGES;   // [2] an accumulator is complete
    uint64_t* acc_empty = acc_full + 2;              // [2] the epilogue has read it (one arrival per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.splits;
    const int rank = S > 1 ? (int)cluster_rank() : 0;
    const int cluster_id = blockIdx.x / S, n_clusters = gridDim.x / S;
    const int b_begin = rank * p.blocks_per_split;                                        // this CTA's k-blocks
    const int my_blocks = min(p.k_blocks, b_begin + p.blocks_per_split) - b_begin;         // >= 1 (the launcher checks)
    const int my_iters = (my_blocks + p.kb - 1) / p.kb;                                    // stages per tile
    const int my_tiles = cluster_id < p.n_tiles ? (p.n_tiles - cluster_id + n_clusters - 1) / n_clusters : 0;
    const int total = my_iters * my_tiles;
    const int acc_stride = p.nx <= 64 ? 64 : 128;        // columns between the two accumulators
    const uint32_t tmem_cols = 2 * acc_stride;
    // iteration `it` is k-blocks b_begin + (it % my_iters) kb .. + kb of tile cluster_id + (it / my_iters) n_clusters
    const int pre = min(p.stages, total);

    // one operand of one stage: a three-dimensional copy, or kb two-dimensional ones
    auto copy = [&](const CUtensorMap* map, uint32_t dst, uint32_t bar, int block0, int row0, int tile_bytes) {
        if (p.map3d) {
            tma_load_3d(dst, map, bar, 0, row0, block0);
        } else {
            for (int j = 0; j < p.kb; ++j) tma_load_2d(dst + j * tile_bytes, map, bar, (block0 + j) * GS_BK, row0);
        }
    };

    if (threadIdx.x == 0) {
        tma_prefetch_map(&map_w);
        tma_prefetch_map(&map_x);
        abort_flag[0] = 0;
        abort_flag[1] = 0;        // private flag of the producer's drain loop
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(s_addr(&full[s]), 2);               // the thread that copies W and the one that copies x
            mbar_init(s_addr(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_addr(&acc_full[b]), 1);
            mbar_init(s_addr(&acc_empty[b]), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // W needs nothing from an earlier kernel and nothing from the other warps: its first copies leave now
        for (int it = 0; it < pre; ++it) {
            const uint32_t fb = s_addr(&full[it]);
            mbar_expect_tx(fb, x_off);
            const int n0 = (cluster_id + (it / my_iters) * n_clusters) * GS_BM;
            copy(&map_w, s_addr(tiles + it * stage_bytes), fb, b_begin + (it % my_iters) * p.kb, n0, GS_W_BYTES);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_launch_dependents();

    // The CTAs of a cluster write into each other's shared memory further down; none may do so before every
    // one of them runs.  Arrive now, wait just before the first such write (by then long complete).
    if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    if (warp == 0 && lane == 0) {
        // ---- producer of W (two producer threads keep more copies in flight than one: 101 against 66 GB/s
        //      per SM measured with 16 KB copies) ----
        int it = pre;
        for (; it < total; ++it) {
            const int s = it % p.stages;
            if (!mbar_wait(s_addr(&empty[s]), ((it / p.stages) - 1) & 1, abort_flag, p.status, p.wait_ns)) break;
            if (*abort_flag) break;
            const uint32_t fb = s_addr(&full[s]);
            mbar_expect_tx(fb, x_off);
            const int n0 = (cluster_id + (it / my_iters) * n_clusters) * GS_BM;
            copy(&map_w, s_addr(tiles + s * stage_bytes), fb, b_begin + (it % my_iters) * p.kb, n0, GS_W_BYTES);
        }
        if (*abort_flag) {
            // let the copies already under way (of both producers) land before the CTA goes away
            for (int j = max(0, it - p.stages); j < it; ++j)
                mbar_wait(s_addr(&full[j % p.stages]), (j / p.stages) & 1, abort_flag + 1, nullptr, p.wait_ns);
        }
    } else if (warp == 6 && lane == 0) {
        // ---- producer of x: written by the kernel before this one ----
        pdl_wait();
        for (int it = 0; it < total; ++it) {
            const int s = it % p.stages;
            if (it >= p.stages && !mbar_wait(s_addr(&empty[s]), ((it / p.stages) - 1) & 1, abort_flag, p.status, p.wait_ns)) break;
            if (*abort_flag) break;
            if (p.skip_last && it == total - 1) break;            // tests: this stage never completes
            const uint32_t fb = s_addr(&full[s]);
            mbar_expect_tx(fb, stage_bytes - x_off);
            copy(&map_x, s_addr(tiles + s * stage_bytes + x_off), fb, b_begin + (it % my_iters) * p.kb, 0, x_bytes);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        // instruction descriptor: D float, A and B bf16, both K-major, N / 8, M / 16
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.nx >> 3) << 17) | ((uint32_t)(GS_BM >> 4) << 24);
        int it = 0;
        bool ok = true;
        for (int t = 0; ok && t < my_tiles; ++t) {
            const int buf = t & 1;
            if (t >= 2 && !mbar_wait(s_addr(&acc_empty[buf]), ((t >> 1) - 1) & 1, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
            tc_fence_after();
            const uint32_t acc = tmem + buf * acc_stride;
            for (int k = 0; k < my_iters; ++k, ++it) {
                const int s = it % p.stages;
                if (!mbar_wait(s_addr(&full[s]), (it / p.stages) & 1, abort_flag, p.status, p.wait_ns)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a = s_addr(tiles + s * stage_bytes);
                for (int j = 0; j < p.kb; ++j) {
                    const uint64_t adesc = smem_desc_sw128(a + j * GS_W_BYTES), bdesc = smem_desc_sw128(a + x_off + j * x_bytes);
#pragma unroll
                    for (int kk = 0; kk < GS_BK / 16; ++kk)    // 32 bytes further along the swizzled row per K = 16
                        tc_mma(acc, adesc + 2 * kk, bdesc + 2 * kk, idesc, (k | j | kk) != 0);
                }
                tc_commit(s_addr(&empty[s]));                  // the stage is free once these MMAs have read it
            }
            if (ok) tc_commit(s_addr(&acc_full[buf]));         // the accumulator is complete
        }
        if (!ok || *abort_flag) { tc_commit(s_addr(&acc_full[0])); tc_commit(s_addr(&acc_full[1])); }
    } else if (warp >= 2 && warp <= 5) {
        // ---- epilogue: warp w may touch lanes 32 (w % 4) .. + 32 of tensor memory ----
        const int quarter = warp & 3;
        const int et = threadIdx.x - 64;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        pdl_wait();
        if (p.mode == 4) {
            for (int m = et; m < p.nx; m += 128) gs_token(p, ra, m, s_pos, s_kv);
        }
        const int rows_here = GS_BM / S;                   // rows of the tile that each CTA of the cluster finishes
        const int n_local = quarter * 32 + lane;           // this thread's row of the tile
        // where this thread's partial sums go: CTA n_local / rows_here, parts[rank][row of x][n_local % rows_here]
        const uint32_t push_base = map_to_rank(s_addr(ftile), S > 1 ? n_local / rows_here : 0) +
                                   (uint32_t)(rank * p.nx * rows_here + n_local % rows_here) * 4u;
        if (S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        for (int t = 0; t < my_tiles; ++t) {
            const int buf = t & 1;
            const int n0 = (cluster_id + t * n_clusters) * GS_BM;
            // all four warps go on or leave together: they meet at named barriers below
            const bool ok = mbar_wait(s_addr(&acc_full[buf]), (t >> 1) & 1, abort_flag, p.status, p.wait_ns) && *abort_flag == 0;
            if (!epi_bar_and(ok)) break;
            tc_fence_after();
            // accumulator (thread = row of W, 16 rows of x per load) -> float partial sums in the shared memory of the
            // CTA that finishes the row
            for (int c0 = 0; c0 < p.nx; c0 += 16) {
                uint32_t v[16];
                tc_ld16(tmem + lane_base + buf * acc_stride + c0, v);
                tc_wait_ld();
                if (S > 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < p.M) st_cluster_f32(push_base + (uint32_t)((c0 + j) * rows_here) * 4u, __uint_as_float(v[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) ftile[(c0 + j) * GS_BM + n_local] = __uint_as_float(v[j]);
                }
            }
            // the accumulator may be overwritten once all epilogue warps have read it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_addr(&acc_empty[buf]));
            if (S > 1) break;                              // one tile per cluster: finished after the cluster barrier below
            epi_bar_sync();
            gs_finish(p, ra, ftile, s_pos, s_kv, n0, 0, 7, et);
            epi_bar_sync();                                // the float tile is free for the next accumulator
        }
    }
    tc_fence_before();
    __syncthreads();
    if (S > 1) {
        if (warp < 2 || warp > 5) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");    // the arrival at the top
        cluster_sync_all();                                // every CTA's partial sums have arrived in their owners' memories
        if (warp >= 2 && warp <= 5 && my_tiles > 0) {
            const int rows_shift = S == 8 ? 4 : (S == 4 ? 5 : 6);      // 128 / S rows per CTA
            gs_finish(p, ra, ftile, s_pos, s_kv, cluster_id * GS_BM, rank << rows_shift, rows_shift, threadIdx.x - 64);
        }
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
}

// How the launcher cuts a product: splits of K (CTAs per cluster), k-blocks per stage, stages of the ring.
struct GsPlan {
    int nx, splits, kb, stages, k_blocks, blocks_per_split, n_tiles, grid, smem;
};

static int gs_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return sms;
}

// Once per process: let the kernel use the whole shared memory (also what the occupancy query below needs).
static int gs_configure() {
    static int state = 0;            // 0: not tried, 1: done, -1: failed
    if (state == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_SMEM_LIMIT);
        state = e == cudaSuccess ? 1 : -1;
        if (e != cudaSuccess) fail(-3, "gemm_stream: cannot get %d bytes of shared memory: %s", GS_SMEM_LIMIT, cudaGetErrorString(e));
    }
    return state == 1 ? 0 : -3;
}

static int gs_smem_for(int nx, int kb, int stages) {
    return stages * kb * (GS_W_BYTES + nx * 128) + nx * GS_BM * 4 + GS_FIXED_SMEM;
}

// Clusters of S CTAs of this kernel, each with `smem` bytes, that the GPU runs at one time (its GPCs hold
// whole clusters only, so this is less than SMs / S).  Cached; 0 if the query fails.
static int gs_max_clusters(int S, int smem) {
    static std::map<std::pair<int, int>, int> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_pair(S, smem);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S * 64);
    cfg.blockDim = dim3(GS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = S; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_stream_tcgen05_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;                    // not cached: asked again next time
    }
    cache[key] = n;
    return n;
}

// k-blocks per stage and stages for a CTA that walks `blocks` k-blocks per tile.
static bool gs_stages(int nx, int blocks, int tiles_per_cta, int* kb_out, int* stages_out) {
    // a short range of K in one stage (two copies in all); else two blocks per stage: 32 KB copies of W
    int kb = blocks <= GS_MAX_KB ? blocks : 2;
    while (kb > 1 && gs_smem_for(nx, kb, 2) > GS_SMEM_LIMIT && blocks > kb) --kb;
    while (kb > 1 && gs_smem_for(nx, kb, 1) > GS_SMEM_LIMIT) --kb;
    const int iters = ((blocks + kb - 1) / kb) * tiles_per_cta;
    int stages = (GS_SMEM_LIMIT - GS_FIXED_SMEM - nx * GS_BM * 4) / (kb * (GS_W_BYTES + nx * 128));
    if (stages > GS_MAX_STAGES) stages = GS_MAX_STAGES;
    if (stages > iters) stages = iters;
    if (stages < 1) return false;
    *kb_out = kb;
    *stages_out = stages;
    return true;
}

static bool gs_try(int M, int N, int K, int S, GsPlan* pl) {
    const int sms = gs_sm_count();
    pl->nx = (M + 15) / 16 * 16;
    pl->k_blocks = (K + GS_BK - 1) / GS_BK;
    pl->n_tiles = (N + GS_BM - 1) / GS_BM;
    pl->splits = S;
    int per = (pl->k_blocks + S - 1) / S;
    const int grid = S > 1 ? pl->n_tiles * S : (pl->n_tiles < sms ? pl->n_tiles : sms);
    const int tiles_per_cta = S > 1 ? 1 : (pl->n_tiles + grid - 1) / grid;
    if (!gs_stages(pl->nx, per, tiles_per_cta, &pl->kb, &pl->stages)) return false;
    per = (per + pl->kb - 1) / pl->kb * pl->kb;                       // whole stages per CTA
    if ((long long)per * (S - 1) >= pl->k_blocks) return false;        // a CTA without a k-block
    pl->blocks_per_split = per;
    pl->grid = grid;
    pl->smem = gs_smem_for(pl->nx, pl->kb, pl->stages);
    return true;
}

// want_splits 0: the launcher chooses.  Returns false for sizes the kernel does not take.
static bool gs_plan(int M, int N, int K, int want_splits, GsPlan* pl) {
    if (M < 1 || M > GS_MAX_NX || N < 1 || K < 8 || K % 8 != 0) return false;
    if (want_splits != 0 && want_splits != 1 && want_splits != 2 && want_splits != 4 && want_splits != 8) return false;
    if (want_splits > 0) {
        for (int S = want_splits; S >= 1; S /= 2)
            if (gs_try(M, N, K, S, pl)) return true;
        return false;
    }
    // The most CTAs that run at one time in one wave, while every CTA keeps two k-blocks or more.
    const int tiles = (N + GS_BM - 1) / GS_BM, blocks = (K + GS_BK - 1) / GS_BK;
    for (int S = 8; S > 1; S /= 2) {
        if (blocks / S < 2 || !gs_try(M, N, K, S, pl)) continue;
        if (tiles <= gs_max_clusters(S, pl->smem)) return true;
    }
    return gs_try(M, N, K, 1, pl);
}

static int g_gs_last_map3d = 0;
int g_gs_pdl = 1;           // 1: the kernel is launched with the programmatic-dependent-launch attribute (fd_gemm_stream_set_pdl)
int g_gs_force_2d = 0;      // tests: two-dimensional copies even where the three-dimensional map applies

static int launch_gs(const void* x, const void* w, GsParams& p, const TcRope& ra, int want_splits, cudaStream_t stream,
                     const char* what) {
    if (gs_configure() != 0) return -3;
    GsPlan pl;
    FD_REQUIRE(gs_plan(p.M, p.N, p.K, want_splits, &pl), -2,
               "%s: sizes not taken (M=%d must be 1..%d, K=%d a multiple of 8, splits %d one of 0, 1, 2, 4, 8)", what, p.M,
               GS_MAX_NX, p.K, want_splits);
    p.nx = pl.nx; p.splits = pl.splits; p.stages = pl.stages; p.kb = pl.kb; p.k_blocks = pl.k_blocks;
    p.blocks_per_split = pl.blocks_per_split; p.n_tiles = pl.n_tiles;
    p.wait_ns = g_tc_wait_ns; p.skip_last = g_tc_skip_last;
    CUtensorMap mw, mx;
    p.map3d = 0;
    if (p.K % 64 == 0 && !g_gs_force_2d && tensor_map_blocks(w, p.N, p.K, &mw, GS_BM, pl.kb) == 0 &&
        tensor_map_blocks(x, p.M, p.K, &mx, pl.nx, pl.kb) == 0)
        p.map3d = 1;
    if (!p.map3d) {
        int rc = tensor_map(w, p.N, p.K, &mw, GS_BM);
        if (rc != 0) return rc;
        rc = tensor_map(x, p.M, p.K, &mx, pl.nx);
        if (rc != 0) return rc;
    }
    g_gs_last_map3d = p.map3d;
    const int pdl_before = g_pdl;
    g_pdl = g_pdl || g_gs_pdl;
    const int rc = launch(what, gemm_stream_tcgen05_kernel, dim3(pl.grid), dim3(GS_THREADS), pl.smem, stream, dim3(pl.splits, 1, 1),
                          mw, mx, p, ra);
    g_pdl = pdl_before;
    return rc;
}

}  // namespace fd

using namespace fd;

// Splits of K (CTAs per cluster) the streaming tcgen05 product would use for these sizes; 0: sizes
// not taken (more than 128 rows of x, K not a multiple of 8, no tensor-map support in the driver).
// 1 (the default): launch the product so that it may start, and fetch its first weights, while the kernel
// before it in the stream still runs (programmatic dependent launch); it waits for that kernel before it
// reads x or writes anything.  Measured on B200 inside the captured decode step of Qwen2.5-1.5B sizes:
// 2.68 against 2.79 ms at batch 64, 1.90 against 2.00 ms at batch 17.
extern "C" int fd_gemm_stream_set_pdl(int on) {
    g_gs_pdl = on ? 1 : 0;
    return 0;
}

// Tests: 1 makes the launcher use two-dimensional copies even where K is a multiple of 64.
extern "C" int fd_gemm_stream_force_2d(int on) {
    g_gs_force_2d = on ? 1 : 0;
    return 0;
}

// 1 if the last launch of the product read its operands through three-dimensional tensor maps.
extern "C" int fd_gemm_stream_last_map3d() { return g_gs_last_map3d; }

extern "C" int fd_gemm_stream_splits(int M, int N, int K) {
    GsPlan pl;
    if (encode_fn() == nullptr || gs_configure() != 0 || !gs_plan(M, N, K, 0, &pl)) return 0;
    return pl.splits;
}

// mode 1: out bf16 [M, N] (+ bias); 2: out float [M, N] (+ bias); 3: W rows in tiles of 8 gate + 8 up
// rows, out bf16 [M, N / 2] = silu(gate) * up (N a multiple of 16).  splits 0: chosen by the launcher.
extern "C" int fd_gemm_stream(const void* x, const void* w, const void* bias, int bias_f32, void* out, int mode,
                              int M, int N, int K, int splits, int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    FD_REQUIRE(mode >= 1 && mode <= 3, -2, "gemm_stream: mode %d", mode);
    FD_REQUIRE(mode != 3 || N % 16 == 0, -2, "gemm_stream: the gated form needs N (= 2 x outputs) to be a multiple of 16, got %d", N);
    FD_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)bias % 16 == 0, -2,
               "gemm_stream: x, W, bias and out must be 16-byte aligned");
    GsParams p = {};
    p.bias = bias; p.out = out; p.status = status; p.M = M; p.N = N; p.K = K; p.mode = mode; p.bias_f32 = bias_f32;
    TcRope ra = {};
    return launch_gs(x, w, p, ra, splits, stream, "gemm_stream");
}

// The q/k/v projection of a decode step with bias, rotary encoding and the append to the paged cache in
// its epilogue (see TcRope for the row order W and bias must have).
extern "C" int fd_gemm_stream_qkv_rope(const void* x, const void* w, const void* bias, int bias_f32, void* q_out,
                                       int M, int K, int splits, const float* cos_t, const float* sin_t, int table_len,
                                       const int* tok_row, const int* tok_pos, const int* row_slot, void* k_pool,
                                       void* v_pool, const int* block_table, int max_blocks, int num_blocks,
                                       int block_size, int n_q, int n_kv, int d, int write_kv, int* status,
                                       cudaStream_t stream) {
    if (M == 0) return 0;
    FD_REQUIRE(d >= 16 && d % 16 == 0, -2, "gemm_stream_qkv_rope: head size %d must be a multiple of 16", d);
    FD_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pool % 16 == 0 &&
               (uintptr_t)v_pool % 16 == 0 && (uintptr_t)cos_t % 16 == 0 && (uintptr_t)sin_t % 16 == 0 && (uintptr_t)bias % 16 == 0,
               -2, "gemm_stream_qkv_rope: all arrays must be 16-byte aligned");
    GsParams p = {};
    p.bias = bias; p.out = q_out; p.status = status; p.M = M; p.N = (n_q + 2 * n_kv) * d; p.K = K; p.mode = 4;
    p.bias_f32 = bias_f32;
    TcRope ra;
    ra.cos_t = cos_t; ra.sin_t = sin_t; ra.tok_row = tok_row; ra.tok_pos = tok_pos; ra.row_slot = row_slot;
    ra.k_pool = (__nv_bfloat16*)k_pool; ra.v_pool = (__nv_bfloat16*)v_pool; ra.block_table = block_table;
    ra.table_len = table_len; ra.max_blocks = max_blocks; ra.num_blocks = num_blocks; ra.block_size = block_size;
    ra.n_q = n_q; ra.n_kv = n_kv; ra.d = d; ra.write_kv = write_kv;
    return launch_gs(x, w, p, ra, splits, stream, "gemm_stream_qkv_rope");
}
