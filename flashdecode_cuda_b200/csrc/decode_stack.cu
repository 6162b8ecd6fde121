// A whole stack of decoder layers for one decode step (at most 16 rows, bfloat16) in ONE
// persistent kernel.
//
// A decode step of a small batch is a chain of short phases (projection, attention, projection,
// norm, feed-forward ...), each of which alone cannot fill the GPU for longer than it takes to
// start: as separate kernels the step is bound by launch gaps and by the ramp of each kernel's
// first loads, not by bytes.  Here one CTA per SM stays resident for all layers:
//
//   per layer   1. q/k/v projection + bias + rotary encoding + cache append        | grid barrier
//               2. split-KV attention (two groups of 4 warps per CTA, each a         |
//                  (sequence, KV head, split); the last group to finish a           |
//                  (sequence, KV head) merges its splits)                            | grid barrier
//               3. output projection -> float partial sums                          | grid barrier, whose last
//                  arriver adds them to the residual stream and applies the second norm
//               4. gate/up projection with the SiLU epilogue                        | grid barrier
//               5. down projection -> float partial sums                            | grid barrier, whose last
//                  arriver adds them and applies the next layer's first norm (after the last layer
//                  the partial sums are left for the caller's next norm)
//
// While a phase runs, the CTAs ask the L2 cache for the weights of the next phases
// (cp.async.bulk.prefetch.L2), so HBM keeps streaming through the barriers and a phase's first
// loads hit L2.  Weights are read with the non-coherent path; everything the kernel itself
// writes (activations, partial sums, the residual stream) is read with L2-only loads after
// the barrier's acquire, never through the non-coherent path.
//
// The matrix products are those of gemv_mma.cu (16 rows of W x 8 rows of x per mma.m16n8k16,
// weights straight from global memory into fragments), the attention that of
// attention_decode_mma.cu; only the work distribution differs: items are dealt to the resident
// CTAs instead of to a grid.
//
// The grid barrier is an arrival counter and a release word in global memory.  Every wait is
// bounded (half a second): a CTA that gives up sets a status bit and an abort word that the
// others see, and all leave.  The kernel is launched cooperatively, so all CTAs are resident.
#include <string.h>

#include "attention_decode_body.cuh"
#include "gemv_common.cuh"

namespace fd {

constexpr int DS_WARPS = 16;
constexpr int DS_THREADS = DS_WARPS * 32;
constexpr int DS_GROUPS = 2;                       // attention groups (of DM_WARPS warps) per CTA
constexpr unsigned long long DS_WAIT_NS = 500ull * 1000 * 1000;

struct StackLayer {
    const __nv_bfloat16* w_qkv;       // [(n_q + 2 n_kv) d, H], q and k heads in the paired row order
    const void* b_qkv;                // same order, or null
    const __nv_bfloat16* w_o;         // [H, n_q d]
    const __nv_bfloat16* w_gate_up;   // [2 I, H] in tiles of 8 gate + 8 up rows
    const __nv_bfloat16* w_down;      // [H, I]
    const void* norm2_w;              // [H]
    const void* next_norm_w;          // [H]: the first norm of the next layer; null after the last
    __nv_bfloat16* k_pool;
    __nv_bfloat16* v_pool;
    const int* block_table;
    float eps2, eps_next;
    int window, write_kv, max_blocks, num_blocks, block_size, pad_;
};

struct StackParams {
    const StackLayer* layers;
    const int* tok_row;
    const int* tok_pos;
    const int* row_slot;
    const int* row_q_start;
    const int* row_q_len;
    const int* row_ctx_len;
    const float* cos_t;
    const float* sin_t;
    float* resid;                     // [M, H] residual stream; its pending delta has been added already
    __nv_bfloat16* xn;                // [M, H] in: first norm of the first layer applied to resid
    __nv_bfloat16* q;                 // [M, n_q d]
    __nv_bfloat16* attn;              // [M, n_q d]
    float* o_parts;                   // [o_splits, M, H]
    __nv_bfloat16* act;               // [M, I]
    float* down_parts;                // [down_splits, M, H]: after the last layer, the caller's pending delta
    float* attn_scratch;              // the splits' partial results
    int* attn_counters;               // [M, n_kv], zero between launches
    unsigned* barrier;                // [4]: arrivals, release, abort, unused; zero between launches
    int* status;
    int n_layers, M, H, I, n_q, n_kv, d, table_len;
    int n_splits, split_len;
    int qkv_wk, o_wk, o_splits, gu_wk, down_wk, down_splits;
    int bias_f32, norm_w_f32;
    float scale;
    int skip;                         // timing studies: phases to leave out (bit 0 q/k/v, 1 attention, 2 o, 3 gate/up, 4 down, 5 prefetches, 6 norms)
};

struct GemvJob {
    const __nv_bfloat16* x;
    const __nv_bfloat16* w;
    const void* bias;
    void* out;
    int M, N, K, wk, splits, mode, bias_f32;
};

__device__ __forceinline__ unsigned long long ds_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Ask L2 for the part of [base, base + bytes) that falls to this CTA; `lane_id` of `n_lanes`
// threads of the CTA share the requests (4 KB each).
__device__ __forceinline__ void ds_prefetch(const void* base, size_t bytes, int cta, int ncta, int lane_id, int n_lanes) {
    constexpr size_t PIECE = 4096;
    const size_t pieces = (bytes + PIECE - 1) / PIECE;
    const size_t per = (pieces + ncta - 1) / ncta;
    const size_t p0 = (size_t)cta * per;
    const size_t p1 = p0 + per < pieces ? p0 + per : pieces;
    const char* b = static_cast<const char*>(base);
    for (size_t i = p0 + lane_id; i < p1; i += n_lanes) {
        const size_t off = i * PIECE;
        const unsigned n = (unsigned)((bytes - off < PIECE ? bytes - off : PIECE) & ~(size_t)15);
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(b + off), "r"(n) : "memory");
    }
}

// Barrier of all CTAs.  The CTA that arrives last runs `serial` (all its threads) before it
// releases the others.  Returns false when the wait ran out or another CTA gave up: the caller
// leaves the kernel.  `flag`: one int of shared memory.
template <typename F>
__device__ __forceinline__ bool ds_grid_sync(unsigned* bar, unsigned& epoch, int* status, int* flag, F&& serial) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();                                    // this CTA's writes, before its arrival
        const unsigned old = atomicAdd(&bar[0], 1u);
        *flag = old + 1 == (epoch + 1) * gridDim.x ? 1 : 0;
    }
    __syncthreads();
    if (*flag == 1) {
        __threadfence();                                    // the others' writes, after their arrivals
        serial();
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + 1), "r"(epoch + 1) : "memory");
        }
    } else {
        if (threadIdx.x == 0) {
            unsigned long long t0 = 0;
            int ok = 1;
            for (unsigned spins = 1;; ++spins) {
                unsigned v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar + 1) : "memory");
                if ((int)(v - (epoch + 1)) >= 0) break;
                if ((spins & 255) != 0) continue;
                unsigned ab;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(ab) : "l"(bar + 2) : "memory");
                if (ab != 0) { ok = 0; break; }
                if (t0 == 0) t0 = ds_ns();
                else if (ds_ns() - t0 > DS_WAIT_NS) {
                    set_status(status, STATUS_WAIT_TIMEOUT);
                    atomicExch(bar + 2, 1u);
                    ok = 0;
                    break;
                }
            }
            if (!ok) *flag = 2;
        }
        __syncthreads();
    }
    const bool ok = *flag != 2;
    __syncthreads();                                        // the flag is free again
    ++epoch;
    return ok;
}

// One matrix product of the step, its items dealt to the resident CTAs.  An item is WR = 16 / wk
// row tiles of 16 W rows (one per group of wk warps, which slice K between them and add their
// sums in shared memory in a fixed order) times one of `splits` ranges of K.
template <int NT, int UNROLL>
__device__ __forceinline__ void ds_gemv(const GemvJob& jb, const RopeArgs& ra, float* red, int cta, int ncta) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int WK = jb.wk, WR = DS_WARPS / WK;
    const int wr = warp / WK, wk = warp - wr * WK;
    const int r = lane >> 2, q = lane & 3;
    const int tiles = (jb.N + 15) >> 4;
    const int row_groups = (tiles + WR - 1) / WR;
    const int n_items = row_groups * jb.splits;
    const int chunks = jb.K >> 5;                               // chunks of 32 k
    const int per = (chunks + jb.splits - 1) / jb.splits;
    GemvParams gp;
    gp.x = jb.x; gp.w = jb.w; gp.bias = jb.bias; gp.out = jb.out; gp.M = jb.M; gp.N = jb.N; gp.K = jb.K;
    gp.k_per_split = per * 32; gp.n_splits = jb.splits; gp.mode = jb.mode; gp.bias_f32 = jb.bias_f32;

    for (int item = cta; item < n_items; item += ncta) {
        const int split = item / row_groups, rg = item - split * row_groups;
        const int c0 = split * per;
        const int n_chunks = max(0, min(chunks, c0 + per) - c0);
        const int tile = rg * WR + wr;
        const int row0 = tile * 16 + r;
        const __nv_bfloat16* w0 = jb.w + (size_t)min(row0, jb.N - 1) * jb.K + c0 * 32 + q * 8;
        const __nv_bfloat16* w1 = jb.w + (size_t)min(row0 + 8, jb.N - 1) * jb.K + c0 * 32 + q * 8;
        const __nv_bfloat16* xb[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xb[nt] = jb.x + (size_t)min(nt * 8 + r, jb.M - 1) * jb.K + c0 * 32 + q * 8;
        float acc[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

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
                    xv[u][nt] = __ldcg(reinterpret_cast<const uint4*>(xb[nt] + (kc + u * WK) * 32));
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma16816(acc[nt], a[u].x, b[u].x, a[u].y, b[u].y, xv[u][nt].x, xv[u][nt].y);
                    mma16816(acc[nt], a[u].z, b[u].z, a[u].w, b[u].w, xv[u][nt].z, xv[u][nt].w);
                }
            }
        }
        for (; kc < n_chunks; kc += WK) {
            const uint4 a = ldg_stream(w0 + kc * 32);
            const uint4 b = ldg_stream(w1 + kc * 32);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xv = __ldcg(reinterpret_cast<const uint4*>(xb[nt] + kc * 32));
                mma16816(acc[nt], a.x, b.x, a.y, b.y, xv.x, xv.y);
                mma16816(acc[nt], a.z, b.z, a.w, b.w, xv.z, xv.w);
            }
        }
        if (WK > 1) {
            float* mine = red + (warp * 32 + lane) * NT * 4;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) mine[nt * 4 + e] = acc[nt][e];
            __syncthreads();
            if (wk == 0) {
                for (int k = 1; k < WK; ++k) {
                    const float* other = red + ((warp + k) * 32 + lane) * NT * 4;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) acc[nt][e] += other[nt * 4 + e];
                }
            }
        }
        if (wk == 0 && tile < tiles) {
            RopePre<NT> pre;
            if (gp.mode == 4) {
                rope_prefetch_first<NT>(gp, ra, q, pre);
                rope_prefetch_rest<NT>(gp, ra, row0, r, pre);
                gemv_epilogue<NT, true>(gp, ra, acc, row0, split, r, q, pre);
            } else {
                gemv_epilogue<NT, false>(gp, ra, acc, row0, split, r, q, pre);
            }
        }
        if (WK > 1) __syncthreads();                            // the sums have been read: the next item may write
    }
}

// By one CTA: resid[m] += sum of the partial sums (in order); out[m] = norm(resid[m]) * w.  Warp = row.
__device__ __forceinline__ void ds_add_norm(const StackParams& p, const float* parts, int n_parts, const void* w,
                                            float eps, __nv_bfloat16* out) {
    const int lane = threadIdx.x & 31, m = threadIdx.x >> 5;
    if (m >= p.M) return;
    const int H = p.H;
    const size_t part_stride = (size_t)p.M * H;
    float* rrow = p.resid + (size_t)m * H;
    float ss = 0.f;
#pragma unroll 4
    for (int i = lane * 4; i < H; i += 128) {
        float4 x = __ldcg(reinterpret_cast<const float4*>(rrow + i));
        for (int s = 0; s < n_parts; ++s) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(parts + s * part_stride + (size_t)m * H + i));
            x.x += v.x; x.y += v.y; x.z += v.z; x.w += v.w;
        }
        *reinterpret_cast<float4*>(rrow + i) = x;
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
#pragma unroll 4
    for (int i = lane * 4; i < H; i += 128) {
        const float4 x = *reinterpret_cast<const float4*>(rrow + i);      // this thread's own stores
        float w0, w1, w2, w3;
        if (p.norm_w_f32) {
            const float4 wv = *reinterpret_cast<const float4*>(static_cast<const float*>(w) + i);
            w0 = wv.x; w1 = wv.y; w2 = wv.z; w3 = wv.w;
        } else {
            const uint2 wv = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(w) + i);
            const __nv_bfloat162* w2p = reinterpret_cast<const __nv_bfloat162*>(&wv);
            w0 = __low2float(w2p[0]); w1 = __high2float(w2p[0]); w2 = __low2float(w2p[1]); w3 = __high2float(w2p[1]);
        }
        uint2 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
        o2[0] = __floats2bfloat162_rn(x.x * rstd * w0, x.y * rstd * w1);
        o2[1] = __floats2bfloat162_rn(x.z * rstd * w2, x.w * rstd * w3);
        *reinterpret_cast<uint2*>(out + (size_t)m * H + i) = o;
    }
}

template <int NT, int D>
__global__ void __launch_bounds__(DS_THREADS, 1)
decode_stack_kernel(const StackParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int UNROLL = NT == 1 ? 8 : 4;
    float* red = reinterpret_cast<float*>(smem);
    __shared__ int flag;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int tid = threadIdx.x, warp = tid >> 5;
    unsigned epoch = 0;
    const int qkv_rows = (p.n_q + 2 * p.n_kv) * p.d;
    const int qd = p.n_q * p.d;

    RopeArgs ra;
    ra.cos_t = p.cos_t; ra.sin_t = p.sin_t; ra.tok_row = p.tok_row; ra.tok_pos = p.tok_pos; ra.row_slot = p.row_slot;
    ra.status = p.status; ra.table_len = p.table_len; ra.n_q = p.n_q; ra.n_kv = p.n_kv; ra.d = p.d;

    AttnParams ap;
    ap.q = p.q; ap.out = p.attn;
    {
        const size_t n_part = (size_t)p.M * p.n_q * p.n_splits;
        ap.part_acc = p.attn_scratch;
        ap.part_m = p.attn_scratch ? p.attn_scratch + n_part * D : nullptr;
        ap.part_l = p.attn_scratch ? p.attn_scratch + n_part * D + n_part : nullptr;
    }
    ap.row_slot = p.row_slot; ap.row_q_start = p.row_q_start; ap.row_q_len = p.row_q_len; ap.row_ctx_len = p.row_ctx_len;
    ap.status = p.status; ap.counters = p.attn_counters;
    ap.n_q = p.n_q; ap.n_kv = p.n_kv; ap.G = p.n_q / p.n_kv; ap.d = D; ap.QT = 1;
    ap.n_splits = p.n_splits; ap.split_len = p.split_len; ap.scale = p.scale;
    const int attn_items = p.M * p.n_kv * p.n_splits;
    auto nothing = [] {};

    for (int l = 0; l < p.n_layers; ++l) {
        const StackLayer L = p.layers[l];
        ra.k_pool = L.k_pool; ra.v_pool = L.v_pool; ra.block_table = L.block_table; ra.max_blocks = L.max_blocks;
        ra.num_blocks = L.num_blocks; ra.block_size = L.block_size; ra.write_kv = L.write_kv;

        // 1. q/k/v projection, rotary encoding, cache append
        if (!(p.skip & 32)) ds_prefetch(L.w_o, (size_t)p.H * qd * 2, cta, ncta, tid, DS_THREADS);
        if (!(p.skip & 1)) {
            GemvJob jb = {p.xn, L.w_qkv, L.b_qkv, p.q, p.M, qkv_rows, p.H, p.qkv_wk, 1, 4, p.bias_f32};
            ds_gemv<NT, UNROLL>(jb, ra, red, cta, ncta);
        }
        if (!ds_grid_sync(p.barrier, epoch, p.status, &flag, nothing)) return;

        // 2. attention; the warps without a group fetch the feed-forward's first matrix meanwhile
        if (p.skip & 2) {
        } else if (warp < DS_GROUPS * DM_WARPS) {
            const int g = warp / DM_WARPS;
            ap.k_pool = L.k_pool; ap.v_pool = L.v_pool; ap.block_table = L.block_table;
            ap.max_blocks = L.max_blocks; ap.num_blocks = L.num_blocks; ap.block_size = L.block_size;
            ap.window = L.window;
            constexpr size_t GROUP_BYTES = (dm_smem_bytes<D>() + 127) / 128 * 128;
            unsigned char* gs = smem + g * GROUP_BYTES;
            const GroupSync gsync = {g + 1};
            for (int item = cta * DS_GROUPS + g; item < attn_items; item += ncta * DS_GROUPS) {
                const int split = item % p.n_splits;
                const int pair = item / p.n_splits;
                attn_decode_item<D, false>(ap, split, pair % p.n_kv, pair / p.n_kv, gs, tid - g * DM_THREADS, gsync);
                gsync();                                        // the group's shared memory is free again
            }
        } else if (!(p.skip & 32)) {
            ds_prefetch(L.w_gate_up, (size_t)2 * p.I * p.H * 2, cta, ncta, tid - DS_GROUPS * DM_THREADS,
                        DS_THREADS - DS_GROUPS * DM_THREADS);
        }
        if (!ds_grid_sync(p.barrier, epoch, p.status, &flag, nothing)) return;

        // 3. output projection; then resid += it, second norm
        if (!(p.skip & 4)) {
            GemvJob jb = {p.attn, L.w_o, nullptr, p.o_parts, p.M, p.H, qd, p.o_wk, p.o_splits, 0, 0};
            ds_gemv<NT, UNROLL>(jb, ra, red, cta, ncta);
        }
        if (!ds_grid_sync(p.barrier, epoch, p.status, &flag,
                          [&] { if (!(p.skip & 64)) ds_add_norm(p, p.o_parts, p.o_splits, L.norm2_w, L.eps2, p.xn); })) return;

        // 4. gate/up projection with SiLU; the down matrix and the next layer's q/k/v matrix are on their way
        if (!(p.skip & 32)) ds_prefetch(L.w_down, (size_t)p.H * p.I * 2, cta, ncta, tid, DS_THREADS);
        if (l + 1 < p.n_layers && !(p.skip & 32))
            ds_prefetch(p.layers[l + 1].w_qkv, (size_t)qkv_rows * p.H * 2, cta, ncta, tid, DS_THREADS);
        if (!(p.skip & 8)) {
            GemvJob jb = {p.xn, L.w_gate_up, nullptr, p.act, p.M, 2 * p.I, p.H, p.gu_wk, 1, 3, 0};
            ds_gemv<NT, UNROLL>(jb, ra, red, cta, ncta);
        }
        if (!ds_grid_sync(p.barrier, epoch, p.status, &flag, nothing)) return;

        // 5. down projection; then (between layers) resid += it, the next layer's first norm
        if (!(p.skip & 16)) {
            GemvJob jb = {p.act, L.w_down, nullptr, p.down_parts, p.M, p.H, p.I, p.down_wk, p.down_splits, 0, 0};
            ds_gemv<NT, UNROLL>(jb, ra, red, cta, ncta);
        }
        if (l + 1 < p.n_layers) {
            if (!ds_grid_sync(p.barrier, epoch, p.status, &flag,
                              [&] { if (!(p.skip & 64)) ds_add_norm(p, p.down_parts, p.down_splits, L.next_norm_w, L.eps_next, p.xn); }))
                return;
        }
    }
    // the last arrival leaves the barrier ready for the next launch; nobody waits
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(&p.barrier[0], 1u);
        if (old + 1 == (epoch + 1) * gridDim.x) {
            p.barrier[1] = 0;
            __threadfence();
            p.barrier[0] = 0;
        }
    }
}

template <int NT, int D>
static int launch_stack(const StackParams& p, int grid, cudaStream_t stream) {
    constexpr size_t group = (dm_smem_bytes<D>() + 127) / 128 * 128;
    constexpr size_t red = (size_t)DS_WARPS * 32 * NT * 4 * sizeof(float);
    constexpr size_t smem = DS_GROUPS * group > red ? DS_GROUPS * group : red;
    auto k = decode_stack_kernel<NT, D>;
    static bool configured = false;
    static int resident = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-3, "decode_stack: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, k, DS_THREADS, smem);
        if (e != cudaSuccess) return fail(-3, "decode_stack: occupancy query failed: %s", cudaGetErrorString(e));
        configured = true;
    }
    FD_REQUIRE(resident >= 1, -3, "decode_stack: no CTA of %d threads and %zu bytes of shared memory fits an SM", DS_THREADS, smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(DS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;       // all CTAs resident together, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, k, p);
    if (e != cudaSuccess) return fail(-100, "decode_stack: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace fd

using namespace fd;

extern "C" int fd_decode_stack_layer_bytes() { return (int)sizeof(StackLayer); }
extern "C" int fd_decode_stack_params_bytes() { return (int)sizeof(StackParams); }

// How a product [M <= 16, K] x [N, K]^T is dealt to `ctas` resident CTAs of 16 warps: wk warps
// share a row tile and slice K, `splits` ranges of K go to different CTAs (only where the
// consumer adds partial sums: max_splits > 1).  Returns wk | splits << 8.
extern "C" int fd_decode_stack_plan(int N, int K, int ctas, int max_splits) {
    const int tiles = (N + 15) / 16, chunks = K / 32;
    int best_wk = DS_WARPS, best_s = 1;
    double best = 1e30;
    for (int wk = 1; wk <= DS_WARPS; wk *= 2) {
        const int wr = DS_WARPS / wk;
        for (int s = 1; s <= max_splits; ++s) {
            const int per = (chunks + s - 1) / s;
            if ((long long)per * (s - 1) >= chunks) continue;         // an empty split
            const long long items = (long long)((tiles + wr - 1) / wr) * s;
            const long long rounds = (items + ctas - 1) / ctas;
            // a round costs the chunks a warp walks plus a fixed part (first loads, the sum in shared memory)
            const double cost = rounds * ((double)(per + wk - 1) / wk + 4.0) + 0.5 * (s - 1);
            if (cost < best) { best = cost; best_wk = wk; best_s = s; }
        }
    }
    return best_wk | (best_s << 8);
}

// Runs the stack.  `params`: a StackParams image of fd_decode_stack_params_bytes() bytes on the
// host (the caller packs it field by field); its `layers` points to n_layers StackLayer images
// on the device.  `ctas`: CTAs to launch (the SM count).
extern "C" int fd_decode_stack(const void* params, int n_bytes, int ctas, cudaStream_t stream) {
    FD_REQUIRE(n_bytes == (int)sizeof(StackParams), -2, "decode_stack: parameter block of %d bytes, expected %zu", n_bytes,
               sizeof(StackParams));
    StackParams p;
    memcpy(&p, params, sizeof(p));
    FD_REQUIRE(p.n_layers >= 1 && p.M >= 1 && p.M <= 16, -2, "decode_stack: %d layers, %d rows (1..16)", p.n_layers, p.M);
    FD_REQUIRE(p.d == 64 || p.d == 128, -2, "decode_stack: head size %d (64 or 128)", p.d);
    FD_REQUIRE(p.n_kv > 0 && p.n_q % p.n_kv == 0 && p.n_q / p.n_kv <= 16, -2, "decode_stack: %d query heads for %d KV heads", p.n_q, p.n_kv);
    FD_REQUIRE(p.H % 32 == 0 && p.I % 32 == 0 && (p.n_q * p.d) % 32 == 0, -2, "decode_stack: widths must be multiples of 32");
    FD_REQUIRE(p.I % 8 == 0, -2, "decode_stack: the gated layout needs a multiple of 8 outputs");
    FD_REQUIRE(p.n_splits >= 1 && (p.n_splits == 1 || (p.split_len > 0 && p.split_len % DM_TILE == 0)), -2,
               "decode_stack: attention splits %d x %d", p.n_splits, p.split_len);
    FD_REQUIRE((size_t)(p.n_q / p.n_kv) * p.n_splits * sizeof(float) <= 16 * 1024, -2, "decode_stack: too many attention splits");
    FD_REQUIRE(p.n_splits == 1 || (p.attn_scratch != nullptr && p.attn_counters != nullptr), -2, "decode_stack: split attention needs scratch memory");
    for (int wk : {p.qkv_wk, p.o_wk, p.gu_wk, p.down_wk})
        FD_REQUIRE(wk >= 1 && wk <= DS_WARPS && (wk & (wk - 1)) == 0, -2, "decode_stack: %d warps per row tile", wk);
    FD_REQUIRE(p.o_splits >= 1 && p.down_splits >= 1, -2, "decode_stack: splits");
    FD_REQUIRE(ctas >= 1, -2, "decode_stack: %d CTAs", ctas);
    const bool one = p.M <= 8;
    if (p.d == 128) return one ? launch_stack<1, 128>(p, ctas, stream) : launch_stack<2, 128>(p, ctas, stream);
    return one ? launch_stack<1, 64>(p, ctas, stream) : launch_stack<2, 64>(p, ctas, stream);
}
