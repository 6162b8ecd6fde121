// Pieces of the decode matrix product of gemv_mma.cu: the mma.sync and streaming-load wrappers, its
// parameters and its epilogues.
#pragma once

#include "common.cuh"

namespace fd {

__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    // weights are read once per step: do not let them displace activations in L1
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

struct GemvParams {
    const __nv_bfloat16* x;      // [M, K]
    const __nv_bfloat16* w;      // [N, K]
    const void* bias;            // [N] or null (bf16 or float, see bias_f32)
    void* out;                   // see mode
    int M, N, K;
    int k_per_split;             // multiple of 32
    int n_splits;
    int mode;                    // 0: partial float [split, M, N]; 1: bf16 [M, N]; 2: float [M, N]; 3: gated bf16 [M, N / 2];
                                 // 4: q/k/v projection with rotary encoding and cache append (see RopeArgs)
    int bias_f32;
    // Memory that a later kernel will stream (for the q/k/v projection the output projection's weights, which are
    // read after the attention; for a block's last product the next block's first weights), or null: each CTA asks
    // L2 for its share once its own loads are through, so that HBM goes on delivering through this kernel's tail and
    // what follows.  It pays for what arrives before it is wanted: a few MB.  Measured in the decode step of
    // Qwen2.5-1.5B: - 1 % at batch 8 and - 1.8 % at batch 1 for the 4.7 MB of the output projection; asking for all
    // 27.5 MB of the down projection from the gate/up kernel made the step 1.2 % slower.
    const unsigned char* pf_ptr;
    unsigned long long pf_bytes;
};

// Mode 4.  W rows are the q heads, then the k heads, then the v heads.  Inside a
// q or k head the rows come in tiles of 16: dims 8t .. 8t+7 and then their
// rotation partners d/2 + 8t .. d/2 + 8t+7, so the thread that holds x_j also
// holds x_{j + d/2}.  v heads are in natural order.  `out` is q_out [M, n_q d].
struct RopeArgs {
    const float* cos_t;          // [table_len, d/2]
    const float* sin_t;
    const int* tok_row;          // [M]
    const int* tok_pos;          // [M]
    const int* row_slot;
    __nv_bfloat16* k_pool;       // [num_blocks, n_kv, block_size, d]
    __nv_bfloat16* v_pool;
    const int* block_table;
    int* status;
    int table_len, max_blocks, num_blocks, block_size;
    int n_q, n_kv, d, write_kv;
};

// Mode 4: what a thread's epilogue needs from the step's index arrays and tables, per x row it holds
// (m = nt * 8 + q * 2 + e at index nt * 2 + e).  Every value hangs on a chain of loads (token -> sequence ->
// slot -> block; position -> cosine and sine): three trips to L2 one after another, which in the epilogue were
// most of its time.  They are fetched in two steps instead: the token's sequence and position before the
// product's first weight loads are issued (nothing waits for them there), the rest right after those loads are
// issued, so that the chain's waits pass while the weights are on their way.
template <int NT>
struct RopePre {
    int slot[NT * 2], pos[NT * 2], blk[NT * 2];      // slot: first the token's row of the step, then its slot
    float c[NT * 2], sn[NT * 2];
};

template <int NT>
__device__ __forceinline__ void rope_prefetch_first(const GemvParams& p, const RopeArgs& ra, int q, RopePre<NT>& pre) {
#pragma unroll
    for (int i = 0; i < NT * 2; ++i) {
        const int m = (i >> 1) * 8 + q * 2 + (i & 1);
        pre.slot[i] = m < p.M ? ra.tok_row[m] : -1;
        pre.pos[i] = m < p.M ? ra.tok_pos[m] : 0;
    }
}

template <int NT>
__device__ __forceinline__ void rope_prefetch_rest(const GemvParams& p, const RopeArgs& ra, int row0, int r, RopePre<NT>& pre) {
    const int d = ra.d, half = d >> 1, tiles_per_head = d >> 4;
    const int tile = row0 >> 4;
    const int head = tile / tiles_per_head, t_in = tile - head * tiles_per_head;
    const bool is_v = head >= ra.n_q + ra.n_kv;
    const int j0 = is_v ? t_in * 16 + r : t_in * 8 + r;
    const bool live = head < ra.n_q + 2 * ra.n_kv;
#pragma unroll
    for (int i = 0; i < NT * 2; ++i) pre.slot[i] = live && pre.slot[i] >= 0 ? ra.row_slot[pre.slot[i]] : -1;
#pragma unroll
    for (int i = 0; i < NT * 2; ++i) {
        pre.blk[i] = -1; pre.c[i] = 1.f; pre.sn[i] = 0.f;
        const int slot = pre.slot[i], pos = pre.pos[i];
        if (slot < 0 || pos < 0 || pos >= ra.table_len) continue;
        if (!is_v) {
            pre.c[i] = ra.cos_t[(size_t)pos * half + j0];
            pre.sn[i] = ra.sin_t[(size_t)pos * half + j0];
        }
        if (head >= ra.n_q && ra.write_kv) pre.blk[i] = ra.block_table[(size_t)slot * ra.max_blocks + pos / ra.block_size];
    }
}

// What the owner of a finished row tile does with it.  acc[nt][0..1]: W row row0, x rows
// nt*8 + q*2 + {0,1}; acc[nt][2..3]: W row row0 + 8 (r = lane / 4, q = lane % 4, row0 the
// tile's first row + r).
template <int NT, bool ROPE>
__device__ __forceinline__ void gemv_epilogue(const GemvParams& p, const RopeArgs& ra, float (&acc)[NT][4], int row0,
                                              int split, int r, int q, const RopePre<NT>& pre) {
    if (ROPE) {                                               // mode 4
        const int d = ra.d, half = d >> 1, tiles_per_head = d >> 4;
        const int tile = row0 >> 4;
        const int head = tile / tiles_per_head, t_in = tile - head * tiles_per_head;
        if (head >= ra.n_q + 2 * ra.n_kv) return;
        float b0 = 0.f, b1 = 0.f;
        if (p.bias != nullptr) {
            b0 = p.bias_f32 ? static_cast<const float*>(p.bias)[row0] : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[row0]);
            b1 = p.bias_f32 ? static_cast<const float*>(p.bias)[row0 + 8] : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[row0 + 8]);
        }
        const bool is_v = head >= ra.n_q + ra.n_kv;
        // dims of this thread's two values inside the head
        const int j0 = is_v ? t_in * 16 + r : t_in * 8 + r;
        const int j1 = is_v ? j0 + 8 : j0 + half;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int m = nt * 8 + q * 2 + e, i = nt * 2 + e;
                if (m >= p.M) continue;
                if (pre.slot[i] < 0) continue;                // padding row
                float v0 = acc[nt][e] + b0, v1 = acc[nt][2 + e] + b1;
                const int pos = pre.pos[i];
                const bool pos_ok = pos >= 0 && pos < ra.table_len;
                if (!pos_ok) set_status(ra.status, STATUS_BAD_POSITION);     // rotated by position 0's angle (0)
                if (!is_v) {
                    const float c = pre.c[i], sn = pre.sn[i];
                    const float y0 = v0 * c - v1 * sn, y1 = v1 * c + v0 * sn;
                    v0 = y0; v1 = y1;
                }
                if (head < ra.n_q) {
                    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + ((size_t)m * ra.n_q + head) * d;
                    o[j0] = __float2bfloat16_rn(v0);
                    o[j1] = __float2bfloat16_rn(v1);
                } else if (ra.write_kv && pos_ok) {
                    const int blk = pre.blk[i];
                    if (blk < 0 || blk >= ra.num_blocks) { set_status(ra.status, STATUS_BAD_BLOCK); continue; }
                    const int kvh = is_v ? head - ra.n_q - ra.n_kv : head - ra.n_q;
                    __nv_bfloat16* pool = is_v ? ra.v_pool : ra.k_pool;
                    __nv_bfloat16* o = pool + (((size_t)blk * ra.n_kv + kvh) * ra.block_size + pos % ra.block_size) * d;
                    o[j0] = __float2bfloat16_rn(v0);
                    o[j1] = __float2bfloat16_rn(v1);
                }
            }
        return;
    }
    if (p.mode == 3) {
        // tiles of 16 rows hold 8 gate rows then 8 up rows of the same 8 outputs
        const int tile = row0 >> 4;
        const int o = tile * 8 + r;                   // output feature
        const int NO = p.N >> 1;
        if (o < NO) {
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int m = nt * 8 + q * 2 + e;
                    if (m < p.M) {
                        const float g = acc[nt][e], u = acc[nt][2 + e];
                        out[(size_t)m * NO + o] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
                    }
                }
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int n = row0 + h * 8;
        if (n >= p.N) continue;
        float bias = 0.f;
        if (p.bias != nullptr && p.mode != 0)
            bias = p.bias_f32 ? static_cast<const float*>(p.bias)[n]
                              : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int m = nt * 8 + q * 2 + e;
                if (m >= p.M) continue;
                const float v = acc[nt][h * 2 + e] + bias;
                if (p.mode == 0)
                    static_cast<float*>(p.out)[((size_t)split * p.M + m) * p.N + n] = v;
                else if (p.mode == 1)
                    static_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
                else
                    static_cast<float*>(p.out)[(size_t)m * p.N + n] = v;
            }
    }
}

}  // namespace fd
