// Causal grouped-query attention over the paged KV cache on the CUDA cores,
// for any head size that is a multiple of 16 (up to 256), any group size up
// to 64, any block size, an optional sliding window, float or bfloat16
// storage.  One kernel serves both kinds of step:
//
//  * prompts: a CTA takes QT consecutive query tokens of one sequence and one
//    KV head, i.e. R = QT * G query rows that share the same keys, and walks
//    the keys in tiles of 32;
//  * decode: QT = 1 and the keys of a sequence are cut into n_splits ranges of
//    split_len tokens (flash-decoding); each CTA leaves an unnormalised
//    (max, sum, accumulator) triple per query row in scratch memory and a
//    second kernel merges them.
//
// Tile and split boundaries are fixed in absolute token index, so the order
// of the floating-point sums of a query does not depend on what else is in
// the batch.  Scores, softmax and the value sum are float; bfloat16 is only a
// storage format here.  This is the attention of the true 32-bit path and the
// fallback for head sizes the tensor-core kernels do not take.
#include <math.h>

#include "attention.cuh"

namespace fd {

constexpr int KT = 32;          // keys per tile (= lanes of a warp)
constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int RMAX = 64;        // query rows per CTA
constexpr int RPW = RMAX / ATT_WARPS;   // rows per warp in the score phase
constexpr int RPT_MAX = 16;     // rows per thread in the value phase


template <typename T> struct Pad;            // padding of a key row in shared memory, in elements
template <> struct Pad<float> { static constexpr int v = 4; };
template <> struct Pad<__nv_bfloat16> { static constexpr int v = 4; };

template <typename T> __device__ __forceinline__ float exp_of(float x);
template <> __device__ __forceinline__ float exp_of<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float exp_of<__nv_bfloat16>(float x) { return __expf(x); }

template <typename T> __device__ __forceinline__ void load_chunk4(const T* p, float f[4]);
template <> __device__ __forceinline__ void load_chunk4<float>(const float* p, float f[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_chunk4<__nv_bfloat16>(const __nv_bfloat16* p, float f[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attn_tile_kernel(const AttnParams p) {
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int tile = blockIdx.x / p.n_splits, split = blockIdx.x - tile * p.n_splits;
    const int slot = p.row_slot[b];
    if (slot < 0) return;
    const int q_len = p.row_q_len[b];
    if (tile * p.QT >= q_len) return;
    const int ctx = p.row_ctx_len[b];
    const int tok0 = p.row_q_start[b] + tile * p.QT;       // first query token of this CTA
    const int nq = min(p.QT, q_len - tile * p.QT);
    const int G = p.G, d = p.d;
    const int R = nq * G;
    const int p_first = ctx + tile * p.QT;                  // position of the first query token
    int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
    int hi = p_first + nq;                                   // keys 0 .. last query position
    if (p.n_splits > 1) {
        lo = max(lo, split * p.split_len);
        hi = min(hi, (split + 1) * p.split_len);
    }

    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int KPAD = Pad<T>::v;
    const int kstride = d + KPAD;
    float* q_s = reinterpret_cast<float*>(smem_raw);               // [RMAX][d]
    float* p_s = q_s + RMAX * d;                                      // [RMAX][KT]
    float* alpha_s = p_s + RMAX * KT;                                 // [RMAX]
    float* l_s = alpha_s + RMAX;                                      // [RMAX]
    T* v_s = reinterpret_cast<T*>(l_s + RMAX);                        // [KT][d]
    T* k_s = v_s + KT * d;                                            // [KT][d + KPAD]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* qg = static_cast<const T*>(p.q);
    const T* kp = static_cast<const T*>(p.k_pool);
    const T* vp = static_cast<const T*>(p.v_pool);

    // queries of this CTA, scaled, as float
    for (int e = tid; e < R * d; e += ATT_THREADS) {
        const int r = e / d, j = e - r * d;
        const int qi = r / G, g = r - qi * G;
        q_s[e] = to_float(qg[((size_t)(tok0 + qi) * p.n_q + kvh * G + g) * d + j]) * p.scale;
    }

    float m_run[RPW], l_run[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

    // value phase mapping: a thread owns 4 consecutive dims of several rows
    const int DC = d >> 2;
    const int RG = ATT_THREADS / DC;
    const int dc = tid % DC, rg = tid / DC;
    const bool pv_active = rg < RG;
    float acc[RPT_MAX][4];
#pragma unroll
    for (int i = 0; i < RPT_MAX; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

    constexpr int EPC = 16 / sizeof(T);          // elements per 16-byte chunk
    const int cpr = d / EPC;                      // chunks per key row
    const int bs = p.block_size;

    for (int t0 = (lo / KT) * KT; t0 < hi; t0 += KT) {
        __syncthreads();   // previous tile consumed (and q_s written, first time round)
        // stage keys and values of this tile; tokens outside [lo, hi) read as zero
        for (int c = tid; c < KT * cpr; c += ATT_THREADS) {
            const int tt = c / cpr, cc = c - tt * cpr;
            const int t = t0 + tt;
            uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
            if (t >= lo && t < hi) {
                const int blk = p.block_table[(size_t)slot * p.max_blocks + t / bs];
                if (blk < 0 || blk >= p.num_blocks) {
                    set_status(p.status, STATUS_BAD_BLOCK);
                } else {
                    const size_t off = (((size_t)blk * p.n_kv + kvh) * bs + (t % bs)) * d + cc * EPC;
                    kv4 = *reinterpret_cast<const uint4*>(kp + off);
                    vv4 = *reinterpret_cast<const uint4*>(vp + off);
                }
            }
            *reinterpret_cast<uint4*>(v_s + tt * d + cc * EPC) = vv4;
            uint2* kd = reinterpret_cast<uint2*>(k_s + tt * kstride + cc * EPC);
            kd[0] = make_uint2(kv4.x, kv4.y);
            kd[1] = make_uint2(kv4.z, kv4.w);
        }
        __syncthreads();

        // scores: warp `warp` owns rows warp, warp + 8, ...; a lane is a key
        float s[RPW];
#pragma unroll
        for (int i = 0; i < RPW; ++i) s[i] = 0.f;
        const T* krow = k_s + lane * kstride;
        for (int c = 0; c < DC; ++c) {
            float kf[4];
            load_chunk4<T>(krow + c * 4, kf);
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const int r = warp + i * ATT_WARPS;
                if (r < R) {
                    const float4 qv = *reinterpret_cast<const float4*>(q_s + r * d + c * 4);
                    s[i] = fmaf(qv.x, kf[0], s[i]);
                    s[i] = fmaf(qv.y, kf[1], s[i]);
                    s[i] = fmaf(qv.z, kf[2], s[i]);
                    s[i] = fmaf(qv.w, kf[3], s[i]);
                }
            }
        }
        // online softmax, one row per warp at a time
        const int t = t0 + lane;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp + i * ATT_WARPS;
            if (r < R) {
                const int qpos = p_first + r / G;
                const bool valid = t >= lo && t < hi && t <= qpos && (p.window <= 0 || qpos - t < p.window);
                const float sv = valid ? s[i] : -INFINITY;
                const float m_new = fmaxf(m_run[i], warp_max(sv));
                float pr = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {
                    pr = valid ? exp_of<T>(sv - m_new) : 0.f;
                    alpha = exp_of<T>(m_run[i] - m_new);
                }
                l_run[i] = l_run[i] * alpha + warp_sum(pr);
                m_run[i] = m_new;
                p_s[r * KT + lane] = pr;
                if (lane == 0) alpha_s[r] = alpha;
            }
        }
        __syncthreads();

        // values: acc[r][dims] = acc * alpha + sum_t p[r][t] * v[t][dims]
        if (pv_active) {
#pragma unroll
            for (int i = 0; i < RPT_MAX; ++i) {
                const int r = rg + i * RG;
                if (r < R) {
                    const float a = alpha_s[r];
                    acc[i][0] *= a; acc[i][1] *= a; acc[i][2] *= a; acc[i][3] *= a;
                }
            }
            for (int tt = 0; tt < KT; ++tt) {
                float vf[4];
                load_chunk4<T>(v_s + tt * d + dc * 4, vf);
#pragma unroll
                for (int i = 0; i < RPT_MAX; ++i) {
                    const int r = rg + i * RG;
                    if (r < R) {
                        const float pr = p_s[r * KT + tt];
                        acc[i][0] = fmaf(pr, vf[0], acc[i][0]);
                        acc[i][1] = fmaf(pr, vf[1], acc[i][1]);
                        acc[i][2] = fmaf(pr, vf[2], acc[i][2]);
                        acc[i][3] = fmaf(pr, vf[3], acc[i][3]);
                    }
                }
            }
        }
    }

    // hand the row sums (and maxima, when splitting) to the value threads
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp + i * ATT_WARPS;
            if (r < R) { l_s[r] = l_run[i]; alpha_s[r] = m_run[i]; }
        }
    }
    __syncthreads();
    if (!pv_active) return;
    T* og = static_cast<T*>(p.out);
#pragma unroll
    for (int i = 0; i < RPT_MAX; ++i) {
        const int r = rg + i * RG;
        if (r >= R) continue;
        const int qi = r / G, g = r - qi * G;
        const size_t row = (size_t)(tok0 + qi) * p.n_q + kvh * G + g;
        if (p.n_splits > 1) {
            const size_t pi = row * p.n_splits + split;
            if (dc == 0) { p.part_m[pi] = alpha_s[r]; p.part_l[pi] = l_s[r]; }
            *reinterpret_cast<float4*>(p.part_acc + pi * d + dc * 4) =
                make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        } else {
            const float l = l_s[r];
            const float inv = l > 0.f ? 1.f / l : 0.f;
            T* o = og + row * d + dc * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = from_float<T>(acc[i][j] * inv);
        }
    }
}

// Merge the per-split triples of every (token, query head): m = max m_s,
// l = sum l_s e^(m_s - m), out = sum acc_s e^(m_s - m) / l.  Splits that saw
// no key (l_s == 0) are skipped; a padding row gives zeros.  The weights
// e^(m_s - m) / l are computed once per (token, head) into shared memory; then
// a thread owns one output dim and sums over the splits with independent loads.
constexpr int COMBINE_MAX_SPLITS = 512;

template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                    const float* __restrict__ part_acc, T* __restrict__ out,
                                    const int* __restrict__ tok_row, const int* __restrict__ row_slot,
                                    int n_q, int d, int n_splits) {
    __shared__ float w_s[COMBINE_MAX_SPLITS];
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int tok = blockIdx.y, h = blockIdx.x;
    const size_t row = (size_t)tok * n_q + h;
    T* o = out + row * d;
    if (row_slot[tok_row[tok]] < 0) {
        for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = from_float<T>(0.f);
        return;
    }
    const float* pm = part_m + row * n_splits;
    const float* pl = part_l + row * n_splits;
    // block-wide max of m over the splits that saw a key
    float m = -INFINITY;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x)
        if (pl[s] > 0.f) m = fmaxf(m, pm[s]);
    m = warp_max(m);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = -INFINITY;
    for (int w = 0; w < nwarps; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    // weights and their sum, in split order within a thread; the block sum order is fixed too
    float lsum = 0.f;
    for (int s = threadIdx.x; s < n_splits; s += blockDim.x) {
        const float ls = pl[s];
        const float w = ls > 0.f ? expf(pm[s] - m) : 0.f;
        w_s[s] = w;
        lsum += ls * w;
    }
    const float l = block_sum(lsum, red);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float* pa = part_acc + row * n_splits * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float a = 0.f;
        int s = 0;
        for (; s + 4 <= n_splits; s += 4) {
            const float a0 = pa[(size_t)(s + 0) * d + j], a1 = pa[(size_t)(s + 1) * d + j];
            const float a2 = pa[(size_t)(s + 2) * d + j], a3 = pa[(size_t)(s + 3) * d + j];
            a = fmaf(a0, w_s[s], a); a = fmaf(a1, w_s[s + 1], a);
            a = fmaf(a2, w_s[s + 2], a); a = fmaf(a3, w_s[s + 3], a);
        }
        for (; s < n_splits; ++s) a = fmaf(pa[(size_t)s * d + j], w_s[s], a);
        o[j] = from_float<T>(a * inv);
    }
}

template <typename T>
static size_t attn_smem_bytes(int d) {
    return (size_t)(RMAX * d + RMAX * KT + 2 * RMAX) * sizeof(float) +
           (size_t)(KT * d + KT * (d + Pad<T>::v)) * sizeof(T);
}

template <typename T>
static int launch_attn(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream) {
    const size_t smem = attn_smem_bytes<T>(p.d);
    auto k = attn_tile_kernel<T>;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-3, "attention: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    const int q_tiles = (max_q_len + p.QT - 1) / p.QT;
    dim3 grid(q_tiles * p.n_splits, p.n_kv, n_rows);
    k<<<grid, ATT_THREADS, smem, stream>>>(p);
    return check_launch("attention");
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// Largest number of query tokens a CTA takes for a group size (0: unsupported).
extern "C" int fd_attn_simt_qt(int G) { return G >= 1 && G <= RMAX ? (RMAX / G > 16 ? 16 : RMAX / G) : 0; }

// Floats of scratch the split form needs: part_acc [T, n_q, n_splits, d], then part_m and part_l [T, n_q, n_splits].
extern "C" long long fd_attn_scratch_floats(int T, int n_q, int d, int n_splits) {
    return (long long)T * n_q * n_splits * (d + 2);
}

// dtype: 0 = float32, 1 = bfloat16 (queries, cache and output alike).
// n_splits == 1 writes `out` directly; otherwise `scratch` must hold
// fd_attn_scratch_floats(T, ...) floats and the merge kernel runs after.
// use_mma != 0: decode steps (max_q_len == 1) in bfloat16 go to the
// tensor-core kernel when it takes the head size and group size.
static int attention_impl(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                          const int* block_table, int max_blocks, int num_blocks, int block_size,
                          const int* tok_row, const int* row_slot, const int* row_q_start,
                          const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                          int max_q_len, int n_q, int n_kv, int d, float scale, int window,
                          int n_splits, int split_len, float* scratch, int* counters, int* status, int use_mma,
                          cudaStream_t stream, const void* prefetch = nullptr, unsigned long long prefetch_bytes = 0) {
    if (n_rows == 0 || T == 0) return 0;
    FD_REQUIRE(n_kv > 0 && n_q % n_kv == 0, -2, "attention: %d query heads are not a multiple of %d KV heads", n_q, n_kv);
    const int G = n_q / n_kv;
    FD_REQUIRE(d % 16 == 0 && d >= 16 && d <= 256, -2, "attention: head size %d must be a multiple of 16 in [16, 256]", d);
    FD_REQUIRE(G <= RMAX, -2, "attention: group size %d exceeds %d", G, RMAX);
    FD_REQUIRE(block_size > 0, -2, "attention: block size %d", block_size);
    FD_REQUIRE(n_splits >= 1 && n_splits <= COMBINE_MAX_SPLITS, -2, "attention: n_splits=%d (1..%d)", n_splits, COMBINE_MAX_SPLITS);
    FD_REQUIRE(n_splits == 1 || (split_len > 0 && split_len % KT == 0), -2,
               "attention: split length %d must be a positive multiple of %d", split_len, KT);
    FD_REQUIRE(n_splits == 1 || scratch != nullptr, -2, "attention: split form needs scratch memory");
    FD_REQUIRE((uintptr_t)scratch % 16 == 0 && (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0 &&
               (uintptr_t)q % 16 == 0, -2,
               "attention: queries, cache pools and scratch memory must be 16-byte aligned");
    FD_REQUIRE(n_splits == 1 || T <= 65535, -2, "attention: the split form takes at most 65535 tokens, got %d", T);
    FD_REQUIRE(n_rows <= 65535 && n_kv <= 65535, -2, "attention: batch of %d rows too large", n_rows);

    AttnParams p;
    p.pf_ptr = (const unsigned char*)prefetch; p.pf_bytes = prefetch ? prefetch_bytes : 0;
    p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.out = out;
    const size_t n_part = (size_t)T * n_q * n_splits;
    // accumulators first: they are stored as float4 and must stay 16-byte aligned
    p.part_acc = scratch;
    p.part_m = scratch ? scratch + n_part * d : nullptr;
    p.part_l = scratch ? scratch + n_part * d + n_part : nullptr;
    p.block_table = block_table; p.row_slot = row_slot; p.row_q_start = row_q_start;
    p.row_q_len = row_q_len; p.row_ctx_len = row_ctx_len; p.status = status;
    p.counters = nullptr;
    p.max_blocks = max_blocks; p.num_blocks = num_blocks; p.block_size = block_size;
    p.n_q = n_q; p.n_kv = n_kv; p.G = G; p.d = d;
    int qt = fd_attn_simt_qt(G);
    if (qt > max_q_len) qt = max_q_len;
    p.QT = qt; p.n_splits = n_splits; p.split_len = split_len; p.window = window; p.scale = scale;

    int rc = 1;
    if (use_mma && dtype == 1 && max_q_len == 1) {
        p.counters = n_splits > 1 ? counters : nullptr;     // given: the kernel merges its own splits
        rc = launch_attn_decode_mma(p, n_rows, stream);
        if (rc == 0 && p.counters != nullptr) return 0;
        p.counters = nullptr;
    }
    else if (use_mma && dtype == 1) {
        rc = use_mma == 2 ? 1 : launch_attn_prefill_tcgen05(p, n_rows, T, max_q_len, stream);
        if (rc == 1) rc = launch_attn_prefill_mma(p, n_rows, max_q_len, stream);
    }
    if (rc == 1)
        rc = dtype == 0 ? launch_attn<float>(p, n_rows, max_q_len, stream)
                        : launch_attn<bf16>(p, n_rows, max_q_len, stream);
    if (rc != 0 || n_splits == 1) return rc;
    dim3 grid(n_q, T);
    if (dtype == 0)
        return launch("attention_combine", attn_combine_kernel<float>, grid, dim3(128), 0, stream, dim3(1, 1, 1),
                      (const float*)p.part_m, (const float*)p.part_l, (const float*)p.part_acc, (float*)out, tok_row,
                      row_slot, n_q, d, n_splits);
    return launch("attention_combine", attn_combine_kernel<bf16>, grid, dim3(128), 0, stream, dim3(1, 1, 1),
                  (const float*)p.part_m, (const float*)p.part_l, (const float*)p.part_acc, (bf16*)out, tok_row,
                  row_slot, n_q, d, n_splits);
}

// The CUDA-core kernel for every case.
extern "C" int fd_attention_simt(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                 const int* block_table, int max_blocks, int num_blocks, int block_size,
                                 const int* tok_row, const int* row_slot, const int* row_q_start,
                                 const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                                 int max_q_len, int n_q, int n_kv, int d, float scale, int window,
                                 int n_splits, int split_len, float* scratch, int* status,
                                 cudaStream_t stream) {
    return attention_impl(q, k_pool, v_pool, out, dtype, block_table, max_blocks, num_blocks, block_size, tok_row,
                          row_slot, row_q_start, row_q_len, row_ctx_len, n_rows, T, max_q_len, n_q, n_kv, d, scale,
                          window, n_splits, split_len, scratch, nullptr, status, 0, stream);
}

// The fastest kernel that takes the sizes: tensor cores where possible.  `counters`
// (optional): n_rows * n_kv ints, all zero, which the decode kernel uses to let the last CTA of
// a (sequence, KV head) merge the splits itself (it leaves them zero again); without them the
// separate merge kernel runs.  prefetch / prefetch_bytes (optional, 16-byte aligned): memory that a
// later kernel streams, which the tensor-core decode kernel asks L2 for when its own reads are
// through (the other kernels ignore it).
extern "C" int fd_attention(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                            const int* block_table, int max_blocks, int num_blocks, int block_size,
                            const int* tok_row, const int* row_slot, const int* row_q_start,
                            const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                            int max_q_len, int n_q, int n_kv, int d, float scale, int window,
                            int n_splits, int split_len, float* scratch, int* counters, int* status,
                            const void* prefetch, unsigned long long prefetch_bytes, cudaStream_t stream) {
    FD_REQUIRE((uintptr_t)prefetch % 16 == 0, -2, "attention: the memory to prefetch must be 16-byte aligned");
    return attention_impl(q, k_pool, v_pool, out, dtype, block_table, max_blocks, num_blocks, block_size, tok_row,
                          row_slot, row_q_start, row_q_len, row_ctx_len, n_rows, T, max_q_len, n_q, n_kv, d, scale,
                          window, n_splits, split_len, scratch, counters, status, 1, stream, prefetch, prefetch_bytes);
}

// The same without the tcgen05 kernel: prompts go to the mma.sync kernel (head sizes other than 128 always
// do; this entry lets tests and measurements reach it at 128 too).
extern "C" int fd_attention_mma_sync(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                                     const int* block_table, int max_blocks, int num_blocks, int block_size,
                                     const int* tok_row, const int* row_slot, const int* row_q_start,
                                     const int* row_q_len, const int* row_ctx_len, int n_rows, int T,
                                     int max_q_len, int n_q, int n_kv, int d, float scale, int window,
                                     int n_splits, int split_len, float* scratch, int* counters, int* status,
                                     cudaStream_t stream) {
    return attention_impl(q, k_pool, v_pool, out, dtype, block_table, max_blocks, num_blocks, block_size, tok_row,
                          row_slot, row_q_start, row_q_len, row_ctx_len, n_rows, T, max_q_len, n_q, n_kv, d, scale,
                          window, n_splits, split_len, scratch, counters, status, 2, stream);
}
