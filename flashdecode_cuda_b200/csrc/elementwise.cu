// Row-wise kernels: embedding gather, fused residual-add + RMSNorm, SiLU*up,
// and rotary position encoding fused with the append to the paged KV cache.
//
// All of them are bound by memory traffic or launch latency; each does its
// arithmetic in float and rounds once on store.
#include "common.cuh"

namespace fd {

// ---------------------------------------------------------------------------
// embedding: resid[t, :] = float(table[token[t], :])
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ resid, int H, int V, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t];
    float* dst = resid + (size_t)t * H;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) set_status(status, STATUS_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const TW* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_float(src[i]);
}

// ---------------------------------------------------------------------------
// residual add + RMSNorm.  For output row j (source row r = rows ? rows[j] : j):
//   x = resid[r] + sum_p delta[p][r]        (float; parts added in index order)
//   resid[r] = x                             (if write_resid)
//   out[j] = x * rsqrt(mean(x^2) + eps) * w  (float, rounded once)
// `delta` may be null (plain norm).  Several parts are the partial sums a
// split-K matrix product leaves behind.
// ---------------------------------------------------------------------------
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(const TD* __restrict__ delta, int n_parts, size_t part_stride,
                                   float* __restrict__ resid, int write_resid,
                                   const TW* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* xs = smem;                 // H floats
    float* red = smem + ((H + 3) & ~3);  // 33 floats
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    float* rrow = resid + (size_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = rrow[i];
        if (delta != nullptr) {
            for (int p = 0; p < n_parts; ++p) x += to_float(delta[p * part_stride + (size_t)r * H + i]);
            if (write_resid) rrow[i] = x;
        }
        xs[i] = x;
        ss += x * x;
    }
    const float total = block_sum(ss, red);
    const float rstd = rsqrtf(total / (float)H + eps);
    TO* orow = out + (size_t)j * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        orow[i] = from_float<TO>(xs[i] * rstd * to_float(w[i]));
}

// The same for rows that one CTA can hold in registers (H a multiple of 8, at most 8 * 1024):
// bfloat16 delta and output, one 16-byte load per tensor per thread, every load (the norm
// weight included) issued before the reduction.  This is the form decode steps use, where
// the kernel's time is its chain of dependent memory accesses.
template <typename TW>
__global__ void add_rmsnorm_row_kernel(const __nv_bfloat16* __restrict__ delta, float* __restrict__ resid,
                                       int write_resid, const TW* __restrict__ w, float eps,
                                       __nv_bfloat16* __restrict__ out, const int* __restrict__ rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    const int i = threadIdx.x * 8;
    float x[8], wv[8];
    float ss = 0.f;
    if (i < H) {
        float* rrow = resid + (size_t)r * H + i;
        const float4 r0 = *reinterpret_cast<const float4*>(rrow), r1 = *reinterpret_cast<const float4*>(rrow + 4);
        x[0] = r0.x; x[1] = r0.y; x[2] = r0.z; x[3] = r0.w; x[4] = r1.x; x[5] = r1.y; x[6] = r1.z; x[7] = r1.w;
        if (sizeof(TW) == 2) {
            const uint4 wr = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(w) + i);
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
#pragma unroll
            for (int e = 0; e < 4; ++e) { wv[2 * e] = __low2float(w2[e]); wv[2 * e + 1] = __high2float(w2[e]); }
        } else {
            const float4 w0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i);
            const float4 w1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i + 4);
            wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
        }
        if (delta != nullptr) {
            const uint4 dr = *reinterpret_cast<const uint4*>(delta + (size_t)r * H + i);
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dr);
#pragma unroll
            for (int e = 0; e < 4; ++e) { x[2 * e] += __low2float(d2[e]); x[2 * e + 1] += __high2float(d2[e]); }
            if (write_resid) {
                *reinterpret_cast<float4*>(rrow) = make_float4(x[0], x[1], x[2], x[3]);
                *reinterpret_cast<float4*>(rrow + 4) = make_float4(x[4], x[5], x[6], x[7]);
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
    }
    const float total = block_sum(ss, red);
    if (i < H) {
        const float rstd = rsqrtf(total / (float)H + eps);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(x[2 * e] * rstd * wv[2 * e], x[2 * e + 1] * rstd * wv[2 * e + 1]);
        *reinterpret_cast<uint4*>(out + (size_t)j * H + i) = o;
    }
}

// The row form for a delta that is float partial sums [n_parts <= MAXP][rows][H] of a product split
// over K: every part's loads are issued together with the residual's, and the parts are added in
// order.  MAXP 4, or 8 for rows of up to 4096 elements (512 threads: eight parts' loads in flight take registers
// that a CTA of 1024 threads does not have).
template <typename TW, int MAXP>
__global__ void __launch_bounds__(MAXP > 4 ? 512 : 1024)
add_rmsnorm_row_parts_kernel(const float* __restrict__ parts, int n_parts, size_t part_stride,
                                             float* __restrict__ resid, int write_resid, const TW* __restrict__ w, float eps,
                                             __nv_bfloat16* __restrict__ out, const int* __restrict__ rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    const int i = threadIdx.x * 8;
    float x[8], wv[8];
    float ss = 0.f;
    if (i < H) {
        float* rrow = resid + (size_t)r * H + i;
        const float4 r0 = *reinterpret_cast<const float4*>(rrow), r1 = *reinterpret_cast<const float4*>(rrow + 4);
        float4 d[MAXP][2];
#pragma unroll
        for (int pt = 0; pt < MAXP; ++pt)
            if (pt < n_parts) {
                const float* prow = parts + pt * part_stride + (size_t)r * H + i;
                d[pt][0] = *reinterpret_cast<const float4*>(prow);
                d[pt][1] = *reinterpret_cast<const float4*>(prow + 4);
            }
        if (sizeof(TW) == 2) {
            const uint4 wr = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(w) + i);
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
#pragma unroll
            for (int e = 0; e < 4; ++e) { wv[2 * e] = __low2float(w2[e]); wv[2 * e + 1] = __high2float(w2[e]); }
        } else {
            const float4 w0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i);
            const float4 w1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i + 4);
            wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
        }
        x[0] = r0.x; x[1] = r0.y; x[2] = r0.z; x[3] = r0.w; x[4] = r1.x; x[5] = r1.y; x[6] = r1.z; x[7] = r1.w;
        // the residual, then the parts in order: the order of the general kernel
#pragma unroll
        for (int pt = 0; pt < MAXP; ++pt)
            if (pt < n_parts) {
                x[0] += d[pt][0].x; x[1] += d[pt][0].y; x[2] += d[pt][0].z; x[3] += d[pt][0].w;
                x[4] += d[pt][1].x; x[5] += d[pt][1].y; x[6] += d[pt][1].z; x[7] += d[pt][1].w;
            }
        if (write_resid) {
            *reinterpret_cast<float4*>(rrow) = make_float4(x[0], x[1], x[2], x[3]);
            *reinterpret_cast<float4*>(rrow + 4) = make_float4(x[4], x[5], x[6], x[7]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
    }
    const float total = block_sum(ss, red);
    if (i < H) {
        const float rstd = rsqrtf(total / (float)H + eps);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(x[2 * e] * rstd * wv[2 * e], x[2 * e + 1] * rstd * wv[2 * e + 1]);
        *reinterpret_cast<uint4*>(out + (size_t)j * H + i) = o;
    }
}

// ---------------------------------------------------------------------------
// out[m, i] = silu(gu[m, i]) * gu[m, I + i]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < total; e += stride) {
        const size_t m = e / I;
        const int i = (int)(e - m * I);
        const float g = to_float(gu[m * 2 * I + i]);
        const float u = to_float(gu[m * 2 * I + I + i]);
        out[e] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

// ---------------------------------------------------------------------------
// rotary encoding (rotate-half pairing: j with j + d/2) of q and k, and the
// append of the rotated k and of v to the paged cache at the token's position.
//   qkv  [T, (n_q + 2 n_kv) d]   rows: q heads, then k heads, then v heads
//   q_out[T, n_q d]
//   pools [num_blocks, n_kv, block_size, d]
// ---------------------------------------------------------------------------
template <typename TQ, typename TB>
__device__ __forceinline__ float qkv_value(const TQ* __restrict__ qkv, int n_parts, size_t part_stride, size_t idx,
                                           const TB* __restrict__ bias, int col) {
    float v = to_float(qkv[idx]);
    for (int p = 1; p < n_parts; ++p) v += to_float(qkv[p * part_stride + idx]);
    if (bias != nullptr) v += to_float(bias[col]);
    return v;
}

// TQ: element type of the projection's output (T, or float partial sums of a
// split-K product: n_parts arrays part_stride apart, added in index order,
// plus an optional bias of type TB that the product has not added yet).
template <typename T, typename TQ, typename TB>
__global__ void rope_append_kernel(const TQ* __restrict__ qkv, int n_parts, size_t part_stride,
                                   const TB* __restrict__ bias, T* __restrict__ q_out,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                   int table_len, const int* __restrict__ tok_row,
                                   const int* __restrict__ tok_pos, const int* __restrict__ row_slot,
                                   T* __restrict__ k_pool, T* __restrict__ v_pool,
                                   const int* __restrict__ block_table, int max_blocks, int num_blocks,
                                   int block_size, int n_q, int n_kv, int d, int write_kv, int paired,
                                   int* status) {
    const int t = blockIdx.x;
    const int half = d >> 1;
    const int slot = row_slot[tok_row[t]];
    if (slot < 0) return;             // padding row of a fixed-size batch: nothing to do
    int pos = tok_pos[t];
    bool pos_ok = pos >= 0 && pos < table_len;
    if (!pos_ok) {
        if (threadIdx.x == 0) set_status(status, STATUS_BAD_POSITION);
        pos = 0;
    }
    const float* c = cos_t + (size_t)pos * half;
    const float* s = sin_t + (size_t)pos * half;
    const size_t row = (size_t)t * (n_q + 2 * n_kv) * d;

    // destination of this token's keys and values
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (write_kv && pos_ok) {
        const int blk = block_table[(size_t)slot * max_blocks + pos / block_size];
        if (blk < 0 || blk >= num_blocks) {
            if (threadIdx.x == 0) set_status(status, STATUS_BAD_BLOCK);
        } else {
            const size_t base = ((size_t)blk * n_kv * block_size + (pos % block_size)) * d;
            kdst = k_pool + base;
            vdst = v_pool + base;
        }
    }
    const size_t head_stride = (size_t)block_size * d;   // between kv heads inside a block

    const int n_rot = (n_q + n_kv) * half;
    for (int e = threadIdx.x; e < n_rot; e += blockDim.x) {
        const int h = e / half, j = e - h * half;
        // columns of dim j and of its partner j + d/2: natural order, or (paired) tiles of
        // 16 columns holding dims 8t .. 8t+7 and then d/2 + 8t .. d/2 + 8t+7
        const int c1 = paired ? h * d + (j >> 3) * 16 + (j & 7) : h * d + j;
        const int c2 = paired ? c1 + 8 : c1 + half;
        const float x1 = qkv_value(qkv, n_parts, part_stride, row + c1, bias, c1);
        const float x2 = qkv_value(qkv, n_parts, part_stride, row + c2, bias, c2);
        const float cj = c[j], sj = s[j];
        const T y1 = from_float<T>(x1 * cj - x2 * sj);
        const T y2 = from_float<T>(x2 * cj + x1 * sj);
        if (h < n_q) {
            T* o = q_out + ((size_t)t * n_q + h) * d;
            o[j] = y1;
            o[j + half] = y2;
        } else if (kdst != nullptr) {
            T* o = kdst + (h - n_q) * head_stride;
            o[j] = y1;
            o[j + half] = y2;
        }
    }
    if (vdst != nullptr) {
        const int voff = (n_q + n_kv) * d;
        for (int e = threadIdx.x; e < n_kv * d; e += blockDim.x) {
            const int h = e / d, j = e - h * d;
            vdst[h * head_stride + j] = from_float<T>(qkv_value(qkv, n_parts, part_stride, row + voff + e, bias, voff + e));
        }
    }
}

// out[m, i] = silu(g) * u where gate and up values of a row come in tiles of
// 16 columns: 8 gate values, then the 8 up values of the same outputs.
template <typename T>
__global__ void silu_mul_tiled_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; e < total; e += stride) {
        const size_t m = e / I;
        const int i = (int)(e - m * I);
        const size_t base = m * 2 * I + (size_t)(i >> 3) * 16 + (i & 7);
        const float g = to_float(gu[base]);
        const float u = to_float(gu[base + 8]);
        out[e] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

extern "C" int fd_embed(const int* tokens, const void* table, int table_dtype, float* resid,
                        int T, int H, int V, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(H > 0 && V > 0, -2, "embed: bad sizes H=%d V=%d", H, V);
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == 0)
        return launch("embed", embed_kernel<float>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1), tokens,
                      (const float*)table, resid, H, V, status);
    return launch("embed", embed_kernel<bf16>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1), tokens,
                  (const bf16*)table, resid, H, V, status);
}

template <typename TD, typename TO>
static int launch_norm(const void* delta, int n_parts, size_t part_stride, float* resid, int write_resid,
                       const void* w, int w_dtype, float eps, void* out, const int* rows, int n_out, int H,
                       cudaStream_t stream) {
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const size_t smem = (((H + 3) & ~3) + 40) * sizeof(float);
    FD_REQUIRE(smem <= 200 * 1024, -2, "add_rmsnorm: width %d needs %zu bytes of shared memory (max 200 KB)", H, smem);
    if (w_dtype == 0) {
        auto k = add_rmsnorm_kernel<TD, float, TO>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch("add_rmsnorm", k, dim3(n_out), dim3(threads), smem, stream, dim3(1, 1, 1), (const TD*)delta, n_parts,
                      part_stride, resid, write_resid, (const float*)w, eps, (TO*)out, rows, H);
    } else {
        auto k = add_rmsnorm_kernel<TD, bf16, TO>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch("add_rmsnorm", k, dim3(n_out), dim3(threads), smem, stream, dim3(1, 1, 1), (const TD*)delta, n_parts,
                      part_stride, resid, write_resid, (const bf16*)w, eps, (TO*)out, rows, H);
    }
}

// delta_dtype / w_dtype / out_dtype: 0 = float32, 1 = bfloat16.
extern "C" int fd_add_rmsnorm(const void* delta, int delta_dtype, int n_parts, long long part_stride,
                              float* resid, int write_resid, const void* weight, int w_dtype, float eps,
                              void* out, int out_dtype, const int* rows, int n_out, int H,
                              cudaStream_t stream) {
    if (n_out == 0) return 0;
    FD_REQUIRE(H > 0, -2, "add_rmsnorm: bad width %d", H);
    FD_REQUIRE(delta == nullptr || n_parts >= 1, -2, "add_rmsnorm: n_parts=%d", n_parts);
    const size_t ps = (size_t)part_stride;
    if (out_dtype == 1 && (delta == nullptr || (delta_dtype == 1 && n_parts == 1)) && H % 8 == 0 && H <= 8192 &&
        (uintptr_t)resid % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)weight % 16 == 0 &&
        (uintptr_t)delta % 16 == 0) {
        const int threads = ((H / 8 + 31) / 32) * 32;
        if (w_dtype == 0)
            return launch("add_rmsnorm", add_rmsnorm_row_kernel<float>, dim3(n_out), dim3(threads), 0, stream, dim3(1, 1, 1),
                          (const bf16*)delta, resid, write_resid, (const float*)weight, eps, (bf16*)out, rows, H);
        return launch("add_rmsnorm", add_rmsnorm_row_kernel<bf16>, dim3(n_out), dim3(threads), 0, stream, dim3(1, 1, 1),
                      (const bf16*)delta, resid, write_resid, (const bf16*)weight, eps, (bf16*)out, rows, H);
    }
    if (out_dtype == 1 && delta != nullptr && delta_dtype == 0 && (n_parts <= 4 || (n_parts <= 8 && H <= 4096)) && H % 8 == 0 &&
        H <= 8192 && ps % 4 == 0 &&
        (uintptr_t)resid % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)weight % 16 == 0 && (uintptr_t)delta % 16 == 0) {
        const int threads = ((H / 8 + 31) / 32) * 32;
        if (n_parts <= 4) {
            if (w_dtype == 0)
                return launch("add_rmsnorm", add_rmsnorm_row_parts_kernel<float, 4>, dim3(n_out), dim3(threads), 0, stream, dim3(1, 1, 1),
                              (const float*)delta, n_parts, ps, resid, write_resid, (const float*)weight, eps, (bf16*)out, rows, H);
            return launch("add_rmsnorm", add_rmsnorm_row_parts_kernel<bf16, 4>, dim3(n_out), dim3(threads), 0, stream, dim3(1, 1, 1),
                          (const float*)delta, n_parts, ps, resid, write_resid, (const bf16*)weight, eps, (bf16*)out, rows, H);
        }
        if (w_dtype == 0)
            return launch("add_rmsnorm", add_rmsnorm_row_parts_kernel<float, 8>, dim3(n_out), dim3(threads), 0, stream, dim3(1, 1, 1),
                          (const float*)delta, n_parts, ps, resid, write_resid, (const float*)weight, eps, (bf16*)out, rows, H);
        return launch("add_rmsnorm", add_rmsnorm_row_parts_kernel<bf16, 8>, dim3(n_out), dim3(threads), 0, stream, dim3(1, 1, 1),
                      (const float*)delta, n_parts, ps, resid, write_resid, (const bf16*)weight, eps, (bf16*)out, rows, H);
    }
    if (delta_dtype == 0 && out_dtype == 0)
        return launch_norm<float, float>(delta, n_parts, ps, resid, write_resid, weight, w_dtype, eps, out, rows, n_out, H, stream);
    if (delta_dtype == 1 && out_dtype == 1)
        return launch_norm<bf16, bf16>(delta, n_parts, ps, resid, write_resid, weight, w_dtype, eps, out, rows, n_out, H, stream);
    if (delta_dtype == 0 && out_dtype == 1)
        return launch_norm<float, bf16>(delta, n_parts, ps, resid, write_resid, weight, w_dtype, eps, out, rows, n_out, H, stream);
    return fail(-2, "add_rmsnorm: unsupported dtypes delta=%d out=%d", delta_dtype, out_dtype);
}

// tiled == 0: gu = [gate (I columns) | up (I columns)]; tiled != 0: tiles of 8 gate + 8 up columns.
extern "C" int fd_silu_mul(const void* gu, void* out, int dtype, int M, int I, int tiled, cudaStream_t stream) {
    const size_t total = (size_t)M * I;
    if (total == 0) return 0;
    FD_REQUIRE(!tiled || I % 8 == 0, -2, "silu_mul: the tiled layout needs a multiple of 8 outputs, got %d", I);
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == 0) {
        if (tiled) silu_mul_tiled_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
        else silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
    } else {
        if (tiled) silu_mul_tiled_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, I, total);
        else silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, I, total);
    }
    return check_launch("silu_mul");
}

// qkv_dtype: element type of `qkv` (0 float, 1 bfloat16); with n_parts > 1 it
// holds float partial sums part_stride elements apart.  bias (dtype bias_dtype)
// may be null.  dtype: type of q_out and of the cache.  paired != 0: the
// columns of every q and k head are in tiles of 8 dims + their 8 rotation
// partners (the row order the decode projection kernel wants of W).
extern "C" int fd_rope_append(const void* qkv, int qkv_dtype, int n_parts, long long part_stride,
                              const void* bias, int bias_dtype, void* q_out, int dtype, const float* cos_t,
                              const float* sin_t, int table_len, const int* tok_row, const int* tok_pos,
                              const int* row_slot, void* k_pool, void* v_pool, const int* block_table,
                              int max_blocks, int num_blocks, int block_size, int T, int n_q, int n_kv, int d,
                              int write_kv, int paired, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(d > 0 && d % 2 == 0, -2, "rope_append: head size %d must be even", d);
    FD_REQUIRE(!paired || d % 16 == 0, -2, "rope_append: the paired column order needs a head size that is a multiple of 16, got %d", d);
    FD_REQUIRE(block_size > 0 && n_q > 0 && n_kv > 0, -2, "rope_append: bad sizes");
    FD_REQUIRE(n_parts >= 1 && (n_parts == 1 || qkv_dtype == 0), -2, "rope_append: partial sums must be float");
    const int work = (n_q + n_kv) * d / 2;
    const int threads = work >= 512 ? 256 : 128;
    const size_t ps = (size_t)part_stride;
#define FD_ROPE_LAUNCH(T_, TQ_, TB_)                                                                          \
    rope_append_kernel<T_, TQ_, TB_><<<T, threads, 0, stream>>>(                                               \
        (const TQ_*)qkv, n_parts, ps, (const TB_*)bias, (T_*)q_out, cos_t, sin_t, table_len, tok_row, tok_pos, \
        row_slot, (T_*)k_pool, (T_*)v_pool, block_table, max_blocks, num_blocks, block_size, n_q, n_kv, d,     \
        write_kv, paired, status)
    if (dtype == 0) {
        FD_REQUIRE(qkv_dtype == 0 && (bias == nullptr || bias_dtype == 0), -2, "rope_append: float32 path takes float32 inputs");
        FD_ROPE_LAUNCH(float, float, float);
    } else if (qkv_dtype == 1) {
        if (bias != nullptr && bias_dtype == 0) FD_ROPE_LAUNCH(bf16, bf16, float);
        else FD_ROPE_LAUNCH(bf16, bf16, bf16);
    } else {
        if (bias != nullptr && bias_dtype == 0) FD_ROPE_LAUNCH(bf16, float, float);
        else FD_ROPE_LAUNCH(bf16, float, bf16);
    }
#undef FD_ROPE_LAUNCH
    return check_launch("rope_append");
}
