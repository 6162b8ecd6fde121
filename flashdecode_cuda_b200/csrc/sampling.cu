// Token choice from float logits: greedy (argmax, lowest index wins a tie) or
// temperature sampling by the Gumbel-max rule,
//     token = argmax_i ( logit_i / T + g_i ),   g_i = -log(-log(u_i)),
// which draws exactly from softmax(logits / T) without a prefix sum.  The
// uniform u_i = ((x_i >> 9) + 0.5) / 2^23 (exact in float, never 0 or 1) comes from Philox-4x32-10 with counter (i / 4, step, request)
// and key (seed): a draw depends on the request, its step and the vocabulary
// index only, never on which other rows share the batch.
#include <math.h>

#include "common.cuh"

namespace fd {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    return v > bv || (v == bv && i < bi);
}

constexpr int SAMPLE_CHUNK = 4096;      // vocabulary entries per CTA (a multiple of 4: one Philox call gives 4)
constexpr int SAMPLE_THREADS = 256;

// Score of vocabulary entry i of a row: the logit (greedy) or logit / T + Gumbel noise.
// A CTA scans one chunk of one row and keeps the best (score, index), the
// lowest index winning ties; temperature[row] <= 0 means greedy.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_partial_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                      const long long* __restrict__ request, const int* __restrict__ step,
                      unsigned long long seed, const unsigned long long* __restrict__ seed_ptr,
                      float* __restrict__ part_v, int* __restrict__ part_i, int* __restrict__ out, int n_chunks) {
    pdl_launch_dependents();
    pdl_wait();
    if (seed_ptr != nullptr) seed = *seed_ptr;       // a seed kept on the device: a captured graph serves every seed
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float* x = logits + (size_t)row * V;
    const float temp = temperature ? temperature[row] : 0.f;
    const int begin = chunk * SAMPLE_CHUNK, end = min(V, begin + SAMPLE_CHUNK);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if (temp <= 0.f) {
        for (int i = begin + threadIdx.x; i < end; i += SAMPLE_THREADS) {
            const float v = x[i];
            if (better(v, i, bv, bi)) { bv = v; bi = i; }
        }
    } else {
        const unsigned long long rq = (unsigned long long)request[row];
        const uint32_t st = (uint32_t)step[row];
        const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
        for (int j = begin / 4 + threadIdx.x; j * 4 < end; j += SAMPLE_THREADS) {
            uint32_t r[4];
            philox4x32_10((uint32_t)j, st, (uint32_t)rq, (uint32_t)(rq >> 32), k0, k1, r);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = j * 4 + e;
                if (i < end) {
                    const float u = ((float)(r[e] >> 9) + 0.5f) * (1.0f / 8388608.0f);
                    const float v = x[i] / temp + (-logf(-logf(u)));
                    if (better(v, i, bv, bi)) { bv = v; bi = i; }
                }
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    __shared__ float sv[SAMPLE_THREADS / 32];
    __shared__ int si[SAMPLE_THREADS / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < SAMPLE_THREADS / 32 ? sv[lane] : -INFINITY;
        bi = lane < SAMPLE_THREADS / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            if (n_chunks == 1) {
                out[row] = bi == 0x7fffffff ? 0 : bi;
            } else {
                part_v[(size_t)row * n_chunks + chunk] = bv;
                part_i[(size_t)row * n_chunks + chunk] = bi;
            }
        }
    }
}

// One warp per row merges the chunks' winners.
__global__ void sample_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int n_chunks, int* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, lane = threadIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = lane; c < n_chunks; c += 32) {
        const float v = part_v[(size_t)row * n_chunks + c];
        const int i = part_i[(size_t)row * n_chunks + c];
        if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

}  // namespace fd

using namespace fd;

// 4-byte words of scratch that fd_sample needs for n rows of V logits.
extern "C" long long fd_sample_scratch_words(int n, int V) {
    const long long chunks = (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    return chunks > 1 ? 2 * chunks * n : 0;
}

// logits [n, V] float; temperature [n] float or null (all greedy); request [n]
// int64 and step [n] int32 (needed when any temperature is > 0); out [n] int32;
// scratch: fd_sample_scratch_words(n, V) words (may be null when that is 0).  seed_ptr (optional): the seed is
// read from there (device memory) instead of `seed`.
extern "C" int fd_sample(const float* logits, int n, int V, const float* temperature,
                         const long long* request, const int* step, unsigned long long seed,
                         const unsigned long long* seed_ptr, int* out, void* scratch, cudaStream_t stream) {
    if (n == 0) return 0;
    FD_REQUIRE(V > 0, -2, "sample: vocabulary %d", V);
    FD_REQUIRE(n <= 65535, -2, "sample: %d rows in one call", n);
    FD_REQUIRE(temperature == nullptr || (request != nullptr && step != nullptr), -2,
               "sample: temperature sampling needs request ids and step counters");
    const int chunks = (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    FD_REQUIRE(chunks == 1 || scratch != nullptr, -2, "sample: a vocabulary of %d needs scratch memory", V);
    float* part_v = (float*)scratch;
    int* part_i = (int*)scratch + (size_t)chunks * n;
    dim3 grid(chunks, n);
    sample_partial_kernel<<<grid, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, request, step, seed, seed_ptr,
                                                             part_v, part_i, out, chunks);
    int rc = check_launch("sample");
    if (rc != 0 || chunks == 1) return rc;
    sample_final_kernel<<<n, 32, 0, stream>>>(part_v, part_i, chunks, out);
    return check_launch("sample_final");
}

// ---------------------------------------------------------------------------
// The variant that allocates nothing (declared and described in no_alloc.h).
// ---------------------------------------------------------------------------
#include "no_alloc.h"

// Per-chunk winners of the rows of one call: scores first, then indices.  In
// host code this name is only a handle for cudaGetSymbolAddress; it is not a
// device pointer and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned int g_no_alloc_scratch[2 * FD_NO_ALLOC_MAX_ROWS * FD_NO_ALLOC_MAX_CHUNKS];

namespace {
constexpr int NO_ALLOC_MAX_DEVICES = 64;
void* g_no_alloc_ptr[NO_ALLOC_MAX_DEVICES] = {nullptr};   // device address of the array, per device
}

extern "C" int fd_sample_no_alloc(const float* logits, int n, int V, const float* temperature,
                                  const long long* request, const int* step, unsigned long long seed, int* out,
                                  cudaStream_t stream) {
    if (n == 0) return 0;
    FD_REQUIRE(V > 0, -2, "sample_no_alloc: vocabulary %d", V);
    FD_REQUIRE(n > 0 && n <= FD_NO_ALLOC_MAX_ROWS, -2,
               "sample_no_alloc: %d rows in one call, the static scratch array holds at most %d", n,
               FD_NO_ALLOC_MAX_ROWS);
    const int chunks = (V + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    FD_REQUIRE(chunks <= FD_NO_ALLOC_MAX_CHUNKS, -2,
               "sample_no_alloc: a vocabulary of %d needs %d chunks, the static scratch array holds at most %d "
               "(vocabularies up to %d)", V, chunks, FD_NO_ALLOC_MAX_CHUNKS, FD_NO_ALLOC_MAX_CHUNKS * SAMPLE_CHUNK);
    FD_REQUIRE(temperature == nullptr || (request != nullptr && step != nullptr), -2,
               "sample_no_alloc: temperature sampling needs request ids and step counters");

    // set-up, once per device, with that device current: the array's device address
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(-1, "sample_no_alloc: cudaGetDevice: %s", cudaGetErrorString(e));
    FD_REQUIRE(dev >= 0 && dev < NO_ALLOC_MAX_DEVICES, -2, "sample_no_alloc: device index %d", dev);
    if (g_no_alloc_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_no_alloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(-3, "sample_no_alloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_no_alloc_ptr[dev] = ptr;
    }
    float* part_v = static_cast<float*>(g_no_alloc_ptr[dev]);
    int* part_i = static_cast<int*>(g_no_alloc_ptr[dev]) + (size_t)chunks * n;

    dim3 grid(chunks, n);
    sample_partial_kernel<<<grid, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, request, step, seed, nullptr,
                                                             part_v, part_i, out, chunks);
    int rc = check_launch("sample_no_alloc");
    if (rc != 0 || chunks == 1) return rc;
    sample_final_kernel<<<n, 32, 0, stream>>>(part_v, part_i, chunks, out);
    return check_launch("sample_no_alloc_final");
}
