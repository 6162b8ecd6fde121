// C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]) on the CUDA cores.
//
// This is the matrix product of the true 32-bit path: FFMA only, no tensor
// cores, no reduced-precision mode, no split-K.  Every output element is one
// fmaf chain over k = 0 .. K-1 in that order, so its value does not depend on
// M, N, the tile it falls in or what else is in the batch: a token gives the
// same bits whether it is run alone, in a prompt or in a batch.  The bfloat16
// instantiation (float accumulation) is the fallback for sizes the tensor-core
// kernels refuse.
#include "common.cuh"

namespace fd {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename T>
__device__ __forceinline__ void load4(const T* p, bool vec_ok, int valid, float out[4]);

template <>
__device__ __forceinline__ void load4<float>(const float* p, bool vec_ok, int valid, float out[4]) {
    if (vec_ok && valid == 4) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = i < valid ? p[i] : 0.f;
    }
}

template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, bool vec_ok, int valid, float out[4]) {
    if (vec_ok && valid == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
        out[0] = __low2float(a); out[1] = __high2float(a);
        out[2] = __low2float(b); out[3] = __high2float(b);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = i < valid ? __bfloat162float(p[i]) : 0.f;
    }
}

template <typename T, typename TB, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, const TB* __restrict__ bias,
                 TO* __restrict__ C, int M, int N, int K, int vec_ok) {
    __shared__ float As[BK][BM + PAD];
    __shared__ float Bs[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // each thread stages 4 consecutive k of one row of A and one row of W
    const int lrow = tid >> 2, lk = (tid & 3) * 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float av[4], wv[4];
        const int kk = k0 + lk;
        const int valid = K - kk >= 4 ? 4 : (K - kk > 0 ? K - kk : 0);
        if (m0 + lrow < M && valid > 0) load4<T>(A + (size_t)(m0 + lrow) * K + kk, vec_ok, valid, av);
        else { av[0] = av[1] = av[2] = av[3] = 0.f; }
        if (n0 + lrow < N && valid > 0) load4<T>(W + (size_t)(n0 + lrow) * K + kk, vec_ok, valid, wv);
        else { wv[0] = wv[1] = wv[2] = wv[3] = 0.f; }
        __syncthreads();   // previous tile fully consumed
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lrow] = av[i];
            Bs[lk + i][lrow] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float ar[4] = {a.x, a.y, a.z, a.w};
            const float br[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias != nullptr) v += to_float(bias[n]);
            C[(size_t)m * N + n] = from_float<TO>(v);
        }
    }
}

// The same product for up to 16 rows of A in float32 (the decode steps of the 32-bit path), built around
// the stream of W: a CTA takes 64 rows of W and all rows of A, k in steps of 32; the loads of the next step are
// in flight in registers while this one is computed, and several CTAs share an SM.  Every output element is the
// SAME fmaf chain over k = 0 .. K-1 as in the kernel above (zeros beyond K add nothing), so a token gives the
// same bits through either.
constexpr int RN = 64, RK = 32, RM = 16;

__global__ void __launch_bounds__(256)
gemm_simt_rows_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                      float* __restrict__ C, int M, int N, int K, int vec_ok) {
    __shared__ float Ws[RK][RN + 1];            // [k][row of W]: a warp reads 32 neighbouring rows of one k
    __shared__ __align__(16) float As[RK][RM];  // [k][row of A]: read as one float4 per four rows
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * RN;
    const int nl = tid & 63, mg = tid >> 6;     // this thread's row of W and its four rows of A
    // staging: two float4 of W per thread (rows tid / 8 and tid / 8 + 32, k 4 (tid % 8) ..), one of A for threads < 128
    const int lrow = tid >> 3, lk = (tid & 7) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float w0[4], w1[4], av[4];
    auto fetch = [&](int k0) {
        const int kk = k0 + lk;
        const int valid = K - kk >= 4 ? 4 : (K - kk > 0 ? K - kk : 0);
        w0[0] = w0[1] = w0[2] = w0[3] = 0.f;
        w1[0] = w1[1] = w1[2] = w1[3] = 0.f;
        av[0] = av[1] = av[2] = av[3] = 0.f;
        if (valid > 0) {
            if (n0 + lrow < N) load4<float>(W + (size_t)(n0 + lrow) * K + kk, vec_ok, valid, w0);
            if (n0 + lrow + 32 < N) load4<float>(W + (size_t)(n0 + lrow + 32) * K + kk, vec_ok, valid, w1);
            if (tid < 128 && lrow < M) load4<float>(A + (size_t)lrow * K + kk, vec_ok, valid, av);
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += RK) {
        __syncthreads();   // previous tile fully consumed
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            Ws[lk + i][lrow] = w0[i];
            Ws[lk + i][lrow + 32] = w1[i];
            if (tid < 128) As[lk + i][lrow] = av[i];
        }
        __syncthreads();
        if (k0 + RK < K) fetch(k0 + RK);        // on their way while this tile is computed
#pragma unroll
        for (int k = 0; k < RK; ++k) {
            const float w = Ws[k][nl];
            const float4 a = *reinterpret_cast<const float4*>(&As[k][mg * 4]);
            acc[0] = fmaf(a.x, w, acc[0]);
            acc[1] = fmaf(a.y, w, acc[1]);
            acc[2] = fmaf(a.z, w, acc[2]);
            acc[3] = fmaf(a.w, w, acc[3]);
        }
    }
    const int n = n0 + nl;
    if (n >= N) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = mg * 4 + i;
        if (m >= M) continue;
        float v = acc[i];
        if (bias != nullptr) v += bias[n];
        C[(size_t)m * N + n] = v;
    }
}

// The same again for matrices with few rows (the q/k/v, o and down projections: N / 64 CTAs would leave most SMs
// idle): 16 rows of W per CTA, k in steps of 128, the same 8 KB of W per step and the same chain per output.
constexpr int SN = 16, SK = 128;

__global__ void __launch_bounds__(256)
gemm_simt_rows_narrow_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                             float* __restrict__ C, int M, int N, int K, int vec_ok) {
    __shared__ float Ws[SK][SN + 1];
    __shared__ float As[SK][RM + 1];         // odd strides: the staging stores of a warp (32 values of k, one row) spread over the banks
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * SN;
    const int nl = tid & 15, mg = (tid >> 4) & 3;          // threads 0..63 compute: a row of W, four rows of A
    // staging: rows tid / 32 and tid / 32 + 8 of both W and A, k 4 (tid % 32) ..
    const int lrow = tid >> 5, lk = (tid & 31) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float w0[4], w1[4], a0[4], a1[4];
    auto fetch = [&](int k0) {
        const int kk = k0 + lk;
        const int valid = K - kk >= 4 ? 4 : (K - kk > 0 ? K - kk : 0);
#pragma unroll
        for (int i = 0; i < 4; ++i) w0[i] = w1[i] = a0[i] = a1[i] = 0.f;
        if (valid > 0) {
            if (n0 + lrow < N) load4<float>(W + (size_t)(n0 + lrow) * K + kk, vec_ok, valid, w0);
            if (n0 + lrow + 8 < N) load4<float>(W + (size_t)(n0 + lrow + 8) * K + kk, vec_ok, valid, w1);
            if (lrow < M) load4<float>(A + (size_t)lrow * K + kk, vec_ok, valid, a0);
            if (lrow + 8 < M) load4<float>(A + (size_t)(lrow + 8) * K + kk, vec_ok, valid, a1);
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += SK) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            Ws[lk + i][lrow] = w0[i];
            Ws[lk + i][lrow + 8] = w1[i];
            As[lk + i][lrow] = a0[i];
            As[lk + i][lrow + 8] = a1[i];
        }
        __syncthreads();
        if (k0 + SK < K) fetch(k0 + SK);
        if (tid < 64) {
#pragma unroll 16
            for (int k = 0; k < SK; ++k) {
                const float w = Ws[k][nl];
                acc[0] = fmaf(As[k][mg * 4], w, acc[0]);
                acc[1] = fmaf(As[k][mg * 4 + 1], w, acc[1]);
                acc[2] = fmaf(As[k][mg * 4 + 2], w, acc[2]);
                acc[3] = fmaf(As[k][mg * 4 + 3], w, acc[3]);
            }
        }
    }
    const int n = n0 + nl;
    if (tid >= 64 || n >= N) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = mg * 4 + i;
        if (m >= M) continue;
        float v = acc[i];
        if (bias != nullptr) v += bias[n];
        C[(size_t)m * N + n] = v;
    }
}

template <typename T, typename TB, typename TO>
static int launch(const void* A, const void* W, const void* bias, void* C, int M, int N, int K,
                  cudaStream_t stream) {
    const size_t esz = sizeof(T) * 4;   // bytes of one 4-element vector
    const int vec_ok = (K % 4 == 0) && ((uintptr_t)A % esz == 0) && ((uintptr_t)W % esz == 0);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_simt_kernel<T, TB, TO><<<grid, 256, 0, stream>>>((const T*)A, (const T*)W, (const TB*)bias, (TO*)C,
                                                         M, N, K, vec_ok);
    return check_launch("gemm_simt");
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// dtype: element type of A and W; bias_dtype, out_dtype: 0 = float32, 1 = bfloat16.
extern "C" int fd_gemm_simt(const void* A, const void* W, const void* bias, void* C, int dtype,
                            int bias_dtype, int out_dtype, int M, int N, int K, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    FD_REQUIRE(K > 0, -2, "gemm_simt: K=%d", K);
    FD_REQUIRE((M + BM - 1) / BM <= 65535, -2, "gemm_simt: M=%d too large for one launch", M);
    const int key = dtype * 4 + (bias ? bias_dtype : dtype) * 2 + out_dtype;
    if (key == 0 && M <= RM) {
        const int vec_ok = (K % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
        if (N <= 64 * 148 && K >= 512)
            gemm_simt_rows_narrow_kernel<<<(N + SN - 1) / SN, 256, 0, stream>>>((const float*)A, (const float*)W, (const float*)bias,
                                                                               (float*)C, M, N, K, vec_ok);
        else
            gemm_simt_rows_kernel<<<(N + RN - 1) / RN, 256, 0, stream>>>((const float*)A, (const float*)W, (const float*)bias,
                                                                        (float*)C, M, N, K, vec_ok);
        return check_launch("gemm_simt_rows");
    }
    switch (key) {
        case 0: return launch<float, float, float>(A, W, bias, C, M, N, K, stream);
        case 4 + 2 + 1: return launch<bf16, bf16, bf16>(A, W, bias, C, M, N, K, stream);
        case 4 + 2 + 0: return launch<bf16, bf16, float>(A, W, bias, C, M, N, K, stream);
        case 4 + 0 + 1: return launch<bf16, float, bf16>(A, W, bias, C, M, N, K, stream);
        case 4 + 0 + 0: return launch<bf16, float, float>(A, W, bias, C, M, N, K, stream);
        default: return fail(-2, "gemm_simt: unsupported dtypes in=%d bias=%d out=%d", dtype, bias_dtype, out_dtype);
    }
}
