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
    switch (key) {
        case 0: return launch<float, float, float>(A, W, bias, C, M, N, K, stream);
        case 4 + 2 + 1: return launch<bf16, bf16, bf16>(A, W, bias, C, M, N, K, stream);
        case 4 + 2 + 0: return launch<bf16, bf16, float>(A, W, bias, C, M, N, K, stream);
        case 4 + 0 + 1: return launch<bf16, float, bf16>(A, W, bias, C, M, N, K, stream);
        case 4 + 0 + 0: return launch<bf16, float, float>(A, W, bias, C, M, N, K, stream);
        default: return fail(-2, "gemm_simt: unsupported dtypes in=%d bias=%d out=%d", dtype, bias_dtype, out_dtype);
    }
}
