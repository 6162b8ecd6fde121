// Shared device helpers for the sm_100a kernels of this library.
//
// Conventions used by every kernel file:
//  * activations and weights are `float` (true 32-bit path) or `__nv_bfloat16`
//    (serving path); every reduction, softmax, norm and rotation is done in
//    float and rounded once on store;
//  * every launcher is `extern "C"`, takes raw device pointers and a stream,
//    launches without allocating, and returns 0 or a negative error code whose
//    text `fd_last_error()` gives;
//  * kernels that index through tables (token ids, block tables) check the
//    index and, instead of faulting, skip the access and set a bit in a status
//    word that the host reads at its next synchronisation.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fd {

// status bits written by kernels (host: flashdecode_cuda_b200/kernels.py)
constexpr int STATUS_BAD_TOKEN = 1;       // token id outside the embedding table
constexpr int STATUS_BAD_BLOCK = 2;       // block table entry < 0 or >= num_blocks where a token lies
constexpr int STATUS_BAD_POSITION = 4;    // position beyond the rotation table
constexpr int STATUS_WAIT_TIMEOUT = 8;    // a bounded mbarrier wait gave up

__device__ __forceinline__ void set_status(int* status, int bit) {
    if (status != nullptr) atomicOr(status, bit);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a thread block; every thread gets the result.  `scratch` holds at
// least 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    const float total = scratch[32];
    __syncthreads();
    return total;
}

}  // namespace fd

namespace fd {

// Programmatic dependent launch.  A kernel launched through fd::launch may begin while the
// kernel before it in the stream is still running: it calls pdl_launch_dependents() at its
// top (so the one after it can be set up early too), does what depends on nothing written by
// earlier kernels (fetching weights), and calls pdl_wait() before it first touches anything an
// earlier kernel wrote or still reads.  pdl_wait() returns once every earlier kernel has
// completed and its writes are visible.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace fd

namespace fd {
// This CTA's share (by its place in the grid) of `bytes` at `ptr` (16-byte aligned) that a later kernel will stream:
// asked for from L2 as bulk prefetches of up to 128 KB (with 16 KB pieces a CTA of a small grid issued sixteen of them,
// a couple of microseconds of one thread's time: the step at batch 1 is 1 % faster this way, at batch 8 the same).
// Called by ONE thread of every CTA of the grid.
__device__ __forceinline__ void l2_prefetch_share(const unsigned char* ptr, unsigned long long bytes) {
    const unsigned long long n_ctas = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
    const unsigned long long cta = ((unsigned long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    const unsigned long long per = ((bytes + n_ctas - 1) / n_ctas + 127) & ~127ull;
    const unsigned long long lo = cta * per;
    if (lo >= bytes) return;
    const unsigned long long hi = lo + per < bytes ? lo + per : (bytes & ~15ull);
    for (unsigned long long o = lo; o < hi; o += 131072) {
        const unsigned n = (unsigned)(hi - o < 131072 ? hi - o : 131072);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(ptr + o), "r"(n) : "memory");
    }
}
}  // namespace fd

// error reporting shared by the launchers (defined in runtime.cu)
extern "C" const char* fd_last_error();
namespace fd {
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
}  // namespace fd

namespace fd {
extern int g_pdl;      // 1: launches carry the programmatic-serialization attribute (runtime.cu)
extern unsigned long long g_launches;      // kernels of this library launched so far (runtime.cu)

// Launch with the attributes this library uses: programmatic dependent launch (when enabled)
// and an optional thread-block cluster shape.
template <typename... KArgs, typename... Args>
inline int launch(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                  dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int n = 0;
    if (g_pdl) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = cluster.x;
        attrs[n].val.clusterDim.y = cluster.y;
        attrs[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return fail(-100, "%s: launch failed: %s", what, cudaGetErrorString(e));
    ++g_launches;
    return 0;
}
}  // namespace fd

#define FD_REQUIRE(cond, code, ...) \
    do { if (!(cond)) return fd::fail(code, __VA_ARGS__); } while (0)
