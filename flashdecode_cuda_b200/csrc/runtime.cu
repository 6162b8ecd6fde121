// Error reporting and device queries shared by all launchers.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace {
thread_local char g_error[512] = "";
}

extern "C" const char* fd_last_error() { return g_error; }

namespace fd {

int g_pdl = 0;
unsigned long long g_launches = 0;

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

// After a kernel<<<...>>> launch: its error, if any; counts the launch otherwise.
int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(-100, "%s: launch failed: %s", what, cudaGetErrorString(e));
    ++g_launches;
    return 0;
}

}  // namespace fd

// Compute capability of the current device as major*10+minor, or a negative
// error code.  The package refuses to run on anything but 10.x.
extern "C" int fd_device_arch() {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fd::fail(-1, "no CUDA device");
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    return major * 10 + minor;
}

extern "C" int fd_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fd::fail(-1, "no CUDA device");
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
}

// Kernels of this library launched so far by this process (every launch goes through fd::launch or
// fd::check_launch), captured launches included: one count per launch call, not per replay of a graph.
extern "C" unsigned long long fd_launch_count() { return fd::g_launches; }

// Turn programmatic dependent launch on (1) or off (0, the default) for later launches.
extern "C" int fd_set_pdl(int on) {
    fd::g_pdl = on ? 1 : 0;
    return 0;
}

// One asynchronous copy from pinned host memory to the device on the given stream (the per-step index
// array of a decode step; a plain call costs a fraction of a tensor-library copy on the host).
// One copy from the device into pinned host memory on the given stream, and the wait for it: what a decode step's
// tokens cost on their way to the host (one call instead of a tensor-library copy and a stream object's synchronize).
extern "C" int fd_copy_d2h_sync(void* dst, const void* src, long long bytes, cudaStream_t stream) {
    if (bytes <= 0) return 0;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fd::fail(-100, "copy to the host failed: %s", cudaGetErrorString(e));
    return 0;
}

extern "C" int fd_copy_h2d_async(void* dst, const void* src, long long bytes, cudaStream_t stream) {
    if (bytes <= 0) return 0;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fd::fail(-100, "copy to the device failed: %s", cudaGetErrorString(e));
    return 0;
}
