// What the TMA + tcgen05 matrix-product kernels of this library share: PTX wrappers (mbarriers with
// bounded waits, tiled bulk copies, tcgen05.mma / commit / ld, cluster addressing), the shared-memory
// descriptor of a 128-byte-swizzled K-major tile, the arguments of the q/k/v epilogue, and on the host
// the tensor maps (made through the driver's cuTensorMapEncodeTiled, cached by address and shape).
//
// Every wait on an mbarrier is bounded in time.  When one runs out the waiting thread sets an abort
// flag in its CTA's shared memory and STATUS_WAIT_TIMEOUT in the status word; every role then leaves
// its loop, copies in flight are waited for, tensor memory is freed and the kernel returns (wrong
// output, a reported error, no hang).
#pragma once

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace fd {

constexpr unsigned long long TC_WAIT_NS = 200ull * 1000 * 1000;   // 0.2 s per wait, then give up

// Set by fd_tc_test_hook (tests only): the limit of every bounded wait, and whether the TMA producer
// leaves out the last copy of its last stage, so that a wait runs out without anything being wrong.
inline unsigned long long g_tc_wait_ns = TC_WAIT_NS;
inline int g_tc_skip_last = 0;

// The q/k/v epilogue: the rows of W (columns of the product) are the q heads, the k heads, then the v
// heads; inside a q or k head they come in tiles of 16: dims 8t .. 8t+7, then their rotation
// partners d/2 + 8t .. d/2 + 8t+7; v heads in natural order.  `out` is q_out [M, n_q d].
struct TcRope {
    const float* cos_t;          // [table_len, d/2]
    const float* sin_t;
    const int* tok_row;          // [M]
    const int* tok_pos;          // [M]
    const int* row_slot;
    __nv_bfloat16* k_pool;       // [num_blocks, n_kv, block_size, d]
    __nv_bfloat16* v_pool;
    const int* block_table;
    int table_len, max_blocks, num_blocks, block_size;
    int n_q, n_kv, d, write_kv;
};

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait for the phase with the given parity.  False: the time ran out (or another
// thread already gave up); the caller leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t spins = 0;; ++spins) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((spins & 63) != 63) continue;                    // the clock and the flag only now and then
        if (*abort_flag) return false;
        if (t0 == 0) t0 = global_ns();
        else if (global_ns() - t0 > limit_ns) {
            *abort_flag = 1;
            set_status(status, STATUS_WAIT_TIMEOUT);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t v[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t v[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes, laid out
// by TMA with the 128-byte swizzle: 8-row groups of 1024 bytes (SBO), version 1, layout 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);       // start address, 16-byte units
    d |= (uint64_t)1 << 16;                       // leading byte offset: not used by swizzled K-major layouts
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                       // 128-byte swizzle
    return d;
}

// ---- thread-block clusters --------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the shared::cluster address of the same variable in the CTA of the given rank
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// A float out of the shared memory of any CTA of the cluster (address from map_to_rank).  Volatile, so
// that a run of these stays in program order and ahead of the arithmetic that uses them.
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr_cluster) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr_cluster));
    return v;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr_cluster, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr_cluster), "f"(v) : "memory");
}

// ---- host side ------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// Tensor map of a row-major bf16 matrix [rows, cols] read in boxes of box_rows rows x 64 columns with the
// 128-byte swizzle; rows and columns beyond the matrix read as zero.  Maps are cached by (address, shape,
// box): weights and workspace buffers keep their addresses.
inline int tensor_map(const void* ptr, int rows, int cols, CUtensorMap* out, int box_rows) {
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(ptr, rows, cols, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return fail(-4, "tcgen05 product: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(-4, "tcgen05 product: cuTensorMapEncodeTiled failed with code %d for a %d x %d matrix", (int)r, rows, cols);
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return 0;
}

// Three-dimensional tensor map of a row-major bf16 matrix [rows, cols], cols a multiple of 64:
// (k inside a block of 64, row, k-block), read in boxes of 64 x box_rows x kb, so that ONE copy brings kb
// swizzled [box_rows x 64] tiles one after another.  Returns 1 if the driver refuses the layout.
inline int tensor_map_blocks(const void* ptr, int rows, int cols, CUtensorMap* out, int box_rows, int kb) {
    static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(ptr, rows, cols, box_rows, kb);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return 1;
    cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 2, 128u};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)kb};
    cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return 0;
}

}  // namespace fd
