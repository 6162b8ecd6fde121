// Decode attention (one new token per sequence) over the paged bfloat16 cache
// on the tensor cores: split-KV flash-decoding.
//
// A CTA serves one (sequence, KV head, split of the keys); its 4 or 8 warps take
// 16-key tiles of the split round-robin, each with its own three-stage
// cp.async pipeline into swizzled shared memory and its own online-softmax
// state, so the main loop has no block-wide barrier.  All G query heads of the
// KV head form the M = 16 rows of the tile (rows >= G are zero), so every key
// and value byte is read from HBM once for the whole group:
//     S[16 heads, 16 keys]  = Q[16, D] K^T          (mma.m16n8k16, bf16 -> f32)
//     O[16 heads, D]       += P[16, 16] V[16 keys, D]
// Scores, softmax state and O are float.  The warps' results are merged in
// shared memory; with more than one split the CTA leaves (max, sum, O) per head
// in scratch memory for the merge kernel, otherwise it writes the output.
//
// This kernel is bound by HBM bandwidth; the tensor work is negligible, which
// is why the legacy warp-level mma is enough here (one CTA cannot feed a
// 128-row tcgen05 tile from a 6-row problem anyway).
#include "attention_decode_body.cuh"

namespace fd {

template <int D, int W, bool TR>
__global__ void __launch_bounds__(W * 32)
attn_decode_mma_kernel(const AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem[];
    attn_decode_item<D, W, TR>(p, blockIdx.x, blockIdx.y, blockIdx.z, smem, threadIdx.x);
}

template <int D, int W, bool TR>
static int launch_dm(const AttnParams& p, int n_rows, cudaStream_t stream) {
    constexpr size_t smem = dm_smem_bytes<D, W>();
    static_assert(DM_STAGES * 2 * DM_TILE * D * 2 >= 16 * D * 4, "a warp's staging area must hold its float O tile");
    auto k = attn_decode_mma_kernel<D, W, TR>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(-3, "attention: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(p.n_splits, p.n_kv, n_rows);
    return launch("attention_decode_mma", k, grid, dim3(W * 32), smem, stream, dim3(1, 1, 1), p);
}

int g_dm_form = 0;       // tests and measurements: 0 = the launcher chooses; bit 0: heads as rows even for small groups;
                         // bit 1: four warps per CTA always; bit 2: eight warps per CTA always

template <int D>
static int launch_dm_d(const AttnParams& p, int n_rows, cudaStream_t stream) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    // Few (sequence, KV head) pairs and therefore many splits: CTAs of eight warps, one per SM, so that twice as
    // much of a sequence's merge happens in shared memory and the last CTA has half as many splits to add up.
    bool wide = p.n_splits >= 4 && (long long)p.n_splits * p.n_kv * n_rows <= sms;
    if (g_dm_form & 2) wide = false;
    if (g_dm_form & 4) wide = true;
    const bool tr = p.G <= 8 && !(g_dm_form & 1);
    if (wide) return tr ? launch_dm<D, 8, true>(p, n_rows, stream) : launch_dm<D, 8, false>(p, n_rows, stream);
    return tr ? launch_dm<D, 4, true>(p, n_rows, stream) : launch_dm<D, 4, false>(p, n_rows, stream);
}

int launch_attn_decode_mma(const AttnParams& p, int n_rows, cudaStream_t stream) {
    if (p.G > 16) return 1;
    // the in-kernel merge keeps G * n_splits weights in the 64 KB (32 KB at D = 64) staging area
    if (p.counters != nullptr && (size_t)p.G * p.n_splits * sizeof(float) > 16 * 1024) return 1;
    if (p.d == 128) return launch_dm_d<128>(p, n_rows, stream);
    if (p.d == 64) return launch_dm_d<64>(p, n_rows, stream);
    return 1;
}

}  // namespace fd

// Which form the tensor-core decode attention takes from now on (tests and measurements): 0 = the launcher
// chooses; bit 0 set: the heads as the rows of the MMAs even for groups of up to 8; bit 1: CTAs of four
// warps always; bit 2: CTAs of eight warps always.
extern "C" int fd_attn_decode_set_form(int form) {
    fd::g_dm_form = form;
    return 0;
}
