// Parameters shared by the attention kernels (CUDA-core and tensor-core forms).
#pragma once

#include "common.cuh"

namespace fd {

struct AttnParams {
    const void* q;             // [T, n_q * d]
    const void* k_pool;        // [num_blocks, n_kv, block_size, d]
    const void* v_pool;
    void* out;                 // [T, n_q * d]
    float* part_m;             // [T, n_q, n_splits]
    float* part_l;
    float* part_acc;           // [T, n_q, n_splits, d]
    const int* block_table;    // [slots, max_blocks]
    const int* row_slot;       // per batch row: cache slot, or -1 for a padding row
    const int* row_q_start;    // first token of the row in the flat token arrays
    const int* row_q_len;      // new tokens of the row in this step
    const int* row_ctx_len;    // tokens of the row cached before this step
    int* status;
    int* counters;             // [rows, n_kv] arrival counts for the in-kernel merge of the splits (all zero between launches), or null
    int max_blocks, num_blocks, block_size;
    int n_q, n_kv, G, d;
    int QT, n_splits, split_len, window;
    float scale;
    // decode steps on the tensor cores only: memory that a later kernel streams (the next part's first weights), or
    // null; every CTA asks L2 for its share once its own keys and values are through
    const unsigned char* pf_ptr;
    unsigned long long pf_bytes;
};

// decode steps (one new token per row) on the tensor cores; returns 1 if it
// does not take the sizes (the caller then uses the CUDA-core kernel)
int launch_attn_decode_mma(const AttnParams& p, int n_rows, cudaStream_t stream);
// prompt steps (several new tokens per row) on the tensor cores; same return convention
int launch_attn_prefill_mma(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream);
// the same on the tcgen05 tensor cores (head size 128, block sizes 8..128 that divide 128)
int launch_attn_prefill_tcgen05(const AttnParams& p, int n_rows, int T, int max_q_len, cudaStream_t stream);

}  // namespace fd
