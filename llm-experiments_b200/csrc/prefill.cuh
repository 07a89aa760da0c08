// Arguments shared by the two prefill kernels (SIMT and tensor core).
#pragma once

#include "b2kv_common.cuh"

namespace b2kv {

struct PrefillParams {
    const void* Q;
    const void* K;
    const void* V;
    void* O;
    float* L;
    float* M;
    void* k_cache;
    void* v_cache;
    int64_t stride_b, stride_t, stride_h;
    int B, N, H;
    float q_prescale;
    // paged cache (tensor-core kernel): k_cache / v_cache are block pools and the prompt's rows go through the table
    const int32_t* block_table;  // [B, max_blocks], null for a contiguous cache
    int max_blocks, block_size, n_blocks;
    int rows_per_store;  // rows of one TMA store into a pool block: min(block_size, 128)
    int n_whole;         // tokens covered by whole blocks (N rounded down to a multiple of block_size)
    int32_t* dev_status;  // optional status word: receives B2KV_DEV_WAIT_TIMEOUT when a bounded wait ran out
    int test_expire;      // test hook: the softmax warps of the one-CTA tensor-core kernel give up before their first wait
    int group;  // tensor-core kernel: (sequence, head) pairs whose row blocks are launched next to each other; 0 = by size, < 0 = all
};

// SIMT kernel: every supported head_dim and storage type.
int prefill_simt(const PrefillParams& p, int D, int dtype, void* stream);
// Tensor-core kernel: returns B2KV_ERR_UNSUPPORTED when the shape is not one it takes.
int prefill_tensor_core(const PrefillParams& p, int D, int dtype, void* stream);
// Tensor-core kernel for fp32 prompts (head_dim 128 or 64): operands split into bfloat16 halves in `scratch`
// (prefill_f32_scratch_bytes), three MMAs per product.  Writes no cache rows.  B2KV_ERR_UNSUPPORTED when the shape or
// the scratch does not fit.
size_t prefill_f32_scratch_bytes(int B, int N, int H, int D);
int prefill_tensor_core_f32(const PrefillParams& p, int D, void* scratch, size_t scratch_bytes, void* stream);
// Tensor-core kernel on CTA pairs (bf16, head_dim 128, N a multiple of 256): same contract.
int prefill_tensor_core_pair(const PrefillParams& p, int D, int dtype, void* stream);

}  // namespace b2kv
