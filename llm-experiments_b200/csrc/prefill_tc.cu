// Causal flash-attention prefill on the tcgen05 tensor cores (bf16, head_dim 128).
#include "prefill.cuh"

namespace b2kv {

int prefill_tensor_core(const PrefillParams& p, int D, int dtype, void* stream) {
    (void)p;
    (void)D;
    (void)dtype;
    (void)stream;
    return B2KV_ERR_UNSUPPORTED;
}

}  // namespace b2kv
