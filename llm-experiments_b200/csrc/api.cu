// Library-level entry points: status text, CUDA error record, tuning knobs.
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "b2kv_common.cuh"

namespace b2kv {

static thread_local char g_last_error[256] = "no error";

int note_cuda_error(cudaError_t e, const char* where) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e), where);
    cudaGetLastError();  // clear the sticky-free error so that the next call starts clean
    return B2KV_ERR_CUDA;
}

struct Knob {
    const char* name;
    int value;
};

static Knob g_knobs[] = {
    {"decode_variant", 0},      // which compiled (tile, stages, warps) variant of the split kernel
    {"decode_grid_per_sm", 0},  // resident CTAs per SM to launch; 0 = occupancy
    {"decode_no_tensor_map", 0},  // 1 = row-strided caches use one bulk copy per row instead of tiled TMA loads
    {"decode_merge_kernel", 0},  // 1 = the partials of the plain decode are merged by a second launch, not in the split kernel
    {"decode_l2_keep", 0},  // 1 = K/V bulk copies use the default L2 policy instead of evict-first
    {"prefill_force_simt", 0},  // 1 = never take the tensor-core prefill kernel
    {"prefill_variant", 0},
    {"prefill_f32_simt", 0},  // 1 = fp32 prompts never take the split-bfloat16 tensor-core kernel
    {"prefill_unfused_paged", 0},  // 1 = a paged cache is always filled by the copy kernel behind the attention
    {"prefill_test_expire", 0},  // test hook: 1 = the softmax warps of the one-CTA tensor-core prefill give up at once
    {"prefill_group", 0},  // one-CTA tensor-core prefill: (sequence, head) pairs per launch group; 0 = by size, -1 = all
    {"matmul_splits", 0},  // ranges of input features per tile in b2kv_matmul_rows (0 = by shape)
    {"decode_dynamic_chunks", 0},  // small chunks of the decode's token space handed out on demand: 0 = by size, 1 = always, 2 = never
    {"serial_launches", 0},  // 1 = no kernel is launched ahead of the end of the kernel before it (plain stream order)
    {"gemm_variant", 0},   // b2kv_matmul: 0 = by shape and device, 1 = one CTA per tile, 2 / 3 = CTA pairs, 64 / 128 features per stage
};

int tune_get(const char* name) {
    for (auto& k : g_knobs)
        if (strcmp(k.name, name) == 0) return k.value;
    return 0;
}

int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace b2kv

extern "C" {

const char* b2kv_strerror(int status) {
    switch (status) {
        case B2KV_OK: return "ok";
        case B2KV_ERR_BAD_ARG: return "bad argument (null pointer, non-positive dimension or inconsistent sizes)";
        case B2KV_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
        case B2KV_ERR_UNSUPPORTED: return "unsupported head_dim / dtype / block_size combination";
        case B2KV_ERR_WORKSPACE: return "workspace missing or too small";
        case B2KV_ERR_CUDA: return "CUDA runtime error (see b2kv_last_cuda_error)";
        case B2KV_ERR_STATIC_LIMIT:
            return "b2kv_decode_static: this shape needs more scratch than the built-in array holds "
                   "(B2KV_STATIC_SCRATCH_BYTES); call b2kv_decode with a workspace instead";
        default: return "unknown status";
    }
}

const char* b2kv_last_cuda_error(void) { return b2kv::g_last_error; }

int b2kv_version(void) { return 2; }

int b2kv_tune(const char* name, int value) {
    if (name == nullptr) return B2KV_ERR_BAD_ARG;
    for (auto& k : b2kv::g_knobs) {
        if (strcmp(k.name, name) == 0) {
            k.value = value;
            return B2KV_OK;
        }
    }
    return B2KV_ERR_BAD_ARG;
}

}  // extern "C"
