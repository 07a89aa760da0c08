// Shared device helpers of the b2kv kernels: storage-type traits, mbarrier and bulk-copy
// (TMA) PTX wrappers with bounded waits, host-side argument checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b2kv.h"

namespace b2kv {

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------

// Records a CUDA error for b2kv_last_cuda_error and returns B2KV_ERR_CUDA.
int note_cuda_error(cudaError_t e, const char* where);

#define B2KV_CUDA_TRY(expr)                                             \
    do {                                                                \
        cudaError_t e__ = (expr);                                       \
        if (e__ != cudaSuccess) return ::b2kv::note_cuda_error(e__, #expr); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int elt_bytes(int dtype) { return dtype == B2KV_DTYPE_F32 ? 4 : (dtype == B2KV_DTYPE_BF16 ? 2 : 0); }
inline bool stride_ok(int64_t s, int es) { return s >= 0 && ((s * es) & 15) == 0; }

int tune_get(const char* name);
int device_sm_count();

// Launch configuration of a kernel that takes part in programmatic dependent launch: the grid may be
// scheduled while the kernel before it in the stream is still running, as soon as every CTA of that
// kernel has executed grid_launch_dependents() (or has exited); nothing of what the earlier kernels wrote
// may be read, and nothing written, before grid_dependency_wait() returns.  A kernel launched this way
// must execute grid_dependency_wait() on every path, or kernels after it could overtake kernels before it.
// The knob "serial_launches" != 0 leaves the attribute out (plain stream order).
struct OverlapLaunch {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    OverlapLaunch(dim3 grid, dim3 block, size_t smem, void* stream, unsigned cluster_x = 1) : cfg{}, attr{} {
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = static_cast<cudaStream_t>(stream);
        cfg.attrs = attr;
        if (cluster_x > 1) {
            attr[cfg.numAttrs].id = cudaLaunchAttributeClusterDimension;
            attr[cfg.numAttrs].val.clusterDim.x = cluster_x;
            attr[cfg.numAttrs].val.clusterDim.y = 1;
            attr[cfg.numAttrs].val.clusterDim.z = 1;
            ++cfg.numAttrs;
        }
        if (tune_get("serial_launches") == 0) {
            attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
            ++cfg.numAttrs;
        }
    }
};

// ---------------------------------------------------------------------------------------
// storage types: 16-byte chunks widened to float
// ---------------------------------------------------------------------------------------

template <typename T>
struct Elt;

template <>
struct Elt<float> {
    static constexpr int kPerChunk = 4;  // elements per 16 bytes
    __device__ static __forceinline__ void widen(const uint4& c, float* f) {
        f[0] = __uint_as_float(c.x);
        f[1] = __uint_as_float(c.y);
        f[2] = __uint_as_float(c.z);
        f[3] = __uint_as_float(c.w);
    }
    __device__ static __forceinline__ float to_float(float x) { return x; }
    __device__ static __forceinline__ float from_float(float x) { return x; }
};

template <>
struct Elt<__nv_bfloat16> {
    static constexpr int kPerChunk = 8;
    // bf16 -> fp32 is a 16-bit shift; the low half of each word is the even element.
    __device__ static __forceinline__ void widen(const uint4& c, float* f) {
        f[0] = __uint_as_float(c.x << 16);
        f[1] = __uint_as_float(c.x & 0xffff0000u);
        f[2] = __uint_as_float(c.y << 16);
        f[3] = __uint_as_float(c.y & 0xffff0000u);
        f[4] = __uint_as_float(c.z << 16);
        f[5] = __uint_as_float(c.z & 0xffff0000u);
        f[6] = __uint_as_float(c.w << 16);
        f[7] = __uint_as_float(c.w & 0xffff0000u);
    }
    __device__ static __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    __device__ static __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

// ---------------------------------------------------------------------------------------
// mbarrier + bulk copy (TMA, untiled) wrappers
// ---------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes barrier initialisation visible to the async (copy) proxy.
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after kWaitLimit polls or about kWaitLimitNs of wall time, whichever comes
// first (a poll blocks for a short, hardware-defined time, so the polls alone do not say how long a
// wait may last), and returns false, so that no kernel can spin for ever on a barrier that will not
// complete.
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t it = 0; it < 128; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    for (uint32_t it = 128; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(32);
        if ((it & 255u) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) return false;
    }
    return false;
}

// Global -> shared bulk copy; completion is counted in bytes on `bar`.  Source, destination
// and size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// L2 policy for data that is read once: evict it first.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// bulk_g2s with an L2 cache policy.
__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

template <int kThreads>
__device__ __forceinline__ void named_barrier_sync(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kThreads) : "memory");
}

// Programmatic dependent launch, device side (no-ops in a kernel launched in plain stream order).
// wait: returns when every kernel before this one in the stream has completed and its writes are visible.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// launch_dependents: this CTA no longer holds back the start of the next kernel in the stream.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void report_status(int32_t* dev_status, int code) {
    if (dev_status != nullptr) atomicCAS(dev_status, 0, code);
}

}  // namespace b2kv
