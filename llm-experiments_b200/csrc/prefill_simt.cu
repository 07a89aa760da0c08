// Causal flash-attention prefill, SIMT version: any supported head_dim, fp32 or bf16 storage,
// fp32 arithmetic.  It serves the shapes that the tensor-core kernel does not take (fp32
// data, head_dim other than 128) and is the numerical cross-check of that kernel.
//
// Same tiling idea as the reference kernel (simple-llm/src/gpu/gpu_kernels.py:499-770): a
// CTA owns a block of query rows of one (sequence, head) and walks the K/V blocks up to the
// diagonal with an online softmax.  Differences: 32x32 tiles; each warp owns 8 query rows
// for all three phases (scores, softmax, P.V), so only the K/V tile loads need a CTA-wide
// barrier; the running (m, l) and the output accumulators live in registers; scores are
// kept in the log2 domain.  L and M are written as the reference writes them (:762-768):
// L = sum of exp(s - max), M = max of the scaled scores.
// Optionally copies the K / V rows of the CTA's query block into the cache (bit-exact).
#include <math.h>

#include "b2kv_common.cuh"
#include "prefill.cuh"

namespace b2kv {


constexpr int kBr = 32, kBc = 32, kPrefillThreads = 128, kRowsPerWarpP = 8;

template <typename T, int D>
__global__ void __launch_bounds__(kPrefillThreads) prefill_simt_kernel(const PrefillParams p) {
    constexpr int KS = D + 4;  // padded K row (floats): 16-byte reads of 8 lanes hit distinct banks
    constexpr int DPL = (D + 31) / 32;
    constexpr int EPC = Elt<T>::kPerChunk;
    constexpr int CPR = D / EPC;  // 16-byte chunks per row
    extern __shared__ __align__(16) float smem_f[];
    float* Qs = smem_f;             // [kBr][D]
    float* Ks = Qs + kBr * D;       // [kBc][KS]
    float* Vs = Ks + kBc * KS;      // [kBc][D]
    float* Ss = Vs + kBc * D;       // [kBr][kBc + 1]

    const int nqb = (p.N + kBr - 1) / kBr;
    const int qb = nqb - 1 - blockIdx.x;  // longest rows first
    const int h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int E = p.H * D;
    const int q_start = qb * kBr;
    const int q_end = min(q_start + kBr, p.N);
    const T* Qg = static_cast<const T*>(p.Q) + static_cast<size_t>(b) * p.N * E + static_cast<size_t>(h) * D;
    const T* Kg = static_cast<const T*>(p.K) + static_cast<size_t>(b) * p.N * E + static_cast<size_t>(h) * D;
    const T* Vg = static_cast<const T*>(p.V) + static_cast<size_t>(b) * p.N * E + static_cast<size_t>(h) * D;

    // Q block -> shared, pre-scaled; rows past N are zero
    for (int i = tid; i < kBr * CPR; i += kPrefillThreads) {
        const int r = i / CPR, c = i - r * CPR;
        float f[EPC];
        if (q_start + r < p.N) {
            const uint4 raw = *reinterpret_cast<const uint4*>(Qg + static_cast<size_t>(q_start + r) * E + c * EPC);
            Elt<T>::widen(raw, f);
        } else {
#pragma unroll
            for (int e = 0; e < EPC; ++e) f[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < EPC; ++e) Qs[r * D + c * EPC + e] = f[e] * p.q_prescale;
    }

    float m[kRowsPerWarpP], l[kRowsPerWarpP], acc[kRowsPerWarpP][DPL];
#pragma unroll
    for (int i = 0; i < kRowsPerWarpP; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int k = 0; k < DPL; ++k) acc[i][k] = 0.f;
    }
    const int r0 = warp * kRowsPerWarpP;  // this warp's rows inside the block

    const int n_kv = (q_end - 1) / kBc + 1;  // K/V blocks that hold a visible key
    for (int jb = 0; jb < n_kv; ++jb) {
        const int kv_start = jb * kBc;
        __syncthreads();  // previous tile fully used (and Q stored, first time round)
        for (int i = tid; i < kBc * CPR; i += kPrefillThreads) {
            const int r = i / CPR, c = i - r * CPR;
            float kf[EPC], vf[EPC];
            if (kv_start + r < p.N) {
                const size_t off = static_cast<size_t>(kv_start + r) * E + c * EPC;
                Elt<T>::widen(*reinterpret_cast<const uint4*>(Kg + off), kf);
                Elt<T>::widen(*reinterpret_cast<const uint4*>(Vg + off), vf);
            } else {
#pragma unroll
                for (int e = 0; e < EPC; ++e) kf[e] = vf[e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < EPC; ++e) {
                Ks[r * KS + c * EPC + e] = kf[e];
                Vs[r * D + c * EPC + e] = vf[e];
            }
        }
        __syncthreads();

        // scores: lane = key column, 8 query rows of this warp
        float s[kRowsPerWarpP];
#pragma unroll
        for (int i = 0; i < kRowsPerWarpP; ++i) s[i] = 0.f;
        for (int d = 0; d < D; d += 4) {
            const float4 kk = *reinterpret_cast<const float4*>(&Ks[lane * KS + d]);
#pragma unroll
            for (int i = 0; i < kRowsPerWarpP; ++i) {
                const float4 qq = *reinterpret_cast<const float4*>(&Qs[(r0 + i) * D + d]);
                s[i] = fmaf(qq.x, kk.x, s[i]);
                s[i] = fmaf(qq.y, kk.y, s[i]);
                s[i] = fmaf(qq.z, kk.z, s[i]);
                s[i] = fmaf(qq.w, kk.w, s[i]);
            }
        }
        // online softmax per row; P goes to shared for the P.V phase
        const int key = kv_start + lane;
#pragma unroll
        for (int i = 0; i < kRowsPerWarpP; ++i) {
            const int row = q_start + r0 + i;
            const bool visible = (key <= row) && (key < p.N);
            float sv = visible ? s[i] : -INFINITY;
            float mx = sv;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m[i], mx);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float pr = exp2f(sv - m_use);
            float sum = pr;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            const float corr = exp2f(m[i] - m_use);
            l[i] = l[i] * corr + sum;
            m[i] = m_new;
#pragma unroll
            for (int k = 0; k < DPL; ++k) acc[i][k] *= corr;
            Ss[(r0 + i) * (kBc + 1) + lane] = pr;
        }
        __syncwarp();
        // P.V: lane = output column (d = lane + 32k)
        for (int c = 0; c < kBc; ++c) {
            float vv[DPL];
#pragma unroll
            for (int k = 0; k < DPL; ++k) {
                const int d = lane + 32 * k;
                vv[k] = (d < D) ? Vs[c * D + d] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < kRowsPerWarpP; ++i) {
                const float pr = Ss[(r0 + i) * (kBc + 1) + c];
#pragma unroll
                for (int k = 0; k < DPL; ++k) acc[i][k] = fmaf(pr, vv[k], acc[i][k]);
            }
        }
        __syncwarp();
    }

    // epilogue: O = acc / max(l, 1e-8), statistics, optional cache rows
    T* Og = static_cast<T*>(p.O) + static_cast<size_t>(b) * p.N * E + static_cast<size_t>(h) * D;
#pragma unroll
    for (int i = 0; i < kRowsPerWarpP; ++i) {
        const int row = q_start + r0 + i;
        if (row >= p.N) continue;
        const float inv = 1.f / fmaxf(l[i], 1e-8f);
#pragma unroll
        for (int k = 0; k < DPL; ++k) {
            const int d = lane + 32 * k;
            if (d < D) Og[static_cast<size_t>(row) * E + d] = Elt<T>::from_float(acc[i][k] * inv);
        }
        if (lane == 0) {
            const size_t sidx = (static_cast<size_t>(b) * p.N + row) * p.H + h;
            if (p.L) p.L[sidx] = l[i];
            if (p.M) p.M[sidx] = m[i] * 0.6931471805599453f;  // back from the log2 domain
        }
    }
    if (p.k_cache != nullptr) {
        T* kc = static_cast<T*>(p.k_cache);
        T* vc = static_cast<T*>(p.v_cache);
        for (int i = tid; i < (q_end - q_start) * CPR; i += kPrefillThreads) {
            const int r = i / CPR, c = i - r * CPR;
            const size_t src = static_cast<size_t>(q_start + r) * E + c * EPC;
            const int64_t dst = static_cast<int64_t>(b) * p.stride_b + static_cast<int64_t>(q_start + r) * p.stride_t +
                                static_cast<int64_t>(h) * p.stride_h + c * EPC;
            *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(Kg + src);
            *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(Vg + src);
        }
    }
}

template <typename T, int D>
static int launch_prefill_simt(const PrefillParams& p, void* stream) {
    constexpr size_t smem = (static_cast<size_t>(kBr) * D + kBc * (D + 4) + kBc * D + kBr * (kBc + 1)) * sizeof(float);
    auto kernel = prefill_simt_kernel<T, D>;
    static bool configured[64] = {false};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured[dev] = true;
    }
    if (p.H > 65535 || p.B > 65535) return B2KV_ERR_UNSUPPORTED;
    dim3 grid((p.N + kBr - 1) / kBr, p.H, p.B);
    kernel<<<grid, kPrefillThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

template <typename T>
static int dispatch_prefill_simt(const PrefillParams& p, int D, void* stream) {
    switch (D) {
        case 16: return launch_prefill_simt<T, 16>(p, stream);
        case 32: return launch_prefill_simt<T, 32>(p, stream);
        case 64: return launch_prefill_simt<T, 64>(p, stream);
        case 128: return launch_prefill_simt<T, 128>(p, stream);
        case 256: return launch_prefill_simt<T, 256>(p, stream);
        default: return B2KV_ERR_UNSUPPORTED;
    }
}

int prefill_simt(const PrefillParams& p, int D, int dtype, void* stream) {
    if (dtype == B2KV_DTYPE_F32) return dispatch_prefill_simt<float>(p, D, stream);
    return dispatch_prefill_simt<__nv_bfloat16>(p, D, stream);
}

}  // namespace b2kv

using namespace b2kv;

extern "C" int b2kv_prefill(const void* Q, const void* K, const void* V, void* O, float* L, float* M, void* k_cache,
                            void* v_cache, int64_t stride_b, int64_t stride_t, int64_t stride_h, int T_max, int B,
                            int N, int H, int D, int dtype, int32_t* dev_status, void* stream) {
    const int es = elt_bytes(dtype);
    if (es == 0) return B2KV_ERR_UNSUPPORTED;
    if (!Q || !K || !V || !O) return B2KV_ERR_BAD_ARG;
    if (B <= 0 || N <= 0 || H <= 0 || D <= 0) return B2KV_ERR_BAD_ARG;
    if ((k_cache == nullptr) != (v_cache == nullptr)) return B2KV_ERR_BAD_ARG;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O) || !aligned16(k_cache) || !aligned16(v_cache))
        return B2KV_ERR_ALIGN;
    if ((D * es) % 16 != 0) return B2KV_ERR_UNSUPPORTED;
    if (k_cache) {
        if (N > T_max) return B2KV_ERR_BAD_ARG;
        if (!stride_ok(stride_b, es) || !stride_ok(stride_t, es) || !stride_ok(stride_h, es)) return B2KV_ERR_ALIGN;
    }
    PrefillParams p{Q, K, V, O, L, M, k_cache, v_cache, stride_b, stride_t, stride_h, B, N, H,
                    static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(D))), nullptr, 0, 0, 0, 0, 0,
                    dev_status, tune_get("prefill_test_expire"), tune_get("prefill_group")};
    if (!tune_get("prefill_force_simt")) {
        // "prefill_variant": 0 = one-CTA tensor-core kernel (default), 2 = CTA-pair kernel where its
        // shape limits allow
        int rc = B2KV_ERR_UNSUPPORTED;
        if (tune_get("prefill_variant") == 2) rc = prefill_tensor_core_pair(p, D, dtype, stream);
        if (rc == B2KV_ERR_UNSUPPORTED) rc = prefill_tensor_core(p, D, dtype, stream);
        if (rc != B2KV_ERR_UNSUPPORTED) return rc;
    }
    return prefill_simt(p, D, dtype, stream);
}

namespace b2kv {
// append.cu: rows [b * src_rows_per_seq + src_first + i], i < n_rows, of k_rows / v_rows to position first_pos + i of
// sequence b through the block table.
int append_rows_paged_from(const void* k_rows, const void* v_rows, void* k_pool, void* v_pool, const int32_t* block_table,
                           int max_blocks, int block_size, int n_blocks, int B, int n_rows, int first_pos,
                           int src_rows_per_seq, int src_first, int H, int D, int64_t stride_blk, int64_t stride_t,
                           int64_t stride_h, int dtype, int32_t* dev_status, void* stream);
}  // namespace b2kv

namespace b2kv {
int append_rows_contiguous(const void* k_rows, const void* v_rows, void* k_cache, void* v_cache, int B, int n_rows, int H,
                           int D, int T_max, int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype,
                           int32_t* dev_status, void* stream);
}  // namespace b2kv

extern "C" size_t b2kv_prefill_workspace_bytes(int B, int N, int H, int D, int dtype) {
    // scratch only buys something for fp32 prompts that the tensor-core kernel takes, and only from a row block on
    if (dtype != B2KV_DTYPE_F32 || B <= 0 || N < 128 || H <= 0) return 0;
    return prefill_f32_scratch_bytes(B, N, H, D);
}

extern "C" int b2kv_prefill_ws(const void* Q, const void* K, const void* V, void* O, float* L, float* M, void* k_cache,
                               void* v_cache, int64_t stride_b, int64_t stride_t, int64_t stride_h, int T_max, int B,
                               int N, int H, int D, int dtype, void* workspace, size_t workspace_bytes,
                               int32_t* dev_status, void* stream) {
    const size_t need = b2kv_prefill_workspace_bytes(B, N, H, D, dtype);
    if (need == 0 || workspace == nullptr || workspace_bytes < need || tune_get("prefill_force_simt") ||
        tune_get("prefill_f32_simt"))
        return b2kv_prefill(Q, K, V, O, L, M, k_cache, v_cache, stride_b, stride_t, stride_h, T_max, B, N, H, D, dtype,
                            dev_status, stream);
    // the same argument checks as b2kv_prefill, then the tensor-core kernel and, for a cache, the copy kernel
    if (!Q || !K || !V || !O) return B2KV_ERR_BAD_ARG;
    if ((k_cache == nullptr) != (v_cache == nullptr)) return B2KV_ERR_BAD_ARG;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O) || !aligned16(k_cache) || !aligned16(v_cache) ||
        !aligned16(workspace))
        return B2KV_ERR_ALIGN;
    if (k_cache) {
        if (N > T_max) return B2KV_ERR_BAD_ARG;
        if (!stride_ok(stride_b, 4) || !stride_ok(stride_t, 4) || !stride_ok(stride_h, 4)) return B2KV_ERR_ALIGN;
    }
    PrefillParams p{Q, K, V, O, L, M, nullptr, nullptr, 0, 0, 0, B, N, H,
                    static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(D))), nullptr, 0, 0, 0, 0, 0,
                    dev_status, 0, tune_get("prefill_group")};
    int rc = prefill_tensor_core_f32(p, D, workspace, workspace_bytes, stream);
    if (rc == B2KV_ERR_UNSUPPORTED)
        return b2kv_prefill(Q, K, V, O, L, M, k_cache, v_cache, stride_b, stride_t, stride_h, T_max, B, N, H, D, dtype,
                            dev_status, stream);
    if (rc != B2KV_OK || k_cache == nullptr) return rc;
    return append_rows_contiguous(K, V, k_cache, v_cache, B, N, H, D, T_max, stride_b, stride_t, stride_h, dtype,
                                  dev_status, stream);
}

extern "C" int b2kv_prefill_paged(const void* Q, const void* K, const void* V, void* O, float* L, float* M, void* k_pool,
                                  void* v_pool, const int32_t* block_table, int max_blocks, int block_size, int n_blocks,
                                  int64_t stride_blk, int64_t stride_t, int64_t stride_h, int B, int N, int H, int D,
                                  int dtype, int32_t* dev_status, void* stream) {
    const int es = elt_bytes(dtype);
    if (es == 0) return B2KV_ERR_UNSUPPORTED;
    if (!Q || !K || !V || !O || !k_pool || !v_pool || !block_table) return B2KV_ERR_BAD_ARG;
    if (B <= 0 || N <= 0 || H <= 0 || D <= 0 || max_blocks <= 0 || block_size <= 0 || n_blocks <= 0) return B2KV_ERR_BAD_ARG;
    if (static_cast<long long>(max_blocks) * block_size < N) return B2KV_ERR_BAD_ARG;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O) || !aligned16(k_pool) || !aligned16(v_pool))
        return B2KV_ERR_ALIGN;
    if ((D * es) % 16 != 0) return B2KV_ERR_UNSUPPORTED;
    if (!stride_ok(stride_blk, es) || !stride_ok(stride_t, es) || !stride_ok(stride_h, es)) return B2KV_ERR_ALIGN;
    PrefillParams p{Q, K, V, O, L, M, nullptr, nullptr, stride_blk, stride_t, stride_h, B, N, H,
                    static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(D))), nullptr, 0, 0, 0, 0, 0,
                    dev_status, tune_get("prefill_test_expire"), tune_get("prefill_group")};
    // The tensor-core kernel stores the whole blocks of the prompt itself, straight from its K / V rings, when a
    // block is a whole number of 1 KB swizzle atoms (8 rows) and blocks tile its 128-row K / V tiles.
    const bool tiles = block_size % 8 == 0 && (128 % block_size == 0 || block_size % 128 == 0);
    int whole = 0;  // tokens that the attention kernel has written
    if (!tune_get("prefill_force_simt") && !tune_get("prefill_unfused_paged") && tiles) {
        PrefillParams pp = p;
        pp.k_cache = k_pool;
        pp.v_cache = v_pool;
        pp.block_table = block_table;
        pp.max_blocks = max_blocks;
        pp.block_size = block_size;
        pp.n_blocks = n_blocks;
        pp.rows_per_store = block_size < 128 ? block_size : 128;
        pp.n_whole = N / block_size * block_size;
        const int rc = prefill_tensor_core(pp, D, dtype, stream);
        if (rc == B2KV_OK) whole = pp.n_whole;
        else if (rc != B2KV_ERR_UNSUPPORTED) return rc;
    }
    if (whole == 0) {
        int rc = B2KV_ERR_UNSUPPORTED;
        if (!tune_get("prefill_force_simt")) rc = prefill_tensor_core(p, D, dtype, stream);
        if (rc == B2KV_ERR_UNSUPPORTED) rc = prefill_simt(p, D, dtype, stream);
        if (rc != B2KV_OK) return rc;
    }
    if (whole == N) return B2KV_OK;
    // what the attention kernel did not write (a last, partly filled block; or everything): a copy kernel behind it
    return append_rows_paged_from(K, V, k_pool, v_pool, block_table, max_blocks, block_size, n_blocks, B, N - whole, whole,
                                  N, whole, H, D, stride_blk, stride_t, stride_h, dtype, dev_status, stream);
}
