// Q / K / V projection of one decode step fused with the KV-cache append (bf16, fp32 accumulate).
//
// The reference runs three matmul dispatches per layer (simple-llm/src/wgpu_backend.py:812-831,
// src/gpu/gpu_pass_forward.py:35-82: C = A @ B, A = the normalised hidden state [rows, E], B = a weight
// matrix [E, E]) and would then copy the new K / V rows into the cache with kv_cache_update
// (src/gpu/gpu_kv_cache.py:113-186).  At decode time A has one row per sequence, so the work is a
// stream over 3 * E * E weights (HBM-bound: 6 bytes of weights per output feature and input feature)
// with a few FLOPs per byte that only the tensor cores can keep up with.  Here:
//
//   * the product is computed transposed, D[feature, sequence] = W^T x^T, so that the 128 rows of an MMA
//     are output features (plentiful) and its columns are the sequences (few): one CTA per 128 output
//     features of Wq | Wk | Wv.  A = a [64 k x 128 features] tile of W, which is an MN-major operand
//     exactly as the weight matrix lies in memory; B = x, K-major;
//   * warp 4 streams the W and x tiles with TMA (128-byte swizzle) through a ring of stages, warp 5
//     issues tcgen05.mma (M = 128, N = padded batch, K = 16) into one accumulator in tensor memory,
//     warps 0-3 are the epilogue: thread = output feature = TMEM lane, it reads the sequences' values,
//     rounds them to bf16 and writes Q to its buffer and K / V straight into cache row seq_pos[b] of every
//     sequence (consecutive lanes write consecutive head_dim elements), so the new K / V never
//     make a round trip through HBM;
//   * every wait is bounded; a position outside the cache is skipped and recorded in the status word.
#include "b2kv_common.cuh"
#include "tc_ptx.cuh"
#include "tma_map.cuh"

namespace b2kv {

namespace proj {

using namespace tc;

constexpr int kFeat = 128;      // output features per CTA (MMA M)
constexpr int kKTile = 64;      // input features per stage (one 128-byte swizzle span of x)
constexpr int kStagesP = 6;
constexpr int kWBytes = kKTile * kFeat * 2;  // 2 feature halves x 64 k x 128 B
constexpr int kWHalf = kKTile * 128;
constexpr int kMaxBatch = 128;
constexpr int kProjThreads = 192;

struct ProjShared {
    alignas(1024) uint8_t w[kStagesP][kWBytes];
    alignas(1024) uint8_t x[kStagesP][kMaxBatch * 128];
    alignas(8) uint64_t full[kStagesP], empty[kStagesP];
    uint64_t done;
    uint32_t tmem_base;
};

struct ProjParams {
    void* q_out;
    void* k_cache;
    void* v_cache;
    const int32_t* seq_pos;
    int32_t* dev_status;
    int64_t stride_b, stride_t, stride_h;
    int pos, B, Bn, E, H, D, T_max;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Instruction descriptor: fp32 accumulate, bf16 operands, A MN-major, B K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t proj_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((static_cast<uint32_t>(n) >> 3) << 17) | ((128u >> 4) << 24);
}

__global__ void __launch_bounds__(kProjThreads, 1)
qkv_append_kernel(const __grid_constant__ CUtensorMap tm_wq, const __grid_constant__ CUtensorMap tm_wk,
                  const __grid_constant__ CUtensorMap tm_wv, const __grid_constant__ CUtensorMap tm_x, const ProjParams p) {
    extern __shared__ uint8_t smem_raw[];
    ProjShared& sm = *reinterpret_cast<ProjShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * kFeat;  // first output feature, in the concatenation Wq | Wk | Wv
    const int which = f0 / p.E;         // 0 = Q, 1 = K, 2 = V
    const int c0 = f0 % p.E;            // first column inside that weight matrix
    const int n_k = p.E / kKTile;
    const uint32_t stage_bytes = kWBytes + static_cast<uint32_t>(p.Bn) * 128u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesP; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.done, 1);
        fence_mbar_init();
    }
    if (warp == 5) {
        tmem_alloc(&sm.tmem_base, kMaxBatch);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 4) {
        if (lane == 0) {
            const CUtensorMap* tw = which == 0 ? &tm_wq : (which == 1 ? &tm_wk : &tm_wv);
            for (int i = 0; i < n_k; ++i) {
                const int st = i % kStagesP;
                if (!mbar_wait(&sm.empty[st], ((i / kStagesP) & 1) ^ 1)) break;
                mbar_arrive_expect_tx(&sm.full[st], stage_bytes);
                // W tile: input features i*64 .. +63 (rows), output features c0 .. c0+127 (two 64-wide boxes)
                tma_load_2d(sm.w[st], tw, &sm.full[st], c0, i * kKTile);
                tma_load_2d(sm.w[st] + kWHalf, tw, &sm.full[st], c0 + 64, i * kKTile);
                // x tile: every sequence (rows past B read as zero), input features i*64 .. +63
                tma_load_2d(sm.x[st], &tm_x, &sm.full[st], i * kKTile, 0);
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        if (lane == 0) {
            const uint32_t idesc = proj_idesc(p.Bn);
            bool ok = true;
            for (int i = 0; i < n_k && ok; ++i) {
                const int st = i % kStagesP;
                ok = mbar_wait(&sm.full[st], (i / kStagesP) & 1);
                if (!ok) break;
                tc_fence_after();
                // A: [half][64 k][64 features] MN-major (halves 8 KB apart, 8 k-rows = 1024 B, 16 k = 2048 B)
                const uint64_t da = smem_desc(smem_u32(sm.w[st]), kWHalf, 1024);
                // B: [sequence][64 k] K-major (16 k = 32 B inside the swizzle span)
                const uint64_t db = smem_desc(smem_u32(sm.x[st]), 16, 1024);
#pragma unroll
                for (int kk = 0; kk < kKTile / 16; ++kk)
                    mma_ss(tmem, da + static_cast<uint64_t>((kk * 2048) >> 4), db + static_cast<uint64_t>((kk * 32) >> 4), idesc,
                           (i | kk) ? 1u : 0u);
                mma_commit(&sm.empty[st]);
            }
            if (ok) mma_commit(&sm.done);
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue: thread = output feature ------------------------------
        const int m = threadIdx.x;  // 0..127, also the TMEM lane
        const uint32_t t_lane = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        if (mbar_wait(&sm.done, 0)) {
            tc_fence_after();
            const int col = c0 + m;  // column inside the weight matrix = element of the output row
            const int h = col / p.D, d = col % p.D;
            __nv_bfloat16* q = static_cast<__nv_bfloat16*>(p.q_out);
            __nv_bfloat16* cache = static_cast<__nv_bfloat16*>(which == 1 ? p.k_cache : p.v_cache);
            for (int nb = 0; nb < p.Bn; nb += 16) {
                uint32_t v[16];
                tmem_ld16(t_lane + nb, v);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int b = nb + j;
                    if (b >= p.B) break;
                    const __nv_bfloat16 val = __float2bfloat16_rn(__uint_as_float(v[j]));
                    if (which == 0) {
                        q[static_cast<size_t>(b) * p.E + col] = val;
                    } else {
                        const int pos = p.seq_pos ? p.seq_pos[b] : p.pos;
                        if (pos < 0 || pos >= p.T_max) {
                            report_status(p.dev_status, B2KV_DEV_BAD_POSITION);
                        } else {
                            cache[static_cast<size_t>(b) * p.stride_b + static_cast<size_t>(pos) * p.stride_t +
                                  static_cast<size_t>(h) * p.stride_h + d] = val;
                        }
                    }
                }
            }
        } else {
            report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, kMaxBatch);
    }
}

// [rows, cols] bf16 row-major matrix, boxes of box_rows x 64 columns, 128-byte swizzle.
static bool make_matrix_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace proj

}  // namespace b2kv

using namespace b2kv;

extern "C" int b2kv_qkv_append(const void* x, const void* wq, const void* wk, const void* wv, void* q_out, void* k_cache,
                               void* v_cache, const int32_t* seq_pos, int pos, int B, int E, int H, int D, int T_max,
                               int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype, int32_t* dev_status,
                               void* stream) {
    if (dtype != B2KV_DTYPE_BF16) return B2KV_ERR_UNSUPPORTED;
    if (!x || !wq || !wk || !wv || !q_out || !k_cache || !v_cache) return B2KV_ERR_BAD_ARG;
    if (B <= 0 || E <= 0 || H <= 0 || D <= 0 || T_max <= 0 || H * D != E) return B2KV_ERR_BAD_ARG;
    if (seq_pos == nullptr && (pos < 0 || pos >= T_max)) return B2KV_ERR_BAD_ARG;
    if (B > proj::kMaxBatch || E % proj::kFeat != 0) return B2KV_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(wq) || !aligned16(wk) || !aligned16(wv) || !aligned16(q_out) || !aligned16(k_cache) ||
        !aligned16(v_cache))
        return B2KV_ERR_ALIGN;
    if (stride_b < 0 || stride_t < 0 || stride_h < 0) return B2KV_ERR_BAD_ARG;
    const int Bn = ((B + 15) / 16) * 16;  // MMA N: a multiple of 16
    CUtensorMap tq, tk, tv, tx;
    if (!proj::make_matrix_map(&tq, wq, E, E, proj::kKTile) || !proj::make_matrix_map(&tk, wk, E, E, proj::kKTile) ||
        !proj::make_matrix_map(&tv, wv, E, E, proj::kKTile) || !proj::make_matrix_map(&tx, x, B, E, Bn))
        return B2KV_ERR_UNSUPPORTED;
    proj::ProjParams p{q_out, k_cache, v_cache, seq_pos, dev_status, stride_b, stride_t, stride_h, pos, B, Bn, E, H, D, T_max};
    constexpr size_t smem = sizeof(proj::ProjShared) + 1024;
    static bool configured[64] = {false};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(proj::qkv_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)));
        configured[dev] = true;
    }
    proj::qkv_append_kernel<<<3 * E / proj::kFeat, proj::kProjThreads, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv,
                                                                                                                   tx, p);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}
