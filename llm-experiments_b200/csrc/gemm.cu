// matmul for many rows on the Blackwell tensor cores: out = act(A @ W + bias) + residual, bf16 operands,
// fp32 accumulation.  This is the reference's matmul dispatch (simple-llm/src/gpu/gpu_pass_forward.py:35-82,
// C = A @ B, kernel src/gpu/gpu_kernels.py:10-134: 16x16 workgroup tiles, scalar fp32 FMAs) for the
// prompt-side projections either side of flash_attention (call sites src/wgpu_backend.py:812-930: Q / K / V,
// the output projection, the MLP), with the bias_add, gelu and residual_add dispatches that follow a
// matmul there folded into the epilogue.  Decode-step shapes (at most 128 rows) go to the weight-streaming
// kernel in qkv_append.cu instead.
//
//   * persistent grid, one CTA per SM; a CTA walks output tiles of 128 rows x 256 columns.  Tiles are
//     ordered in blocks of 8 row tiles x 16 column tiles (about one wave of CTAs), so that the CTAs running
//     together share a few row tiles of A and 4096 columns of W out of L2;
//   * warp 0 streams A (128 rows x 64 input features, K-major) and W (64 input features x 256 columns, the
//     matrix as it lies in memory = an MN-major operand, four 64-column boxes) with TMA tiled loads, 128-byte
//     swizzle, into a 4-stage ring of 48 KB stages that complete on mbarriers;
//   * warp 1 issues tcgen05.mma (M = 128, N = 256, K = 16; four per stage) from one thread into one of two
//     256-column fp32 accumulators in tensor memory, so that the epilogue of a tile runs under the MMAs of
//     the next;
//   * warps 2-5 are the epilogue: thread = output row = TMEM lane, 32 columns at a time: bias, GELU,
//     residual, round to bf16, 16-byte stores.
//
// Operand bytes per MMA are 4 KB of A + 8 KB of W per 128 clocks, 96 B/clk of the SM's 128 B/clk shared-memory
// port.  Rows, columns and input features past the matrix edges are zero-filled by the tensor maps and masked
// in the epilogue.  Every mbarrier wait is bounded; a wait that runs out makes all warps leave through the
// common exit, where the tensor memory is released.
#include <algorithm>

#include "tc_ptx.cuh"
#include "tma_map.cuh"

namespace b2kv {

namespace gemm {

using namespace tc;

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;             // 16 KB: 128 rows x 128 bytes
constexpr int kWSpanBytes = kBK * 128;             // 8 KB: 64 input features x 64 columns
constexpr int kWBytes = (kBN / 64) * kWSpanBytes;  // 32 KB
constexpr int kStageBytes = kABytes + kWBytes;
constexpr int kThreads = 192;  // warp 0 producer, warp 1 MMA issuer, warps 2-5 epilogue
constexpr int kTmemCols = 512;  // two accumulators of 256 columns
constexpr int kBandRows = 8;    // row tiles and
constexpr int kBandCols = 16;   // column tiles per block of the tile order (128 tiles: about one wave of CTAs)

struct GemmParams {
    const __nv_bfloat16* bias;      // [N] or null
    const __nv_bfloat16* residual;  // [M, N] or null
    __nv_bfloat16* out;             // [M, N]
    int M, N, K;
    int gelu;
    int tiles_m, tiles_n;
};

struct SharedStorage {
    alignas(1024) uint8_t stage[kStages][kStageBytes];
    alignas(8) uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    volatile int abort_flag;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Tile t of the order described above -> (row tile, column tile): column bands outermost, then row bands,
// then the tiles of a block with the row tile running fastest.
__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& tm, int& tn) {
    const int cband_tiles = p.tiles_m * kBandCols;
    const int cband = t / cband_tiles;  // only the last column band can be narrower, and nothing follows it
    const int first_col = cband * kBandCols;
    const int cols_here = min(kBandCols, p.tiles_n - first_col);
    const int in_cband = t - cband * cband_tiles;
    const int block_tiles = kBandRows * cols_here;
    const int rband = in_cband / block_tiles;
    const int first_row = rband * kBandRows;
    const int rows_here = min(kBandRows, p.tiles_m - first_row);
    const int within = in_cband - rband * block_tiles;
    tm = first_row + within % rows_here;
    tn = first_col + within / rows_here;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    SharedStorage& sm = *reinterpret_cast<SharedStorage*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = p.tiles_m * p.tiles_n;
    const int n_k = (p.K + kBK - 1) / kBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sm.acc_full[a], 1);
            mbar_init(&sm.acc_empty[a], 4);  // one arrival per epilogue warp
        }
        sm.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&sm.tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            bool ok = true;
            uint32_t it = 0;  // stages filled so far: stage it % kStages, phase it / kStages
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(t, p, tm, tn);
                for (int kb = 0; kb < n_k; ++kb, ++it) {
                    const int s = it % kStages;
                    ok = mbar_wait(&sm.empty[s], ((it / kStages) & 1) ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&sm.full[s], kStageBytes);
                    tma_load_2d(sm.stage[s], &tm_a, &sm.full[s], kb * kBK, tm * kBM);
#pragma unroll
                    for (int sp = 0; sp < kBN / 64; ++sp)
                        tma_load_2d(sm.stage[s] + kABytes + sp * kWSpanBytes, &tm_w, &sm.full[s], tn * kBN + sp * 64, kb * kBK);
                }
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(0, 1, kBN);  // A K-major, W MN-major, N = 256
            bool ok = true;
            uint32_t it = 0, local = 0;  // stages consumed; tiles done by this CTA
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++local) {
                const uint32_t buf = local & 1;
                // the epilogue must have emptied this accumulator (two tiles ago)
                ok = mbar_wait(&sm.acc_empty[buf], ((local >> 1) & 1) ^ 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem + buf * kBN;
                for (int kb = 0; kb < n_k; ++kb, ++it) {
                    const int s = it % kStages;
                    ok = mbar_wait(&sm.full[s], (it / kStages) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = smem_desc(smem_u32(sm.stage[s]), 16, 1024);
                    const uint64_t dw = smem_desc(smem_u32(sm.stage[s] + kABytes), kWSpanBytes, 1024);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {
                        // 16 input features: 32 bytes inside A's swizzle span, 16 rows (2048 bytes) of W
                        mma_ss(d_tmem, da + static_cast<uint64_t>((kk * 32) >> 4), dw + static_cast<uint64_t>((kk * 2048) >> 4),
                               idesc, (kb | kk) ? 1u : 0u);
                    }
                    mma_commit(&sm.empty[s]);
                }
                if (ok) mma_commit(&sm.acc_full[buf]);
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue: thread = output row ------------------------------
        const int quarter = warp & 3;  // the TMEM lanes this warp may read: 32 * (warp % 4) ...
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        bool ok = true;
        uint32_t local = 0;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++local) {
            int tm, tn;
            tile_coords(t, p, tm, tn);
            const uint32_t buf = local & 1;
            ok = mbar_wait(&sm.acc_full[buf], (local >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const int grow = tm * kBM + row;
            const size_t row_off = static_cast<size_t>(grow) * p.N;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
                const int col0 = tn * kBN + c * 32;
                if (col0 >= p.N) break;  // the same for every thread of the CTA
                uint32_t acc[32];
                tmem_ld32(tmem + lane_base + buf * kBN + c * 32, acc);
                tmem_wait_ld();
                if (grow < p.M) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const int col = col0 + v * 8;
                        if (col >= p.N) break;
                        float z[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) z[i] = __uint_as_float(acc[v * 8 + i]);
                        if (p.bias != nullptr) {
                            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
                            const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                z[2 * i] += __uint_as_float(bw[i] << 16);
                                z[2 * i + 1] += __uint_as_float(bw[i] & 0xffff0000u);
                            }
                        }
                        if (p.gelu) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) z[i] = z[i] / (1.0f + __expf(-1.702f * z[i]));
                        }
                        if (p.residual != nullptr) {
                            const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + row_off + col);
                            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                z[2 * i] += __uint_as_float(rw[i] << 16);
                                z[2 * i + 1] += __uint_as_float(rw[i] & 0xffff0000u);
                            }
                        }
                        uint4 w;
                        w.x = pack_bf16(z[0], z[1]);
                        w.y = pack_bf16(z[2], z[3]);
                        w.z = pack_bf16(z[4], z[5]);
                        w.w = pack_bf16(z[6], z[7]);
                        *reinterpret_cast<uint4*>(p.out + row_off + col) = w;
                    }
                }
            }
            // this warp has read its lanes of the accumulator: hand it back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
        }
        if (!ok) sm.abort_flag = 1;
    }

    // common exit: every warp arrives here, then the allocating warp releases the tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// [rows, cols] bf16 row-major matrix, boxes of box_rows x 64 columns, 128-byte swizzle; reads outside the
// matrix give zero.
static bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
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

}  // namespace gemm

}  // namespace b2kv

using namespace b2kv;

extern "C" int b2kv_matmul(const void* a, const void* w, const void* bias, const void* residual, void* out, int M, int K,
                           int N, int activation, int dtype, void* stream) {
    if (dtype != B2KV_DTYPE_BF16) return B2KV_ERR_UNSUPPORTED;
    if (!a || !w || !out) return B2KV_ERR_BAD_ARG;
    if (M <= 0 || K <= 0 || N <= 0 || activation < 0 || activation > 1) return B2KV_ERR_BAD_ARG;
    // row pitches must be multiples of 16 bytes (tensor maps, 16-byte epilogue accesses)
    if (K % 8 != 0 || N % 8 != 0) return B2KV_ERR_UNSUPPORTED;
    if (!aligned16(a) || !aligned16(w) || !aligned16(out) || !aligned16(residual) || !aligned16(bias)) return B2KV_ERR_ALIGN;
    const long long tiles_m = (static_cast<long long>(M) + gemm::kBM - 1) / gemm::kBM;
    const long long tiles_n = (static_cast<long long>(N) + gemm::kBN - 1) / gemm::kBN;
    if (tiles_m * tiles_n > 0x3fffffffLL) return B2KV_ERR_UNSUPPORTED;
    CUtensorMap ta, tw;
    if (!gemm::make_map(&ta, a, M, K, gemm::kBM) || !gemm::make_map(&tw, w, K, N, gemm::kBK)) return B2KV_ERR_UNSUPPORTED;
    gemm::GemmParams p{static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual),
                       static_cast<__nv_bfloat16*>(out), M, N, K, activation, static_cast<int>(tiles_m),
                       static_cast<int>(tiles_n)};
    constexpr size_t smem = sizeof(gemm::SharedStorage) + 1024;
    static bool configured[64] = {false};
    static int sm_count[64] = {0};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(gemm::gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)));
        B2KV_CUDA_TRY(cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
        configured[dev] = true;
    }
    const long long grid = std::min<long long>(tiles_m * tiles_n, sm_count[dev]);
    gemm::gemm_tc_kernel<<<static_cast<unsigned>(grid), gemm::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(ta, tw, p);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}
