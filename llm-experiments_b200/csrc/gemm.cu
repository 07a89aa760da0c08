// matmul for many rows on the Blackwell tensor cores: out = act(A @ W + bias) + residual, bf16 operands,
// fp32 accumulation.  This is the reference's matmul dispatch (simple-llm/src/gpu/gpu_pass_forward.py:35-82,
// C = A @ B, kernel src/gpu/gpu_kernels.py:10-134: 16x16 workgroup tiles, scalar fp32 FMAs) for the
// prompt-side projections either side of flash_attention (call sites src/wgpu_backend.py:812-930: Q / K / V,
// the output projection, the MLP), with the bias_add, gelu and residual_add dispatches that follow a
// matmul there folded into the epilogue.  Decode-step shapes (at most 128 rows) go to the weight-streaming
// kernel in qkv_append.cu instead.  Two forms: one CTA per output tile (described first) and a CTA pair per
// tile (further down; the default where clusters of two can occupy every SM).
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
    int32_t* dev_status;  // optional status word: receives B2KV_DEV_WAIT_TIMEOUT when a bounded wait ran out
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

__device__ __forceinline__ void epilogue_rows(const GemmParams& p, uint32_t t_addr, int grow, int col_base);

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
            epilogue_rows(p, tmem + lane_base + buf * kBN, tm * kBM + row, tn * kBN);
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
    if (threadIdx.x == 0 && sm.abort_flag) report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------------
// CTA-pair form (tcgen05 cta_group::2).  A cluster of two CTAs owns an output tile of 256 rows x 256
// columns: CTA r holds rows [128 r, 128 r + 128) of A and columns [128 r, 128 r + 128) of W, and every MMA
// is M = 256 over the pair, so each SM writes (TMA) and reads (MMA) 16 KB of A + 16 KB of W per 64 input
// features instead of 16 + 32: the one-CTA form's shared-memory port carries 96 B/clk of operand reads plus
// the same again in TMA writes, which holds its tensor pipe at 80 %.  The copies of both CTAs complete on
// the leader's barriers, one thread of the leader issues the MMAs and commits to the barriers of both CTAs,
// and each CTA's epilogue warps drain their own 128 lanes of the accumulator.  No multicast load is used.
// The ring holds 128 input features per stage in three stages by default (the issuing thread then waits,
// fences and commits once per eight MMAs; 4 - 5 % faster than 64 features in six stages).
// ---------------------------------------------------------------------------------------------------
// kBKP input features per ring stage (64 or 128: one or two 128-byte swizzle spans of A), kStagesP stages.
template <int kBKP, int kStagesP>
struct PairStorage {
    static constexpr int kABytesP = kBM * kBKP * 2;       // this CTA's 128 rows of A
    static constexpr int kWSpanP = kBKP * 128;            // kBKP input features x 64 columns
    static constexpr int kStageBytesP = kABytesP + 2 * kWSpanP;  // + this CTA's 128 columns of W
    alignas(1024) uint8_t stage[kStagesP][kStageBytesP];
    alignas(8) uint64_t full[kStagesP];  // leader's copy is used: both CTAs' loads complete there
    uint64_t empty[kStagesP];            // both CTAs (the leader's commits are multicast)
    uint64_t acc_full[2];                // both CTAs
    uint64_t acc_empty[2];               // leader's copy: 8 arrivals, the epilogue warps of both CTAs
    uint32_t tmem_base;
    volatile int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory object in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* ptr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(ptr)), "r"(rank));
    return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tiled load into this CTA's shared memory whose completion is counted on a barrier of either CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, int cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, int cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// Arrives once on `bar` in BOTH CTAs when every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
                     "r"(smem_u32(bar)),
                 "h"(mask)
                 : "memory");
}
// Instruction descriptor: fp32 accumulate, bf16 A and B, M = 256 over the pair, N = n.
__host__ __device__ constexpr uint32_t instr_desc_pair(int a_mn_major, int b_mn_major, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | ((static_cast<uint32_t>(n) >> 3) << 17) | ((256u >> 4) << 24);
}
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum), "r"(0)
        : "memory");
}

// Epilogue of one accumulator for one warp: thread = output row `grow` (TMEM lane of `t_addr`), columns
// [col_base, col_base + 256) clipped to N.
__device__ __forceinline__ void epilogue_rows(const GemmParams& p, uint32_t t_addr, int grow, int col_base) {
    const size_t row_off = static_cast<size_t>(grow) * p.N;
#pragma unroll 1
    for (int c = 0; c < kBN / 32; ++c) {
        const int col0 = col_base + c * 32;
        if (col0 >= p.N) break;  // the same for every thread of the CTA
        uint32_t acc[32];
        tmem_ld32(t_addr + c * 32, acc);
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
}

template <int kBKP, int kStagesP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    using Smem = PairStorage<kBKP, kStagesP>;
    constexpr int kABytesP = Smem::kABytesP, kWSpanP = Smem::kWSpanP, kStageBytesP = Smem::kStageBytesP;
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = static_cast<int>(cluster_ctarank());  // 0 = leader
    const int cid = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int n_tiles = p.tiles_m * p.tiles_n;  // tiles of 256 rows x 256 columns
    const int n_k = (p.K + kBKP - 1) / kBKP;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesP; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sm.acc_full[a], 1);
            mbar_init(&sm.acc_empty[a], 8);  // one arrival per epilogue warp of both CTAs
        }
        sm.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(&sm.tmem_base, kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything is sent to them
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            bool ok = true;
            uint32_t it = 0;
            for (int t = cid; t < n_tiles && ok; t += n_clusters) {
                int tm, tn;
                tile_coords(t, p, tm, tn);
                for (int kb = 0; kb < n_k; ++kb, ++it) {
                    const int s = it % kStagesP;
                    ok = mbar_wait(&sm.empty[s], ((it / kStagesP) & 1) ^ 1);
                    if (!ok) break;
                    if (r == 0) mbar_arrive_expect_tx(&sm.full[s], 2 * kStageBytesP);
                    const uint32_t lead_full = map_to_cta(&sm.full[s], 0);
#pragma unroll
                    for (int ks = 0; ks < kBKP / 64; ++ks)  // 64 input features (one swizzle span) per box of A
                        tma_load_2d_pair(sm.stage[s] + ks * (kBM * 128), &tm_a, lead_full, kb * kBKP + ks * 64,
                                         tm * 2 * kBM + r * kBM);
#pragma unroll
                    for (int sp = 0; sp < 2; ++sp)
                        tma_load_2d_pair(sm.stage[s] + kABytesP + sp * kWSpanP, &tm_w, lead_full,
                                         tn * kBN + r * (kBN / 2) + sp * 64, kb * kBKP);
                }
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (lane == 0 && r == 0) {
            constexpr uint32_t idesc = instr_desc_pair(0, 1, kBN);  // M = 256 over the pair, N = 256
            bool ok = true;
            uint32_t it = 0, local = 0;
            for (int t = cid; t < n_tiles && ok; t += n_clusters, ++local) {
                const uint32_t buf = local & 1;
                ok = mbar_wait(&sm.acc_empty[buf], ((local >> 1) & 1) ^ 1);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem + buf * kBN;
                for (int kb = 0; kb < n_k; ++kb, ++it) {
                    const int s = it % kStagesP;
                    ok = mbar_wait(&sm.full[s], (it / kStagesP) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = smem_desc(smem_u32(sm.stage[s]), 16, 1024);
                    const uint64_t dw = smem_desc(smem_u32(sm.stage[s] + kABytesP), kWSpanP, 1024);
#pragma unroll
                    for (int kk = 0; kk < kBKP / 16; ++kk) {
                        // A: 32 bytes inside a swizzle span, next span after four slices; W: 16 rows of 128 bytes
                        const int a_off = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
                        mma_ss_pair(d_tmem, da + static_cast<uint64_t>(a_off >> 4), dw + static_cast<uint64_t>((kk * 2048) >> 4),
                                    idesc, (kb | kk) ? 1u : 0u);
                    }
                    mma_commit_pair(&sm.empty[s]);
                }
                if (ok) mma_commit_pair(&sm.acc_full[buf]);
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else {
        // ------------------------------ epilogue (both CTAs): thread = output row ------------------------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        bool ok = true;
        uint32_t local = 0;
        for (int t = cid; t < n_tiles && ok; t += n_clusters, ++local) {
            int tm, tn;
            tile_coords(t, p, tm, tn);
            const uint32_t buf = local & 1;
            ok = mbar_wait(&sm.acc_full[buf], (local >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            epilogue_rows(p, tmem + lane_base + buf * kBN, tm * 2 * kBM + r * kBM + row, tn * kBN);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&sm.acc_empty[buf], 0));
        }
        if (!ok) sm.abort_flag = 1;
    }

    // common exit: every warp of both CTAs arrives here, then each CTA's allocating warp releases the pair's
    // tensor memory
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, kTmemCols);
    }
    if (threadIdx.x == 0 && sm.abort_flag) report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
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
                           int N, int activation, int dtype, int32_t* dev_status, void* stream) {
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
                       static_cast<int>(tiles_n), dev_status};
    constexpr size_t smem = sizeof(gemm::SharedStorage) + 1024;
    using Pair64 = gemm::PairStorage<64, 6>;
    using Pair128 = gemm::PairStorage<128, 3>;
    constexpr size_t smem_pair = sizeof(Pair64) + 1024;
    constexpr size_t smem_pair128 = sizeof(Pair128) + 1024;
    auto pair64 = gemm::gemm_pair_kernel<64, 6>;
    auto pair128 = gemm::gemm_pair_kernel<128, 3>;
    static bool configured[64] = {false};
    static int sm_count[64] = {0};
    static int max_clusters[64] = {0};  // CTA pairs of gemm_pair_kernel that can be resident together
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    auto pair_config = [&](cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, unsigned grid, size_t bytes) {
        cfg = cudaLaunchConfig_t{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(gemm::kThreads);
        cfg.dynamicSmemBytes = bytes;
        cfg.stream = static_cast<cudaStream_t>(stream);
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    };
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(gemm::gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)));
        B2KV_CUDA_TRY(cudaFuncSetAttribute(pair64, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_pair)));
        B2KV_CUDA_TRY(cudaFuncSetAttribute(pair128, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_pair128)));
        B2KV_CUDA_TRY(cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        pair_config(cfg, attr, 2u * static_cast<unsigned>(sm_count[dev]), smem_pair);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, pair64, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
        max_clusters[dev] = n;
        configured[dev] = true;
    }
    // "gemm_variant": 0 = choose (CTA pairs with 128 input features per stage where pairs fill the device),
    // 1 = one CTA per tile, 2 = CTA pairs with 64 input features per stage and six stages, 3 = CTA pairs with 128
    // and three stages.  The pair form needs (nearly) every SM to be reachable by a cluster of two; its 256-row
    // tiles pay off from a few hundred rows on.
    const int variant = tune_get("gemm_variant");
    const bool pairs_fill = 2 * max_clusters[dev] >= sm_count[dev] - 8;
    const bool use_pair =
        max_clusters[dev] > 0 && (variant == 2 || variant == 3 || (variant == 0 && pairs_fill && M > 2 * gemm::kBM));
    if (use_pair) {
        p.tiles_m = static_cast<int>((static_cast<long long>(M) + 2 * gemm::kBM - 1) / (2 * gemm::kBM));
        const long long clusters = std::min<long long>(static_cast<long long>(p.tiles_m) * p.tiles_n, max_clusters[dev]);
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        if (variant != 2) {  // default: 128 input features per stage (half as many barrier round trips per flop)
            CUtensorMap tw128;
            if (!gemm::make_map(&tw128, w, K, N, 128)) return B2KV_ERR_UNSUPPORTED;
            pair_config(cfg, attr, static_cast<unsigned>(2 * clusters), smem_pair128);
            B2KV_CUDA_TRY(cudaLaunchKernelEx(&cfg, pair128, ta, tw128, p));
        } else {
            pair_config(cfg, attr, static_cast<unsigned>(2 * clusters), smem_pair);
            B2KV_CUDA_TRY(cudaLaunchKernelEx(&cfg, pair64, ta, tw, p));
        }
        B2KV_CUDA_TRY(cudaGetLastError());
        return B2KV_OK;
    }
    const long long grid = std::min<long long>(tiles_m * tiles_n, sm_count[dev]);
    gemm::gemm_tc_kernel<<<static_cast<unsigned>(grid), gemm::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(ta, tw, p);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}
