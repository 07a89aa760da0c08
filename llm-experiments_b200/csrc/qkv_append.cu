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
//     features of Wq | Wk | Wv.  A = a [128 k x 128 features] tile of W, which is an MN-major operand
//     exactly as the weight matrix lies in memory; B = x, K-major.  (Handing the weights over transposed,
//     so that A is K-major too, was measured and is no faster: the kernel is bound by what one SM pulls
//     from L2 - 32 KB of weights plus 16 KB of x per stage in about 985 clocks - not by the MMAs);
//   * warp 4 streams the W and x tiles with TMA (128-byte swizzle) through a ring of stages, warp 5
//     issues tcgen05.mma (M = 128, N = padded batch, K = 16) into one accumulator in tensor memory,
//     warps 0-3 are the epilogue: thread = output feature = TMEM lane, it reads the sequences' values,
//     rounds them to bf16 and writes Q to its buffer and K / V straight into cache row seq_pos[b] of every
//     sequence (consecutive lanes write consecutive head_dim elements), so the new K / V never
//     make a round trip through HBM;
//   * every wait is bounded; a position outside the cache is skipped and recorded in the status word.
//
// The same kernel with one weight matrix [K, N] is the plain product of a decode step's rows with a
// weight matrix (b2kv_matmul_rows: the attention output projection and the MLP), optionally with a
// bias, the reference's GELU and a residual applied before rounding.
//
// A matrix with few output features (N = E: 32 tiles at E = 4096) would keep only a few SMs streaming.
// Its input features are then cut into `splits` ranges; the CTAs of a tile form a thread-block cluster.
// Every CTA owns a share of the sequences (b mod splits); when its products are done a CTA stores each
// sequence's fp32 partial values into the owner's shared memory (distributed shared memory: stores are
// not waited for, unlike loads from a peer, which cost about 0.7 us each here), and after one cluster
// barrier every CTA adds up its own sequences' partials, in range order, from its own shared memory and
// writes those outputs.  No partial goes to global memory and the sum does not depend on timing.  (With
// enough tiles to fill the machine - the fused Q/K/V form - splitting was measured slower and is not
// used.)
#include <algorithm>

#include "b2kv_common.cuh"
#include "tc_ptx.cuh"
#include "tma_map.cuh"

namespace b2kv {

namespace proj {

using namespace tc;

constexpr int kFeat = 128;      // output features per CTA (MMA M)
// Input features per stage.  The issuing thread pays about 250 clocks per stage for the barrier wait,
// the fence and the commit whatever the stage holds, so a stage carries eight MMAs (128 input features),
// not four.
constexpr int kKTile = 128;
constexpr int kMaxStagesP = 6;
constexpr int kRingBytes = 200 * 1024;  // shared memory given to the ring; as many stages as fit
constexpr int kSmemBytes = 224 * 1024;  // ring and partials of a split tile together (227 KB less alignment and statics)
constexpr int kWBytes = kKTile * kFeat * 2;  // two halves of 16 KB, see the descriptors below
constexpr int kWHalf = kWBytes / 2;
constexpr int kMaxBatch = 128;
constexpr int kProjThreads = 192;

// Dynamic shared memory holds the ring: `stages` W tiles of 32 KB, then `stages` x tiles (two 64-feature
// spans of Bn rows each).  A stage takes about 1.5 us from request to arrival, so the bytes in flight
// decide the streaming rate of an SM: the ring takes all the shared memory there is.
struct ProjShared {
    alignas(8) uint64_t full[kMaxStagesP], empty[kMaxStagesP];
    uint64_t done;
    uint32_t tmem_base;
    int got[8];  // got[s] = 1: the CTA of input range s has stored its partials here (written by that CTA)
    long long row[kMaxBatch];  // element offset of every sequence's output row (-1: outside the cache), computed once
};

struct ProjParams {
    void* q_out;
    void* k_cache;
    void* v_cache;
    const int32_t* seq_pos;
    int32_t* dev_status;
    int64_t stride_b, stride_t, stride_h;
    int pos, B, Bn, E, H, D, T_max;  // E = columns of a weight matrix (output features of one matrix)
    int k_in;                         // rows of a weight matrix (input features)
    const void* residual;             // [B, E] added to the product of the single-matrix form, or null
    const void* bias;                 // [E] added before the activation, or null
    int gelu;                         // x * sigmoid(1.702 x) after the bias (simple-llm/src/gpu/gpu_kernels.py:285-293)
    int stages;
    int splits;       // CTAs per cluster = ranges of input features per tile: a power of two
    int split_shift;  // log2(splits)
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The two halves of a cluster barrier; every thread of every CTA of the cluster executes both, in turn.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Stores a 32-bit word at shared-memory address `local` (an address of this CTA's window) of CTA `rank`.
__device__ __forceinline__ void peer_store_u32(uint32_t local, uint32_t rank, uint32_t v) {
    uint32_t addr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// x * sigmoid(1.702 x), the reference's GELU (simple-llm/src/gpu/gpu_kernels.py:285-293).  The denominator is at
// least one, so the approximate division (2 ulp, no slow path: sixteen of them run interleaved) is safe; it
// vanishes in the rounding to bfloat16.
__device__ __forceinline__ float gelu_sigmoid(float x) { return __fdividef(x, 1.0f + __expf(-1.702f * x)); }

// Instruction descriptor: fp32 accumulate, bf16 operands, A MN-major, B K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t proj_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((static_cast<uint32_t>(n) >> 3) << 17) | ((128u >> 4) << 24);
}

__global__ void __launch_bounds__(kProjThreads, 1)
qkv_append_kernel(const __grid_constant__ CUtensorMap tm_wq, const __grid_constant__ CUtensorMap tm_wk,
                  const __grid_constant__ CUtensorMap tm_wv, const __grid_constant__ CUtensorMap tm_x, const ProjParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ ProjShared sm;
    uint8_t* const w_ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = p.splits > 1 ? static_cast<int>(cluster_rank()) : 0;
    const int f0 = (blockIdx.x / p.splits) * kFeat;  // first output feature, in the concatenation Wq | Wk | Wv
    const int which = f0 / p.E;         // 0 = Q, 1 = K, 2 = V
    const int c0 = f0 % p.E;            // first column inside that weight matrix
    const int n_k_all = p.k_in / kKTile;  // this CTA's range of input-feature tiles
    const int k_first = static_cast<int>(static_cast<long long>(n_k_all) * split / p.splits);
    const int n_k = static_cast<int>(static_cast<long long>(n_k_all) * (split + 1) / p.splits) - k_first;
    const uint32_t x_span = static_cast<uint32_t>(p.Bn) * 128u;  // Bn rows of one 64-feature span
    uint8_t* const x_ring = w_ring + p.stages * kWBytes;
    const int n_st = p.stages;
    // behind the rings when a tile is split: partials of this CTA's sequences, [input range][sequence / splits][feature]
    float* const recv = reinterpret_cast<float*>(x_ring + p.stages * 2 * x_span);
    const int rows_per_cta = p.Bn >> p.split_shift;
    const uint32_t stage_bytes = kWBytes + 2 * x_span;

    grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStagesP; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.done, 1);
        for (int s = 0; s < 8; ++s) sm.got[s] = 0;
        fence_mbar_init();
    }
    __syncthreads();  // barriers are initialised: the producer starts while the rest is set up
    // first cluster barrier: once a CTA has waited for it, all its peers are running with their flags cleared
    // (the copy warp arrives after its first requests: the arrival orders earlier writes and takes half a microsecond)
    if (p.splits > 1 && warp != 4) cluster_arrive();
    if (warp == 5) {
        tmem_alloc(&sm.tmem_base, kMaxBatch);
        tmem_relinquish();
        tc_fence_before();
    }
    // Launched ahead of the end of the kernel before it: only the weights, which no kernel writes, are
    // touched before that kernel is complete.  The copy warp waits after it has asked for the ring's
    // first weight tiles; one thread waits for the epilogue warps (positions, residual, outputs); the
    // issuing warp touches shared and tensor memory only.
    if (threadIdx.x < kMaxBatch) {
        if (threadIdx.x == 0) grid_dependency_wait();
        named_barrier_sync<kMaxBatch>(2);
        // where sequence b's values go: its row of q_out, or its new row of the cache
        const int b = threadIdx.x;
        long long row = -1;
        if (b < p.B) {
            if (which == 0) {
                row = static_cast<long long>(b) * p.E;
            } else {
                const int pos = p.seq_pos ? p.seq_pos[b] : p.pos;
                if (pos < 0 || pos >= p.T_max)
                    report_status(p.dev_status, B2KV_DEV_BAD_POSITION);
                else
                    row = static_cast<long long>(b) * p.stride_b + static_cast<long long>(pos) * p.stride_t;
            }
        }
        sm.row[b] = row;
    }

    // Split tile: where this CTA's own sequences go and what is added to them is fetched ahead of the sums, eight
    // sequences at a time: for the first eight while the weights still stream, for the next under the sums.
    const __nv_bfloat16* const res_split =
        (p.splits > 1 && p.residual) ? static_cast<const __nv_bfloat16*>(p.residual) + c0 + (threadIdx.x & (kFeat - 1)) : nullptr;
    float bias_split = 0.f;
    long long row_next[8];
    float add_next[8];
    auto fetch_split = [&](int r0) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int b = ((r0 + u) << p.split_shift) + split;
            row_next[u] = (r0 + u < rows_per_cta && b < p.B) ? sm.row[b] : -1;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            add_next[u] = (res_split != nullptr && row_next[u] >= 0) ? __bfloat162float(res_split[row_next[u]]) : 0.f;
    };

    if (warp == 4) {
        const CUtensorMap* tw = which == 0 ? &tm_wq : (which == 1 ? &tm_wk : &tm_wv);
        // W tile: input features k0 .. +127 (rows), output features c0 .. c0+127 as two 64-wide boxes
        auto load_w = [&](int st, int k0) {
            tma_load_2d(w_ring + st * kWBytes, tw, &sm.full[st], c0, k0);
            tma_load_2d(w_ring + st * kWBytes + kWHalf, tw, &sm.full[st], c0 + 64, k0);
        };
        // x tile: every sequence (rows past B read as zero), two 64-feature spans
        auto load_x = [&](int st, int k0) {
            tma_load_2d(x_ring + st * 2 * x_span, &tm_x, &sm.full[st], k0, 0);
            tma_load_2d(x_ring + st * 2 * x_span + x_span, &tm_x, &sm.full[st], k0 + 64, 0);
        };
        // the ring starts empty: its first round of weight tiles is on its way before x may be read
        const int ahead = n_k < n_st ? n_k : n_st;
        if (lane == 0) {
            for (int i = 0; i < ahead; ++i) {
                mbar_arrive_expect_tx(&sm.full[i], stage_bytes);
                load_w(i, (k_first + i) * kKTile);
            }
            grid_dependency_wait();
            for (int i = 0; i < ahead; ++i) load_x(i, (k_first + i) * kKTile);
        }
        __syncwarp();
        if (p.splits > 1) cluster_arrive();
        if (lane == 0) {
            for (int i = ahead; i < n_k; ++i) {
                const int st = i % n_st;
                if (!mbar_wait(&sm.empty[st], ((i / n_st) & 1) ^ 1)) break;
                mbar_arrive_expect_tx(&sm.full[st], stage_bytes);
                const int k0 = (k_first + i) * kKTile;
                load_w(st, k0);
                load_x(st, k0);
            }
        }
        __syncwarp();
        if (p.splits > 1) cluster_wait();
    } else if (warp == 5) {
        if (lane == 0) {
            tc_fence_after();
            const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sm.tmem_base);  // allocated by this warp above
            const uint32_t idesc = proj_idesc(p.Bn);
            bool ok = true;
            for (int i = 0; i < n_k && ok; ++i) {
                const int st = i % n_st;
                ok = mbar_wait(&sm.full[st], (i / n_st) & 1);
                if (!ok) break;
                tc_fence_after();
                // A: [feature half][128 k][64 features] MN-major (halves 16 KB apart, 8 k-rows = 1024 B, 16 k =
                // 2048 B).  B: [k span][sequence][64 k] K-major (16 k = 32 B inside the swizzle span).
                const uint64_t da = smem_desc(smem_u32(w_ring + st * kWBytes), kWHalf, 1024);
                const uint64_t db = smem_desc(smem_u32(x_ring + st * 2 * x_span), 16, 1024);
#pragma unroll
                for (int kk = 0; kk < kKTile / 16; ++kk) {
                    const uint32_t b_off = (kk >> 2) * x_span + (kk & 3) * 32;
                    mma_ss(tmem, da + static_cast<uint64_t>((kk * 2048) >> 4), db + static_cast<uint64_t>(b_off >> 4), idesc,
                           (i | kk) ? 1u : 0u);
                }
                mma_commit(&sm.empty[st]);
            }
            if (ok) mma_commit(&sm.done);
        }
        __syncwarp();
        if (p.splits > 1) cluster_wait();
    } else {
        // ------------------------------ epilogue: thread = output feature ------------------------------
        const int m = threadIdx.x;  // 0..127, also the TMEM lane
        named_barrier_sync<128>(1);  // sm.row is complete
        if (p.splits > 1) {
            cluster_wait();
            bias_split = p.bias ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[c0 + m]) : 0.f;
            fetch_split(0);
        }
        if (mbar_wait(&sm.done, 0)) {
            tc_fence_after();
            // (the accumulator's address was stored by the issuing warp before its first MMA)
            const uint32_t t_lane = sm.tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
            if (p.splits > 1) {
                // sequence b's partial goes to CTA b mod splits, slab `split`, row b / splits
                const uint32_t mine = smem_u32(recv) + static_cast<uint32_t>((split * rows_per_cta) * kFeat + m) * 4u;
                for (int nb = 0; nb < p.Bn; nb += 16) {
                    uint32_t v[16];
                    tmem_ld16(t_lane + nb, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int b = nb + j;
                        peer_store_u32(mine + static_cast<uint32_t>((b >> p.split_shift) * kFeat) * 4u,
                                       static_cast<uint32_t>(b & (p.splits - 1)), v[j]);
                    }
                }
                if (m < p.splits) peer_store_u32(smem_u32(&sm.got[split]), static_cast<uint32_t>(m), 1u);
            } else {
                const int col = c0 + m;  // column inside the weight matrix = element of the output row
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(which == 0 ? p.q_out : (which == 1 ? p.k_cache : p.v_cache));
                // inside the row: the element itself for Q, (head, head_dim element) for the cache
                out += which == 0 ? col : static_cast<long long>(col / p.D) * p.stride_h + col % p.D;
                const __nv_bfloat16* res = p.residual ? static_cast<const __nv_bfloat16*>(p.residual) + col : nullptr;
                const float bias = p.bias ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col]) : 0.f;
                for (int nb = 0; nb < p.Bn; nb += 16) {
                    uint32_t v[16];
                    tmem_ld16(t_lane + nb, v);
                    // sixteen sequences at a time, as straight-line code: rows and residuals are fetched together
                    // (-1: past the batch, or a position outside the cache), then the values, then the stores
                    long long row[16];
                    float add[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) row[j] = sm.row[nb + j];
#pragma unroll
                    for (int j = 0; j < 16; ++j) add[j] = (res != nullptr && row[j] >= 0) ? __bfloat162float(res[row[j]]) : 0.f;
                    tmem_wait_ld();
                    __nv_bfloat16 o[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float acc = __uint_as_float(v[j]) + bias;
                        if (p.gelu) acc = gelu_sigmoid(acc);
                        if (res != nullptr) acc += add[j];
                        o[j] = __float2bfloat16_rn(acc);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (row[j] >= 0) out[row[j]] = o[j];
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
        tmem_dealloc(sm.tmem_base, kMaxBatch);
    }
    if (p.splits > 1) {
        // second cluster barrier: the partials of this CTA's sequences have arrived (or a CTA gave up and did not
        // raise its flag: then nothing is written).  Nobody touches a peer's memory after it, so a CTA may leave
        // as soon as it has written its outputs.
        cluster_arrive();
        cluster_wait();
        if (warp < 4) {
            const int m = threadIdx.x;
            bool all = true;
            for (int sp = 0; sp < p.splits; ++sp) all = all && *reinterpret_cast<volatile int*>(&sm.got[sp]) != 0;
            if (all) {
                // this CTA's sequences: split, split + splits, ...; eight at a time
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.q_out) + c0 + m;  // a split tile is a plain row product
                for (int r0 = 0; r0 < rows_per_cta; r0 += 8) {
                    long long row[8];
                    float add[8], acc[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) row[u] = row_next[u], add[u] = add_next[u], acc[u] = bias_split;
                    if (r0 + 8 < rows_per_cta) fetch_split(r0 + 8);
                    for (int sp = 0; sp < p.splits; ++sp) {  // fixed order
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            if (r0 + u < rows_per_cta) acc[u] += recv[(sp * rows_per_cta + r0 + u) * kFeat + m];
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        if (row[u] < 0) continue;
                        float a = acc[u];
                        if (p.gelu) a = gelu_sigmoid(a);
                        if (res_split != nullptr) a += add[u];
                        out[row[u]] = __float2bfloat16_rn(a);
                    }
                }
            }
        }
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

// Raises the kernel's dynamic shared memory limit on this device when a larger ring is asked for.
static cudaError_t configure_smem(int dev, size_t smem) {
    static int configured[64] = {0};
    if (configured[dev] < static_cast<int>(smem)) {
        cudaError_t e = cudaFuncSetAttribute(qkv_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        configured[dev] = static_cast<int>(smem);
    }
    return cudaSuccess;
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
    const int w_box_rows = proj::kKTile;  // 128 input features x 64 output features per box
    if (!proj::make_matrix_map(&tq, wq, E, E, w_box_rows) || !proj::make_matrix_map(&tk, wk, E, E, w_box_rows) ||
        !proj::make_matrix_map(&tv, wv, E, E, w_box_rows) || !proj::make_matrix_map(&tx, x, B, E, Bn))
        return B2KV_ERR_UNSUPPORTED;
    const int stage_bytes = proj::kWBytes + 2 * Bn * 128;
    const int stages = std::max(2, std::min(proj::kMaxStagesP, proj::kRingBytes / stage_bytes));
    const size_t smem = static_cast<size_t>(stages) * stage_bytes + 1024;
    proj::ProjParams p{q_out, k_cache, v_cache, seq_pos, dev_status, stride_b, stride_t, stride_h, pos, B, Bn, E, H, D, T_max,
                       E, nullptr, nullptr, 0, stages, 1, 0};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    B2KV_CUDA_TRY(proj::configure_smem(dev, smem));
    OverlapLaunch launch(3 * E / proj::kFeat, proj::kProjThreads, smem, stream);
    B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, proj::qkv_append_kernel, tq, tk, tv, tx, p));
    return B2KV_OK;
}

extern "C" int b2kv_matmul_rows(const void* x, const void* w, const void* bias, const void* residual, void* out, int B, int K,
                                int N, int activation, int dtype, void* stream) {
    if (dtype != B2KV_DTYPE_BF16) return B2KV_ERR_UNSUPPORTED;
    if (!x || !w || !out) return B2KV_ERR_BAD_ARG;
    if (B <= 0 || K <= 0 || N <= 0 || activation < 0 || activation > 1) return B2KV_ERR_BAD_ARG;
    if (B > proj::kMaxBatch || K % proj::kKTile != 0 || N % proj::kFeat != 0) return B2KV_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(w) || !aligned16(out) || !aligned16(residual) || !aligned16(bias)) return B2KV_ERR_ALIGN;
    const int Bn = ((B + 15) / 16) * 16;
    CUtensorMap tw, tx;
    if (!proj::make_matrix_map(&tw, w, K, N, proj::kKTile) || !proj::make_matrix_map(&tx, x, B, K, Bn))
        return B2KV_ERR_UNSUPPORTED;
    // few tiles: cut the input features so that about 128 CTAs stream (a power of two, at least two stages each)
    const int tiles = N / proj::kFeat, n_k = K / proj::kKTile;
    int splits = 1, split_shift = 0;
    if (tune_get("matmul_splits") > 0) {
        while (splits * 2 <= std::min(std::min(tune_get("matmul_splits"), 8), n_k)) splits *= 2;
    } else {
        while (splits < 8 && tiles * splits * 2 <= 128 && n_k / (splits * 2) >= 2) splits *= 2;
    }
    while ((1 << split_shift) < splits) ++split_shift;
    // a split tile keeps the partials of its own sequences behind the rings: [splits][Bn / splits][128] fp32
    const int recv_bytes = splits > 1 ? Bn * proj::kFeat * 4 : 0;
    const int stage_bytes = proj::kWBytes + 2 * Bn * 128;
    const int ring_bytes = std::min(proj::kRingBytes, proj::kSmemBytes - recv_bytes);
    const int stages = std::max(2, std::min(proj::kMaxStagesP, ring_bytes / stage_bytes));
    const size_t smem = static_cast<size_t>(stages) * stage_bytes + recv_bytes + 1024;
    // one weight matrix: every tile is of kind 0 (plain rows of `out`); the cache fields are unused
    proj::ProjParams p{out, nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, B, Bn, N, 1, N, 1, K, residual, bias, activation,
                       stages, splits, split_shift};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    B2KV_CUDA_TRY(proj::configure_smem(dev, smem));
    OverlapLaunch launch(tiles * splits, proj::kProjThreads, smem, stream, splits);  // cluster = the CTAs of one tile
    B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, proj::qkv_append_kernel, tw, tw, tw, tx, p));
    return B2KV_OK;
}
