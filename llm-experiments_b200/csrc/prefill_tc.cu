// Causal flash-attention prefill on the Blackwell tensor cores: bf16, head_dim 128 or 64.
//
// The reference kernel (simple-llm/src/gpu/gpu_kernels.py:499-770) computes the same tiled
// online softmax with scalar fp32 dot products from workgroup memory.  Here QK^T and PV are
// tcgen05.mma contractions with fp32 accumulators in tensor memory (TMEM):
//
//   * one CTA per (sequence, head, block of 256 query rows) = two 128-row tiles A and B that share
//     every K/V tile; 128-key K/V tiles up to the diagonal (A stops one tile before B);
//   * warp 8 issues TMA tiled loads (cp.async.bulk.tensor, 128-byte swizzle) of Q, K and V tiles
//     into shared memory rings that complete on mbarriers, and at the end TMA-stores the two
//     diagonal K / V tiles (the CTA's own rows) from the ring into the KV cache (a paged cache gets
//     one store per whole block, at the block its table names);
//   * warp 9 issues the MMAs from one thread: S_X = Q_X K^T (both operands K-major in shared memory)
//     into the S buffer of tile X in TMEM, and O_X += P_X V with P_X read from TMEM (it overwrites
//     S_X) and V as an MN-major shared-memory operand.  The order PV_A(j), QK_A(j+1), PV_B(j),
//     QK_B(j+1) keeps the tensor pipe busy with one tile while the other tile's softmax runs;
//   * warps 0-3 (tile A) and 4-7 (tile B) do the softmax: thread i owns query row i (= TMEM lane i),
//     reads its 128 scores with tcgen05.ld, keeps the running max / sum in registers in the log2
//     domain and writes P as packed bf16 with tcgen05.st.  O stays in TMEM for the whole row block
//     and is rescaled only when a row's running max has grown by more than 2^8 since the last
//     rescale (the factor cancels in O / l, so the result is the same);
//   * epilogue: O / max(l, 1e-8) -> bf16, L and M as the reference writes them (:762-768).
//
// TMEM columns: S_A 0-127, S_B 128-255, O_A 256-383, O_B 384-511 (all 512).
// Every mbarrier wait is bounded; a wait that runs out makes all warps fall through to the
// common exit, where the tensor memory is released.
#include <math.h>

#include <algorithm>

#include "prefill.cuh"
#include "tc_ptx.cuh"
#include "tma_map.cuh"

namespace b2kv {

namespace tc {

constexpr int kTileM = 128;   // query rows per tile (two tiles per CTA)
constexpr int kBlockN = 128;  // keys per K/V tile
constexpr int kStages = 2;                      // K ring and V ring depth
constexpr int kHalfTileBytes = 128 * 128;       // 128 rows x 64 bf16 (one 128-byte swizzle span per row)
constexpr int kThreads = 320;
constexpr int kTmemCols = 512;
constexpr int kColS = 0, kColO = 256;       // + 128 for tile B
constexpr float kRescaleThreshold = 8.0f;   // log2 units

template <int kD>
struct SharedStorage {
    static constexpr int kTileBytes = (kD / 64) * kHalfTileBytes;  // 128 rows x kD bf16
    alignas(1024) uint8_t q[2][kTileBytes];
    alignas(1024) uint8_t k[kStages][kTileBytes];
    alignas(1024) uint8_t v[kStages][kTileBytes];
    alignas(8) uint64_t q_full;
    uint64_t k_full[kStages], k_empty[kStages];
    uint64_t v_full[kStages], v_empty[kStages];
    uint64_t s_full[2], p_ready[2], o_done[2];  // per query tile
    uint32_t tmem_base;
    volatile int abort_flag;
};

template <int kD>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                  const __grid_constant__ CUtensorMap tm_vc, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    using Smem = SharedStorage<kD>;
    constexpr int kHalves = kD / 64;  // 64-column (128-byte) spans per row
    constexpr int kTileBytes = Smem::kTileBytes;
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_cb = (p.N + 2 * kTileM - 1) / (2 * kTileM);
    // Launch order: groups of `group` (sequence, head) pairs; inside a group the heaviest row blocks (most K/V
    // tiles) first.  The CTAs running together then share the K/V of few pairs, which stay in L2.
    const int n_bh = p.H * p.B;
    const int group = (p.group > 0 && p.group < n_bh) ? p.group : n_bh;
    const int per_group = group * n_cb;
    const int gi = static_cast<int>(blockIdx.x) / per_group;
    const int first_bh = gi * group;
    const int here = min(group, n_bh - first_bh);  // the last group may be smaller (and nothing follows it)
    const int within = static_cast<int>(blockIdx.x) - gi * per_group;
    const int cb = n_cb - 1 - within / here;
    const int bh = first_bh + within % here;
    const int b = bh / p.H, h = bh % p.H;
    const int q0 = cb * 2 * kTileM;
    const int qa = 2 * cb;                                 // K/V tile index of tile A's diagonal
    const int n_a = qa + 1;                                // tile A attends K/V tiles 0 .. qa
    const int n_b = (q0 + kTileM < p.N) ? qa + 2 : 0;      // tile B attends 0 .. qa + 1 (absent past the end)
    const int n_max = n_b > n_a ? n_b : n_a;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(&sm.s_full[x], 1);
            mbar_init(&sm.p_ready[x], 128);
            mbar_init(&sm.o_done[x], 1);
        }
        sm.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc(&sm.tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            const int x0 = h * kD;
            mbar_arrive_expect_tx(&sm.q_full, (n_b > 0 ? 2 : 1) * kTileBytes);
#pragma unroll
            for (int hf = 0; hf < kHalves; ++hf) {
                tma_load_3d(sm.q[0] + hf * kHalfTileBytes, &tm_q, &sm.q_full, x0 + hf * 64, q0, b);
                if (n_b > 0) tma_load_3d(sm.q[1] + hf * kHalfTileBytes, &tm_q, &sm.q_full, x0 + hf * 64, q0 + kTileM, b);
            }
            bool ok = true;
            for (int j = 0; j < n_max && ok; ++j) {
                const int st = j % kStages;
                const uint32_t par = ((j / kStages) & 1) ^ 1;
                ok = mbar_wait(&sm.k_empty[st], par);
                if (!ok) break;
                mbar_arrive_expect_tx(&sm.k_full[st], kTileBytes);
#pragma unroll
                for (int hf = 0; hf < kHalves; ++hf)
                    tma_load_3d(sm.k[st] + hf * kHalfTileBytes, &tm_k, &sm.k_full[st], x0 + hf * 64, j * kBlockN, b);
                ok = mbar_wait(&sm.v_empty[st], par);
                if (!ok) break;
                mbar_arrive_expect_tx(&sm.v_full[st], kTileBytes);
#pragma unroll
                for (int hf = 0; hf < kHalves; ++hf)
                    tma_load_3d(sm.v[st] + hf * kHalfTileBytes, &tm_v, &sm.v_full[st], x0 + hf * 64, j * kBlockN, b);
            }
            // The CTA's own K / V rows are the last one (A only) or two K/V tiles; they are still in
            // the rings.  Once the MMAs that read a tile have completed (its "empty" barrier), store
            // it to the cache.  Rows past the sequence end are clipped by the tensor map.
            if (ok && p.k_cache != nullptr) {
                // One tile of one ring to the cache: a contiguous cache takes it as one box per 64-column half; a
                // paged cache takes every whole block of it as a box of its own, at the block the table names
                // (rows past the prompt's last whole block are left to the copy kernel that follows).
                auto store_tile = [&](const CUtensorMap* map, const uint8_t* tile, int t) {
                    if (p.block_table == nullptr) {
#pragma unroll
                        for (int hf = 0; hf < kHalves; ++hf)
                            tma_store_4d(map, tile + hf * kHalfTileBytes, hf * 64, t * kBlockN, h, b);
                        return;
                    }
                    for (int r0 = 0; r0 < kBlockN; r0 += p.rows_per_store) {
                        const int tok = t * kBlockN + r0;
                        if (tok + p.rows_per_store > p.n_whole) break;
                        const int blk = p.block_table[static_cast<int64_t>(b) * p.max_blocks + tok / p.block_size];
                        if (blk < 0 || blk >= p.n_blocks) {
                            report_status(p.dev_status, B2KV_DEV_BAD_BLOCK);  // skipped: nothing is written outside the pool
                            continue;
                        }
#pragma unroll
                        for (int hf = 0; hf < kHalves; ++hf)
                            tma_store_4d(map, tile + hf * kHalfTileBytes + r0 * 128, hf * 64, tok % p.block_size, h, blk);
                    }
                };
                for (int t = qa; t < n_max && ok; ++t) {
                    const int st = t % kStages;
                    ok = mbar_wait(&sm.k_empty[st], (t / kStages) & 1);
                    if (!ok) break;
                    store_tile(&tm_kc, sm.k[st], t);
                }
                for (int t = qa; t < n_max && ok; ++t) {
                    const int st = t % kStages;
                    ok = mbar_wait(&sm.v_empty[st], (t / kStages) & 1);
                    if (!ok) break;
                    store_tile(&tm_vc, sm.v[st], t);
                }
                tma_store_commit();
                tma_store_wait();
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(0, 0, kBlockN);  // S[128 x 128 keys]
            constexpr uint32_t idesc_pv = instr_desc(0, 1, kD);       // O[128 x kD]
            // Descriptors are built once; an MMA then only adds its byte offset (in 16-byte units) to
            // the address field.  One thread issues every MMA of the CTA, so the instructions spent per
            // issue bound the rate at which the tensor pipe can be fed.
            const uint64_t dq0 = smem_desc(smem_u32(sm.q[0]), 16, 1024), dq1 = smem_desc(smem_u32(sm.q[1]), 16, 1024);
            const uint64_t dk0 = smem_desc(smem_u32(sm.k[0]), 16, 1024), dk1 = smem_desc(smem_u32(sm.k[1]), 16, 1024);
            const uint64_t dv0 = smem_desc(smem_u32(sm.v[0]), kHalfTileBytes, 1024);
            const uint64_t dv1 = smem_desc(smem_u32(sm.v[1]), kHalfTileBytes, 1024);
            static_assert(kStages == 2, "descriptor selection below assumes a two-stage ring");
            auto issue_qk = [&](int x, int j) {
                const uint64_t dq = x ? dq1 : dq0;
                const uint64_t dk = (j & 1) ? dk1 : dk0;
                const uint32_t s_tmem = tmem + kColS + x * 128;
#pragma unroll
                for (int kb = 0; kb < kHalves; ++kb) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        // 16 elements of head_dim = 32 bytes inside the 128-byte swizzle span
                        const uint64_t off = static_cast<uint64_t>((kb * kHalfTileBytes + kk * 32) >> 4);
                        mma_ss(s_tmem, dq + off, dk + off, idesc_qk, (kb | kk) ? 1u : 0u);
                    }
                }
                mma_commit(&sm.s_full[x]);
            };
            auto issue_pv = [&](int x, int j) {
                const uint64_t dv = (j & 1) ? dv1 : dv0;
                const uint32_t p_tmem = tmem + kColS + x * 128;
                const uint32_t o_tmem = tmem + kColO + x * 128;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // 16 keys per MMA: 8 packed columns of P, 16 rows (2048 bytes) of V
                    mma_ts(o_tmem, p_tmem + kk * 8, dv + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv,
                           (j | kk) ? 1u : 0u);
                }
                mma_commit(&sm.o_done[x]);
            };
            bool ok = mbar_wait(&sm.q_full, 0) && mbar_wait(&sm.k_full[0], 0);
            if (ok) {
                tc_fence_after();
                issue_qk(0, 0);
                if (n_b > 0) issue_qk(1, 0);
                mma_commit(&sm.k_empty[0]);
            }
            for (int j = 0; j < n_max && ok; ++j) {
                const int st = j % kStages;
                const uint32_t par = (j / kStages) & 1;
                const int st1 = (j + 1) % kStages;
                const uint32_t par1 = ((j + 1) / kStages) & 1;
                if (j < n_a) {
                    ok = mbar_wait(&sm.p_ready[0], j & 1) && mbar_wait(&sm.v_full[st], par);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(0, j);
                }
                if (j + 1 < n_a) {
                    ok = mbar_wait(&sm.k_full[st1], par1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(0, j + 1);
                }
                if (j < n_b) {
                    // (a wait costs the issuing thread about 100 clocks even when the barrier is long complete,
                    // and the tensor pipe idles meanwhile: V and K are only waited for once per step)
                    ok = mbar_wait(&sm.p_ready[1], j & 1) && (j < n_a || mbar_wait(&sm.v_full[st], par));
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(1, j);
                }
                mma_commit(&sm.v_empty[st]);
                if (j + 1 < n_b) {
                    ok = j + 1 < n_a || mbar_wait(&sm.k_full[st1], par1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(1, j + 1);
                }
                if (j + 1 < n_max) mma_commit(&sm.k_empty[st1]);
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else {
        // ------------------------------ softmax: thread = query row ------------------------------
        const int x = warp >> 2;             // 0 = tile A, 1 = tile B
        const int row = threadIdx.x & 127;   // row inside the tile, also the TMEM lane
        const int n_x = x ? n_b : n_a;
        const int diag_tile = qa + x;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t s_tmem = tmem + lane_base + kColS + x * 128;
        const uint32_t o_tmem = tmem + lane_base + kColO + x * 128;
        const float c = p.q_prescale;  // log2(e) / sqrt(D)
        float m_used = -INFINITY, m_run = -INFINITY, l = 0.f;
        bool ok = p.test_expire == 0;  // test hook: behave as if the first wait had run out
        for (int j = 0; j < n_x && ok; ++j) {
            ok = mbar_wait(&sm.s_full[x], j & 1);
            if (!ok) break;
            tc_fence_after();
            uint32_t r[128];
            tmem_ld128(s_tmem, r);
            tmem_wait_ld();
            // row maximum with eight independent chains (a single chain of 128 dependent max
            // operations would cost more than the exponentials)
            if (j == diag_tile) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (i > row) r[i] = 0xff800000u;  // -inf: key after the query
            }
            float mxs[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) mxs[a] = __uint_as_float(r[a]);
#pragma unroll
            for (int i = 8; i < 128; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(r[i]));
            const float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                                   fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
            m_run = fmaxf(m_run, mx * c);
            float factor = 1.f;
            bool need = false;
            if (j == 0) {
                m_used = m_run;
            } else if (m_run > m_used + kRescaleThreshold) {
                factor = ex2(m_used - m_run);
                m_used = m_run;
                need = true;
            }
            // P = exp2(s*c - m_used) as packed bf16 over the first 64 columns of the S buffer
            float sums[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) sums[a] = 0.f;
            const float neg_m = -m_used;
            const float2 c2 = make_float2(c, c), neg_m2 = make_float2(neg_m, neg_m);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    // the scaling as one packed fma per pair of scores; the row sums stay scalar (eight chains):
                    // packed adds cost register pairs that this loop does not have.  Measured and dropped here:
                    // every second to eighth pair of exponentials as a cubic on the FMA pipe (3 - 12 % slower:
                    // these warps are short of issue slots and registers, not of special-function throughput)
                    // and three-input maxima in the pass above (no change).
                    const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[cc * 32 + 2 * i]), __uint_as_float(r[cc * 32 + 2 * i + 1])), c2, neg_m2);
                    const float p0 = ex2(x.x), p1 = ex2(x.y);
                    sums[(2 * i) & 7] += p0;
                    sums[(2 * i + 1) & 7] += p1;
                    pk[i] = pack_bf16(p0, p1);
                }
                tmem_st16(s_tmem + cc * 16, pk);
            }
            const float sum0 = (sums[0] + sums[1]) + (sums[2] + sums[3]);
            const float sum1 = (sums[4] + sums[5]) + (sums[6] + sums[7]);
            l = l * factor + (sum0 + sum1);
            // rare: bring O down to the new reference maximum (needs PV of the previous tile finished)
            if (__any_sync(0xffffffffu, need)) {
                ok = mbar_wait(&sm.o_done[x], (j - 1) & 1);
                if (ok) {
                    tc_fence_after();
#pragma unroll 1
                    for (int cc = 0; cc < kD / 32; ++cc) {
                        uint32_t o[32];
                        tmem_ld32(o_tmem + cc * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                        tmem_st32(o_tmem + cc * 32, o);
                    }
                }
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sm.p_ready[x]);
        }
        // A parity wait cannot tell phase j from phase j - 2, so a thread that waits on o_done only now
        // and then must not be more than one phase behind.  It is not: S of tile j exists only after
        // QK^T(j), which was issued after PV(j - 1) into the in-order tensor pipe, so when this thread
        // has finished tile n_x - 1 every PV up to n_x - 2 has completed.
        if (ok && n_x > 0) ok = mbar_wait(&sm.o_done[x], (n_x - 1) & 1);
        if (ok && n_x > 0) {
            tc_fence_after();
            const int grow = q0 + x * kTileM + row;
            const float inv = 1.f / fmaxf(l, 1e-8f);
            const int E = p.H * kD;
            __nv_bfloat16* Og =
                static_cast<__nv_bfloat16*>(p.O) + (static_cast<size_t>(b) * p.N + grow) * E + static_cast<size_t>(h) * kD;
#pragma unroll 1
            for (int cc = 0; cc < kD / 32; ++cc) {
                uint32_t o[32];
                tmem_ld32(o_tmem + cc * 32, o);
                tmem_wait_ld();
                if (grow < p.N) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(Og + cc * 32 + v4 * 8) = w;
                    }
                }
            }
            if (grow < p.N) {
                const size_t sidx = (static_cast<size_t>(b) * p.N + grow) * p.H + h;
                if (p.L) p.L[sidx] = l * ex2(m_used - m_run);
                if (p.M) p.M[sidx] = m_run * 0.6931471805599453f;
            }
        } else if (!ok) {
            sm.abort_flag = 1;
        }
    }

    // common exit: every warp arrives here, then the allocating warp releases the tensor memory and a
    // wait that ran out anywhere in the CTA is reported to the host's status word
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
    if (threadIdx.x == 0 && sm.abort_flag) report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
}

// View of a [B*N, H*D] bf16 matrix as (x = column, y = row inside the sequence, z = sequence), so
// that rows past the end of a sequence read as zero instead of the next sequence's rows.
static bool make_map(CUtensorMap* map, const void* base, int B, int N, int E) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (fn == nullptr) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(E), static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(E) * 2, static_cast<cuuint64_t>(N) * E * 2};
    const cuuint32_t box[3] = {64, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc

template <int kD>
static int launch_prefill_tc(const PrefillParams& p_in, int dtype, void* stream) {
    constexpr int D = kD;
    PrefillParams p = p_in;
    if (p.group == 0) {
        // Launch groups whose K and V together take about 32 MB, a quarter of L2: the 16 row blocks of a
        // (sequence, head) then find its K/V in L2 instead of re-reading them from HBM.  A long run of launches is
        // power-capped, and the DRAM traffic this saves (half of it at N = 4096) buys 10 % more SM clock.
        const long long pair_bytes = 4LL * p.N * D;  // K + V of one (sequence, head), bf16
        p.group = static_cast<int>(std::max<long long>(1, (32LL << 20) / pair_bytes));
    }
    const int E = p.H * D;
    const long long n_cb = (p.N + 2 * tc::kTileM - 1) / (2 * tc::kTileM);
    const long long ctas = n_cb * p.H * p.B;
    if (ctas > 0x7fffffffLL) return B2KV_ERR_UNSUPPORTED;
    CUtensorMap tq, tk, tv, tkc, tvc;
    if (!tc::make_map(&tq, p.Q, p.B, p.N, E) || !tc::make_map(&tk, p.K, p.B, p.N, E) ||
        !tc::make_map(&tv, p.V, p.B, p.N, E))
        return B2KV_ERR_UNSUPPORTED;  // no tensor-map encoder in this driver: the SIMT kernel takes over
    if (p.k_cache != nullptr && p.block_table != nullptr) {
        // block pools as (d, token in block, head, block); one store moves rows_per_store rows of 64 columns
        if (p.stride_t < D || p.stride_h <= 0 || p.stride_b <= 0) return B2KV_ERR_UNSUPPORTED;
        if (!make_cache_tensor_map(&tkc, p.k_cache, dtype, D, p.block_size, p.H, p.n_blocks, p.stride_b, p.stride_t,
                                   p.stride_h, 64, p.rows_per_store, CU_TENSOR_MAP_SWIZZLE_128B) ||
            !make_cache_tensor_map(&tvc, p.v_cache, dtype, D, p.block_size, p.H, p.n_blocks, p.stride_b, p.stride_t,
                                   p.stride_h, 64, p.rows_per_store, CU_TENSOR_MAP_SWIZZLE_128B))
            return B2KV_ERR_UNSUPPORTED;
    } else if (p.k_cache != nullptr) {
        // a cache whose strides a tensor map cannot express goes to the SIMT kernel
        if (p.stride_t < D || p.stride_h <= 0 || p.stride_b <= 0) return B2KV_ERR_UNSUPPORTED;
        // cut to the first N tokens, so that a store of a partly filled tile leaves the rows past the
        // sequence end untouched
        if (!make_cache_tensor_map(&tkc, p.k_cache, dtype, D, p.N, p.H, p.B, p.stride_b, p.stride_t, p.stride_h, 64,
                                   128, CU_TENSOR_MAP_SWIZZLE_128B) ||
            !make_cache_tensor_map(&tvc, p.v_cache, dtype, D, p.N, p.H, p.B, p.stride_b, p.stride_t, p.stride_h, 64,
                                   128, CU_TENSOR_MAP_SWIZZLE_128B))
            return B2KV_ERR_UNSUPPORTED;
    } else {
        tkc = tk;  // never dereferenced when no cache is given
        tvc = tv;
    }
    constexpr size_t smem = sizeof(tc::SharedStorage<kD>) + 1024;
    auto kernel = tc::prefill_tc_kernel<kD>;
    static bool configured[64] = {false};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured[dev] = true;
    }
    kernel<<<static_cast<unsigned>(ctas), tc::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, tkc, tvc, p);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

int prefill_tensor_core(const PrefillParams& p, int D, int dtype, void* stream) {
    if (dtype != B2KV_DTYPE_BF16) return B2KV_ERR_UNSUPPORTED;
    if (D == 128) return launch_prefill_tc<128>(p, dtype, stream);
    if (D == 64) return launch_prefill_tc<64>(p, dtype, stream);
    return B2KV_ERR_UNSUPPORTED;
}

}  // namespace b2kv
