// Causal flash-attention prefill on the Blackwell tensor cores, CTA-pair form: bf16, head_dim 128,
// sequence length a multiple of 256.
//
// Same math as the reference kernel (simple-llm/src/gpu/gpu_kernels.py:499-770) and as the
// two-tile kernel in prefill_tc.cu; what changes is how the work is laid over the SMs:
//
//   * a cluster of two CTAs (tcgen05 `cta_group::2`) owns 256 query rows of a (sequence, head):
//     CTA r holds the 128-row Q tile r.  Every MMA is M = 256 over the pair, so one instruction
//     feeds both SMs while each CTA keeps only HALF of the other operand in its shared memory
//     (64 of the 128 keys of a K tile; 64 of the 128 head_dim columns of a V tile).  That halves the
//     K/V bytes each SM has to pull through TMA and to read per MMA; the one-CTA kernel is limited
//     by exactly that shared-memory traffic;
//   * S has two buffers in tensor memory and P has its own two (it does not overwrite S).  As soon
//     as a softmax group has read the scores of step j into registers, the buffer is free and QK^T of
//     step j + 2 is issued into it, so a group finds its next scores ready when it ends a step:
//     the chain softmax -> PV -> QK^T -> softmax of the one-CTA kernel is broken;
//   * two softmax groups of four warps take the K/V steps in turn (group g: steps j = g, g + 2, ...),
//     thread = query row in both groups.  They share ONE accumulator O in tensor memory, so they
//     agree on the reference maximum step by step: a group publishes the row's reference maximum
//     after its max pass and the other group picks it up before its exponentials.  The maximum
//     is only moved when a row's tile maximum exceeds it by more than 2^8, and then the group that
//     moved it rescales O between PV(j - 1) and PV(j);
//   * warp 8 of each CTA loads its half of K / V (TMA, 128-byte swizzle; the copies of both CTAs
//     complete on the leader's mbarrier), and at the end stores the pair's own K / V rows from the
//     ring into the KV cache; in the leader CTA one thread of warp 9 issues every QK^T and one
//     thread of warp 10 every PV (the two streams share no buffer, so neither waits for the
//     other's barriers and the tensor pipe always has work queued); both commit to the barriers
//     of both CTAs.
//
// Tensor memory per CTA: S0 0-127, S1 128-255, O 256-383, P0 384-447, P1 448-511 (P is bf16, two
// keys per column).  Every mbarrier wait is bounded; a wait that runs out makes the warp
// fall through to the common exit, where both CTAs meet before the tensor memory is released.
#include <math.h>

#include <algorithm>

#include "prefill.cuh"
#include "tc_ptx.cuh"
#include "tma_map.cuh"

namespace b2kv {

namespace pair {

using namespace tc;  // PTX wrappers shared with the one-CTA kernel

constexpr int kD = 128;
constexpr int kRows = 128;          // query rows per CTA (256 per pair)
constexpr int kKeys = 128;          // keys per step (64 held by each CTA)
constexpr int kStages = 4;          // K ring and V ring depth
constexpr int kQBytes = 128 * 128 * 2;       // Q tile: 2 column halves x 128 rows x 128 B
constexpr int kQHalf = 128 * 128;
constexpr int kKBytes = 64 * 128 * 2;        // K half tile: 2 column halves x 64 keys x 128 B
constexpr int kKHalf = 64 * 128;
constexpr int kVBytes = 128 * 64 * 2;        // V half tile: 128 keys x 64 columns
constexpr int kPairThreads = 352;           // 8 softmax warps, TMA warp, two MMA-issuing warps
constexpr int kPairTmemCols = 512;
constexpr int kColS0 = 0, kColOut = 256, kColP0 = 384;
constexpr float kMoveThreshold = 8.0f;       // log2 units
constexpr int kPolyEvery = 3;                // every kPolyEvery-th pair of exponentials runs on the FMA pipe (0 = none)

struct PairShared {
    alignas(1024) uint8_t q[kQBytes];
    alignas(1024) uint8_t k[kStages][kKBytes];
    alignas(1024) uint8_t v[kStages][kVBytes];
    // leader only (the copies of both CTAs complete here)
    alignas(8) uint64_t q_full;
    uint64_t k_full[kStages], v_full[kStages];
    // One lane per warp arrives (after __syncwarp), so that a barrier takes 8 arrivals, not 256
    // serialised ones.
    uint64_t p_ready[2];  // 8 arrivals: the softmax group's 4 warps of both CTAs
    uint64_t s_free[2];   // same warps: the last score of the step has been read, S buffer g may be rewritten
    // in both CTAs (the leader's commits are multicast to the pair)
    uint64_t k_empty[kStages], v_empty[kStages];
    uint64_t s_full[2];   // S buffer g holds the scores of the group's next step
    uint64_t o_done[2];   // PV of a step with parity x has completed
    // inside one CTA, between the two softmax groups
    uint64_t m_ready[2][4];  // warp w of group g has published the reference maxima of its step (its rows)
    uint64_t fin[2][4];      // warp w of group g has left its loop and written its sums
    float m_ref[kRows];   // reference maximum per row (log2 domain), as of the last published step
    float x_l[2][kRows], x_seen[2][kRows], x_true[2][kRows];
    uint32_t tmem_base;
    volatile int abort_flag;
};

// ---- cluster / pair forms of the PTX wrappers ---------------------------------------------

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
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
    return out;
}
// Arrival on a barrier of the peer (or own) CTA.  The data it announces lives in tensor memory and is
// ordered by tcgen05.wait::st + tcgen05.fence::before_thread_sync, so the arrival itself needs no
// cluster-wide release of this thread's memory writes (which costs thousands of cycles per step).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_wait_pair(uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity); }

// TMA tiled load whose completion is counted on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
        "%5}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
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

// Arrives once on `bar` in BOTH CTAs when every tcgen05 operation issued so far by this thread has
// completed.
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

__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accum) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accum), "r"(0)
        : "memory");
}
__device__ __forceinline__ void mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accum) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accum), "r"(0)
        : "memory");
}

// ---- the two passes of a softmax step over one row (thread = row) -----------------------------
// The 128 scores of the row are read from tensor memory twice, 32 columns at a time with the next
// chunk in flight, instead of being held in 128 registers: with the registers that frees, the
// compiler can keep enough exponentials in flight to fill the special-function unit.  kMasked is the
// variant for the step on or after the diagonal (`valid` = number of keys the row may attend); the
// common variant has no branch in it.

template <bool kMasked>
__device__ __forceinline__ float row_max_pass(uint32_t s_tmem, int valid) {
    uint32_t a[32], b[32];
    float mxs[8];
#pragma unroll
    for (int x = 0; x < 8; ++x) mxs[x] = -INFINITY;
    tmem_ld32(s_tmem, a);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
        tmem_wait_ld();
        if (cc < 3) tmem_ld32(s_tmem + (cc + 1) * 32, (cc & 1) ? a : b);
        uint32_t(&cur)[32] = (cc & 1) ? b : a;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float v0 = __uint_as_float(cur[2 * i]), v1 = __uint_as_float(cur[2 * i + 1]);
            if (kMasked) {
                if (cc * 32 + 2 * i >= valid) v0 = -INFINITY;
                if (cc * 32 + 2 * i + 1 >= valid) v1 = -INFINITY;
            }
            mxs[i & 7] = fmaxf(mxs[i & 7], fmaxf(v0, v1));
        }
    }
    return fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])), fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
}

// P = exp2(s * c - m_use) as packed bf16 (two keys per column) into p_tmem; returns the row's sum of P.
// Arrives on `free_bar` once the last score has been read.  The P buffer still feeds the PV of the
// group's previous step when this starts: the first half of P is kept in registers and stored once
// `p_free` (that PV has completed) has the given parity, which by then it normally has.  Sets `ok`
// to false if that wait runs out.
template <bool kMasked>
__device__ __forceinline__ float exp_pass(uint32_t s_tmem, uint32_t p_tmem, float c, float m_use, int valid,
                                          uint32_t free_bar, uint64_t* p_free, uint32_t p_free_parity, bool wait_p_free,
                                          bool& ok) {
    // three chunk buffers: chunks 0 and 1 are requested up front, chunk 2 while chunk 0 is processed and
    // chunk 3 (into the buffer of chunk 0) while chunk 1 is, so that the last score has been read, and
    // the S buffer can be handed back, half way through the exponentials
    uint32_t a[32], b[32], d[32];
    uint32_t pk0[16], pk1[16];
    float2 sums[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) sums[x] = make_float2(0.f, 0.f);
    const float2 c2 = make_float2(c, c), neg_m2 = make_float2(-m_use, -m_use);
    tmem_ld32(s_tmem, a);
    tmem_ld32(s_tmem + 32, b);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
        tmem_wait_ld();
        if (cc == 0) tmem_ld32(s_tmem + 64, d);
        if (cc == 1) tmem_ld32(s_tmem + 96, a);
        if (cc == 2) {
            tc_fence_before();
            __syncwarp();
            if ((threadIdx.x & 31) == 0) mbar_arrive_cluster(free_bar);
        }
        uint32_t(&cur)[32] = (cc == 1) ? b : ((cc == 2) ? d : a);
        uint32_t(&pk)[16] = (cc == 0) ? pk0 : pk1;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float2 x = __ffma2_rn(make_float2(__uint_as_float(cur[2 * i]), __uint_as_float(cur[2 * i + 1])), c2, neg_m2);
            if (kMasked) {
                if (cc * 32 + 2 * i >= valid) x.x = -INFINITY;
                if (cc * 32 + 2 * i + 1 >= valid) x.y = -INFINITY;
            }
            float2 e;
            if (kPolyEvery > 0 && i % (kPolyEvery > 0 ? kPolyEvery : 1) == kPolyEvery - 1) {
                e = ex2_poly2(x);
            } else {
                e.x = ex2(x.x);
                e.y = ex2(x.y);
            }
            sums[i & 3] = __fadd2_rn(sums[i & 3], e);
            pk[i] = pack_bf16(e.x, e.y);
        }
        if (cc == 1) {
            if (wait_p_free) ok = mbar_wait(p_free, p_free_parity);
            tc_fence_after();
            tmem_st16(p_tmem, pk0);
            tmem_st16(p_tmem + 16, pk1);
        } else if (cc > 1) {
            tmem_st16(p_tmem + cc * 16, pk1);
        }
    }
    return ((sums[0].x + sums[0].y) + (sums[1].x + sums[1].y)) + ((sums[2].x + sums[2].y) + (sums[3].x + sums[3].y));
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                    const __grid_constant__ CUtensorMap tm_vc, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    PairShared& sm = *reinterpret_cast<PairShared*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = static_cast<int>(cluster_ctarank());  // 0 = leader
    const int pair_idx = blockIdx.x >> 1;
    const int n_pb = p.N / (2 * kRows);
    // Launch order as in the one-CTA kernel: groups of `group` (sequence, head) pairs, inside a group the heaviest
    // row blocks (most K/V steps) first, so that the clusters running together share the K/V of few pairs in L2.
    const int n_bh = p.H * p.B;
    const int group = (p.group > 0 && p.group < n_bh) ? p.group : n_bh;
    const int per_group = group * n_pb;
    const int gi = pair_idx / per_group;
    const int first_bh = gi * group;
    const int here = min(group, n_bh - first_bh);
    const int within = pair_idx - gi * per_group;
    const int pb = n_pb - 1 - within / here;
    const int bh = first_bh + within % here;
    const int b = bh / p.H, h = bh % p.H;
    const int q0 = pb * 2 * kRows;   // first query row of the pair
    const int n = 2 * pb + 2;        // K/V steps 0 .. 2 pb + 1
    const int diag = 2 * pb + r;     // step that holds this CTA's diagonal

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
            mbar_init(&sm.v_empty[s], 1);
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(&sm.p_ready[x], 8);
            mbar_init(&sm.s_free[x], 8);
            mbar_init(&sm.s_full[x], 1);
            mbar_init(&sm.o_done[x], 1);
            for (int w4 = 0; w4 < 4; ++w4) {
                mbar_init(&sm.m_ready[x][w4], 1);
                mbar_init(&sm.fin[x][w4], 1);
            }
        }
        sm.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 9) {
        tmem_alloc_pair(&sm.tmem_base, kPairTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything is sent to them
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 8) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            const int x0 = h * kD;
            const uint32_t lead_q = map_to_cta(&sm.q_full, 0);
            if (r == 0) mbar_arrive_expect_tx(&sm.q_full, 2 * kQBytes);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) tma_load_3d_pair(sm.q + hf * kQHalf, &tm_q, lead_q, x0 + hf * 64, q0 + r * kRows, b);
            bool ok = true;
            // K runs two steps ahead of V: a V stage is released by PV of four steps back, which is
            // late compared with when QK^T wants the next K (it runs ahead of the softmax).
            for (int jj = 0; jj < n + 2 && ok; ++jj) {
                if (jj < n) {
                    const int st = jj % kStages;
                    ok = mbar_wait_pair(&sm.k_empty[st], ((jj / kStages) & 1) ^ 1);
                    if (!ok) break;
                    if (r == 0) mbar_arrive_expect_tx(&sm.k_full[st], 2 * kKBytes);
                    const uint32_t lead_k = map_to_cta(&sm.k_full[st], 0);
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf)
                        tma_load_3d_pair(sm.k[st] + hf * kKHalf, &tm_k, lead_k, x0 + hf * 64, jj * kKeys + r * 64, b);
                }
                const int jv = jj - 2;
                if (jv >= 0) {
                    const int st = jv % kStages;
                    ok = mbar_wait_pair(&sm.v_empty[st], ((jv / kStages) & 1) ^ 1);
                    if (!ok) break;
                    if (r == 0) mbar_arrive_expect_tx(&sm.v_full[st], 2 * kVBytes);
                    tma_load_3d_pair(sm.v[st], &tm_v, map_to_cta(&sm.v_full[st], 0), x0 + r * 64, jv * kKeys, b);
                }
            }
            // The pair's own K / V rows are the last two steps; they are still in the rings.  Once the
            // MMAs that read a stage have completed (its "empty" barrier), this CTA stores its half of it.
            if (ok && p.k_cache != nullptr) {
                for (int t = n - 2; t < n && ok; ++t) {
                    const int st = t % kStages;
                    ok = mbar_wait_pair(&sm.k_empty[st], (t / kStages) & 1);
                    if (!ok) break;
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf)
                        tma_store_4d(&tm_kc, sm.k[st] + hf * kKHalf, hf * 64, t * kKeys + r * 64, h, b);
                }
                for (int t = n - 2; t < n && ok; ++t) {
                    const int st = t % kStages;
                    ok = mbar_wait_pair(&sm.v_empty[st], (t / kStages) & 1);
                    if (!ok) break;
                    tma_store_4d(&tm_vc, sm.v[st], r * 64, t * kKeys, h, b);
                }
                tma_store_commit();
                tma_store_wait();
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 9) {
        // ------------------------------ QK^T issuer (leader CTA only) ------------------------------
        if (lane == 0 && r == 0) {
            constexpr uint32_t idesc_qk = instr_desc_pair(0, 0, kKeys);  // S[256 x 128 keys]
            const uint64_t dq = smem_desc(smem_u32(sm.q), 16, 1024);
            const uint64_t dk0 = smem_desc(smem_u32(sm.k[0]), 16, 1024);
            bool ok = mbar_wait_pair(&sm.q_full, 0);
            for (int j = 0; j < n && ok; ++j) {
                const int st = j % kStages;
                // S buffer j & 1 is free once the softmax of step j - 2 has its scores in registers
                if (j >= 2) ok = mbar_wait_pair(&sm.s_free[j & 1], ((j - 2) >> 1) & 1);
                ok = ok && mbar_wait_pair(&sm.k_full[st], (j / kStages) & 1);
                if (!ok) break;
                tc_fence_after();
                // S[buffer j & 1] = Q K_j^T: head_dim in 8 slices of 16 (two 64-column halves x 4)
                const uint32_t s_tmem = tmem + kColS0 + (j & 1) * 128;
                const uint64_t dks = dk0 + static_cast<uint64_t>((st * kKBytes) >> 4);
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t offq = static_cast<uint64_t>((kb * kQHalf + kk * 32) >> 4);
                        const uint64_t offk = static_cast<uint64_t>((kb * kKHalf + kk * 32) >> 4);
                        mma_ss_pair(s_tmem, dq + offq, dks + offk, idesc_qk, (kb | kk) ? 1u : 0u);
                    }
                }
                mma_commit_pair(&sm.s_full[j & 1]);
                mma_commit_pair(&sm.k_empty[st]);
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 10) {
        // ------------------------------ PV issuer (leader CTA only) ------------------------------
        if (lane == 0 && r == 0) {
            constexpr uint32_t idesc_pv = instr_desc_pair(0, 1, kD);  // O[256 x 128]
            const uint64_t dv0 = smem_desc(smem_u32(sm.v[0]), kVBytes, 1024);
            const uint32_t o_tmem = tmem + kColOut;
            bool ok = true;
            for (int j = 0; j < n && ok; ++j) {
                const int st = j % kStages;
                ok = mbar_wait_pair(&sm.p_ready[j & 1], (j >> 1) & 1) && mbar_wait_pair(&sm.v_full[st], (j / kStages) & 1);
                if (!ok) break;
                tc_fence_after();
                // O += P_j V_j: keys in 8 slices of 16 (8 packed columns of P, 2048 bytes of V)
                const uint32_t p_tmem = tmem + kColP0 + (j & 1) * 64;
                const uint64_t dvs = dv0 + static_cast<uint64_t>((st * kVBytes) >> 4);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    mma_ts_pair(o_tmem, p_tmem + kk * 8, dvs + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv,
                                (j | kk) ? 1u : 0u);
                mma_commit_pair(&sm.o_done[j & 1]);
                mma_commit_pair(&sm.v_empty[st]);
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else {
        // ------------------------------ softmax: thread = query row, group g = steps g, g + 2, ... ----
        const int g = warp >> 2;
        const int row = threadIdx.x & 127;  // row inside the CTA's tile, also the TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t s_tmem = tmem + lane_base + kColS0 + g * 128;
        const uint32_t o_tmem = tmem + lane_base + kColOut;
        const uint32_t p_tmem = tmem + lane_base + kColP0 + g * 64;
        const uint32_t lead_p = map_to_cta(&sm.p_ready[g], 0);
        const uint32_t lead_free = map_to_cta(&sm.s_free[g], 0);
        const float c = p.q_prescale;  // log2(e) / sqrt(D)
        // m_seen: the reference maximum this group's partial sum l is relative to;
        // m_true: the true maximum over this group's steps (for the M output).
        float m_seen = -INFINITY, m_true = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = g; j < n && ok; j += 2) {
            ok = mbar_wait_pair(&sm.s_full[g], (j >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            // keys of this step the row may attend: all before the diagonal step, none after it
            const int valid = j < diag ? kKeys : (j == diag ? row + 1 : 0);
            const float mxc = c * (j < diag ? row_max_pass<false>(s_tmem, valid) : row_max_pass<true>(s_tmem, valid));
            m_true = fmaxf(m_true, mxc);
            // the reference maximum after the previous step, from the other group
            float m_prev = -INFINITY;
            if (j > 0) {
                ok = mbar_wait(&sm.m_ready[g ^ 1][warp & 3], ((j - 1) >> 1) & 1);
                if (!ok) break;
                m_prev = sm.m_ref[row];
            }
            const float m_use = (j == 0 || mxc > m_prev + kMoveThreshold) ? mxc : m_prev;
            sm.m_ref[row] = m_use;
            __syncwarp();
            if (j + 1 < n && lane == 0) mbar_arrive(&sm.m_ready[g][warp & 3]);
            const bool moved = (j > 0) && (m_use != m_prev);
            if (m_use != m_seen) {
                l *= ex2(m_seen - m_use);
                m_seen = m_use;
            }
            // rare: this step moved the reference maximum, so O (steps < j) comes down to it.  PV(j - 1)
            // must have completed; PV(j) cannot start before this thread's arrival below.  PV(j - 2) is
            // waited for first (this group's own barrier, every use of which it waits for in order): on
            // the other group's barrier the previous use (step j - 3) completed before PV(j - 2), so
            // the parity wait cannot be taken for an older phase.
            if (__any_sync(0xffffffffu, moved)) {
                if (j >= 2) ok = mbar_wait_pair(&sm.o_done[g], ((j - 2) >> 1) & 1);
                ok = ok && mbar_wait_pair(&sm.o_done[(j - 1) & 1], ((j - 1) >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const float factor = moved ? ex2(m_prev - m_use) : 1.f;
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
            // P = exp2(s*c - m_use) as packed bf16, two keys per column
            // (the P buffer of this group is free once PV of the group's previous step has completed)
            l += j < diag ? exp_pass<false>(s_tmem, p_tmem, c, m_use, valid, lead_free, &sm.o_done[g],
                                            ((j - 2) >> 1) & 1, j >= 2, ok)
                          : exp_pass<true>(s_tmem, p_tmem, c, m_use, valid, lead_free, &sm.o_done[g],
                                           ((j - 2) >> 1) & 1, j >= 2, ok);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_p);
        }
        // The two groups add up their sums.  After this exchange both know that the group which took
        // the last step has read its scores, i.e. that PV(n - 3) has completed, which is the previous
        // use of the barrier waited on below.
        sm.x_l[g][row] = l;
        sm.x_seen[g][row] = m_seen;
        sm.x_true[g][row] = m_true;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.fin[g][warp & 3]);
        if (ok) ok = mbar_wait(&sm.fin[g ^ 1][warp & 3], 0);
        if (ok) ok = mbar_wait_pair(&sm.o_done[(n - 1) & 1], ((n - 1) >> 1) & 1);
        if (ok) {
            tc_fence_after();
            const float m_fin = sm.m_ref[row];
            const float l_tot =
                sm.x_l[0][row] * ex2(sm.x_seen[0][row] - m_fin) + sm.x_l[1][row] * ex2(sm.x_seen[1][row] - m_fin);
            const float m_tot = fmaxf(sm.x_true[0][row], sm.x_true[1][row]);
            const int grow = q0 + r * kRows + row;
            const float inv = 1.f / fmaxf(l_tot, 1e-8f);
            const int E = p.H * kD;
            // group g writes head_dim columns g*64 .. g*64 + 63 of the row
            __nv_bfloat16* Og = static_cast<__nv_bfloat16*>(p.O) + (static_cast<size_t>(b) * p.N + grow) * E +
                                static_cast<size_t>(h) * kD + g * 64;
#pragma unroll 1
            for (int cc = 0; cc < 2; ++cc) {
                uint32_t o[32];
                tmem_ld32(o_tmem + g * 64 + cc * 32, o);
                tmem_wait_ld();
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
            if (g == 0) {
                const size_t sidx = (static_cast<size_t>(b) * p.N + grow) * p.H + h;
                if (p.L) p.L[sidx] = l_tot * ex2(m_fin - m_tot);
                if (p.M) p.M[sidx] = m_tot * 0.6931471805599453f;
            }
        } else {
            sm.abort_flag = 1;
        }
    }

    // common exit: every warp of both CTAs arrives here, then each CTA's allocating warp releases
    // the tensor memory of the pair
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, kPairTmemCols);
    }
    if (threadIdx.x == 0 && sm.abort_flag) report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
}

// View of a [B*N, H*D] bf16 matrix as (x = column, y = row inside the sequence, z = sequence).
static bool make_map(CUtensorMap* map, const void* base, int B, int N, int E, int box_rows) {
    EncodeTiledFn fn = tensor_map_encoder();
    if (fn == nullptr) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(E), static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(E) * 2, static_cast<cuuint64_t>(N) * E * 2};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace pair

int prefill_tensor_core_pair(const PrefillParams& p_in, int D, int dtype, void* stream) {
    PrefillParams p = p_in;
    if (p.group == 0) p.group = static_cast<int>(std::max<long long>(1, (32LL << 20) / (4LL * p.N * pair::kD)));
    if (dtype != B2KV_DTYPE_BF16 || D != pair::kD || p.block_table != nullptr) return B2KV_ERR_UNSUPPORTED;
    if (p.N < 2 * pair::kRows || p.N % (2 * pair::kRows) != 0) return B2KV_ERR_UNSUPPORTED;
    const int E = p.H * D;
    const long long ctas = 2LL * (p.N / (2 * pair::kRows)) * p.H * p.B;
    if (ctas > 0x7fffffffLL) return B2KV_ERR_UNSUPPORTED;
    CUtensorMap tq, tk, tv, tkc, tvc;
    if (!pair::make_map(&tq, p.Q, p.B, p.N, E, 128) || !pair::make_map(&tk, p.K, p.B, p.N, E, 64) ||
        !pair::make_map(&tv, p.V, p.B, p.N, E, 128))
        return B2KV_ERR_UNSUPPORTED;
    if (p.k_cache != nullptr) {
        if (p.stride_t < D || p.stride_h <= 0 || p.stride_b <= 0) return B2KV_ERR_UNSUPPORTED;
        if (!make_cache_tensor_map(&tkc, p.k_cache, dtype, D, p.N, p.H, p.B, p.stride_b, p.stride_t, p.stride_h, 64, 64,
                                   CU_TENSOR_MAP_SWIZZLE_128B) ||
            !make_cache_tensor_map(&tvc, p.v_cache, dtype, D, p.N, p.H, p.B, p.stride_b, p.stride_t, p.stride_h, 64,
                                   128, CU_TENSOR_MAP_SWIZZLE_128B))
            return B2KV_ERR_UNSUPPORTED;
    } else {
        tkc = tk;  // never dereferenced when no cache is given
        tvc = tv;
    }
    constexpr size_t smem = sizeof(pair::PairShared) + 1024;
    static bool configured[64] = {false};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(pair::prefill_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)));
        configured[dev] = true;
    }
    pair::prefill_pair_kernel<<<static_cast<unsigned>(ctas), pair::kPairThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        tq, tk, tv, tkc, tvc, p);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

}  // namespace b2kv
