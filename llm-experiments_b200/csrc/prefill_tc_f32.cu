// Causal flash-attention prefill for fp32 prompts on the Blackwell tensor cores: head_dim 128 or 64.
//
// fp32 is the reference's only storage type (simple-llm/src/gpu/gpu_buffer.py:31-39) and its kernel
// (simple-llm/src/gpu/gpu_kernels.py:499-770) is scalar fp32 arithmetic, which results here have to match
// to 1e-4.  The tensor cores have no fp32 inputs and tf32 (10 mantissa bits) cannot hold that bar, so every
// operand is split into two bfloat16 numbers, x = hi + lo with hi = bf16(x), lo = bf16(x - hi), which keeps 16
// mantissa bits, and every product is three MMAs into the same fp32 accumulator:
//
//     a * b  ~  a_hi * b_hi + a_hi * b_lo + a_lo * b_hi        (the dropped a_lo * b_lo is below 2^-16 relative)
//
//   * a first kernel writes the hi and lo halves of Q, K and V into a scratch buffer ([B*N, H*D] bfloat16 each);
//   * one CTA per (sequence, head, 128 query rows).  Warp 4 loads the Q tile and, step by step, a 128-key K tile
//     and V tile (hi and lo: 64 KB each at head_dim 128, so the rings hold one step) with TMA tiled loads into
//     128-byte-swizzled shared memory; warp 5 issues S = Q K^T (3 x head_dim/16 tcgen05.mma, both operands in
//     shared memory) and O += P V (3 x 8, P read from tensor memory, V an MN-major shared-memory operand);
//   * warps 0 - 3: thread = query row = TMEM lane.  Scores in registers, running maximum and sum in the log2
//     domain in fp32, O rescaled only when the maximum has grown by more than 2^8, P written back as hi and lo
//     halves (packed bfloat16) over the score buffer: hi in columns 0 - 63, lo in columns 64 - 127;
//   * epilogue O / max(l, 1e-8) as fp32, L and M as the reference writes them (:762-768).
//
// The K / V rows of the prompt reach a cache (fp32 like the prompt) through the copy kernel of append.cu behind the
// attention: the tiles in shared memory are bfloat16 halves, not the rows themselves.
// Tensor memory: S / P columns 0 - 127, O columns 128 - 255.  Every mbarrier wait is bounded.
#include <math.h>

#include <algorithm>

#include "prefill.cuh"
#include "tc_ptx.cuh"
#include "tma_map.cuh"

namespace b2kv {

namespace tcf {

using namespace tc;

constexpr int kTileM = 128;
constexpr int kBlockN = 128;
constexpr int kHalfTileBytes = 128 * 128;  // 128 rows x 64 bf16
constexpr int kThreads = 192;              // 4 softmax warps, copy warp, MMA warp
constexpr int kTmemCols = 256;
constexpr int kColS = 0, kColO = 128;
constexpr float kRescaleThreshold = 8.0f;

template <int kD>
struct SharedStorage {
    static constexpr int kTileBytes = (kD / 64) * kHalfTileBytes;  // 128 rows x kD bf16
    alignas(1024) uint8_t q[2][kTileBytes];  // [hi / lo]
    alignas(1024) uint8_t k[2][kTileBytes];
    alignas(1024) uint8_t v[2][kTileBytes];
    alignas(8) uint64_t q_full, k_full, k_empty, v_full, v_empty, s_full, p_ready, o_done;
    uint32_t tmem_base;
    volatile int abort_flag;
};

// x -> (bf16(x), bf16(x - bf16(x))), four elements per thread.
__global__ void __launch_bounds__(256) split_kernel(const float4* __restrict__ x, uint2* __restrict__ hi, uint2* __restrict__ lo,
                                                    int64_t n4) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 a = x[i];
    const __nv_bfloat16 h0 = __float2bfloat16_rn(a.x), h1 = __float2bfloat16_rn(a.y), h2 = __float2bfloat16_rn(a.z),
                        h3 = __float2bfloat16_rn(a.w);
    uint2 ph, pl;
    ph.x = pack_bf16(__bfloat162float(h0), __bfloat162float(h1));
    ph.y = pack_bf16(__bfloat162float(h2), __bfloat162float(h3));
    pl.x = pack_bf16(a.x - __bfloat162float(h0), a.y - __bfloat162float(h1));
    pl.y = pack_bf16(a.z - __bfloat162float(h2), a.w - __bfloat162float(h3));
    hi[i] = ph;
    lo[i] = pl;
}

template <int kD>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_f32_kernel(const __grid_constant__ CUtensorMap tm_qh, const __grid_constant__ CUtensorMap tm_ql,
                      const __grid_constant__ CUtensorMap tm_kh, const __grid_constant__ CUtensorMap tm_kl,
                      const __grid_constant__ CUtensorMap tm_vh, const __grid_constant__ CUtensorMap tm_vl,
                      const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    using Smem = SharedStorage<kD>;
    constexpr int kHalves = kD / 64;
    constexpr int kTileBytes = Smem::kTileBytes;
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_rb = (p.N + kTileM - 1) / kTileM;
    // Launch order: groups of `group` (sequence, head) pairs whose K / V halves together fit a quarter of L2; inside a
    // group the heaviest row blocks first.  The CTAs running together then share the K / V of few pairs, which stay
    // in L2 (with all pairs interleaved the halves were re-read from HBM five times over).
    const int n_bh = p.H * p.B;
    const int group = (p.group > 0 && p.group < n_bh) ? p.group : n_bh;
    const int per_group = group * n_rb;
    const int gi = static_cast<int>(blockIdx.x) / per_group;
    const int first_bh = gi * group;
    const int here = min(group, n_bh - first_bh);  // the last group may be smaller (and nothing follows it)
    const int within = static_cast<int>(blockIdx.x) - gi * per_group;
    const int rb = n_rb - 1 - within / here;
    const int bh = first_bh + within % here;
    const int b = bh / p.H, h = bh % p.H;
    const int q0 = rb * kTileM;
    const int n = rb + 1;  // K/V tiles 0 .. rb (the last one holds the diagonal)

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        mbar_init(&sm.k_full, 1);
        mbar_init(&sm.k_empty, 1);
        mbar_init(&sm.v_full, 1);
        mbar_init(&sm.v_empty, 1);
        mbar_init(&sm.s_full, 1);
        mbar_init(&sm.p_ready, 4);
        mbar_init(&sm.o_done, 1);
        sm.abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 5) {
        tmem_alloc(&sm.tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            const int x0 = h * kD;
            mbar_arrive_expect_tx(&sm.q_full, 2 * kTileBytes);
#pragma unroll
            for (int hf = 0; hf < kHalves; ++hf) {
                tma_load_3d(sm.q[0] + hf * kHalfTileBytes, &tm_qh, &sm.q_full, x0 + hf * 64, q0, b);
                tma_load_3d(sm.q[1] + hf * kHalfTileBytes, &tm_ql, &sm.q_full, x0 + hf * 64, q0, b);
            }
            bool ok = true;
            for (int j = 0; j < n && ok; ++j) {
                const uint32_t par = (j & 1) ^ 1;
                ok = mbar_wait(&sm.k_empty, par);
                if (!ok) break;
                mbar_arrive_expect_tx(&sm.k_full, 2 * kTileBytes);
#pragma unroll
                for (int hf = 0; hf < kHalves; ++hf) {
                    tma_load_3d(sm.k[0] + hf * kHalfTileBytes, &tm_kh, &sm.k_full, x0 + hf * 64, j * kBlockN, b);
                    tma_load_3d(sm.k[1] + hf * kHalfTileBytes, &tm_kl, &sm.k_full, x0 + hf * 64, j * kBlockN, b);
                }
                ok = mbar_wait(&sm.v_empty, par);
                if (!ok) break;
                mbar_arrive_expect_tx(&sm.v_full, 2 * kTileBytes);
#pragma unroll
                for (int hf = 0; hf < kHalves; ++hf) {
                    tma_load_3d(sm.v[0] + hf * kHalfTileBytes, &tm_vh, &sm.v_full, x0 + hf * 64, j * kBlockN, b);
                    tma_load_3d(sm.v[1] + hf * kHalfTileBytes, &tm_vl, &sm.v_full, x0 + hf * 64, j * kBlockN, b);
                }
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == 5) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(0, 0, kBlockN);  // S[128 x 128 keys]
            constexpr uint32_t idesc_pv = instr_desc(0, 1, kD);       // O[128 x kD]
            const uint64_t dq[2] = {smem_desc(smem_u32(sm.q[0]), 16, 1024), smem_desc(smem_u32(sm.q[1]), 16, 1024)};
            const uint64_t dk[2] = {smem_desc(smem_u32(sm.k[0]), 16, 1024), smem_desc(smem_u32(sm.k[1]), 16, 1024)};
            const uint64_t dv[2] = {smem_desc(smem_u32(sm.v[0]), kHalfTileBytes, 1024),
                                    smem_desc(smem_u32(sm.v[1]), kHalfTileBytes, 1024)};
            const uint32_t s_tmem = tmem + kColS, o_tmem = tmem + kColO;
            // the three partial products of a split product: (hi, hi), (hi, lo), (lo, hi)
            auto issue_qk = [&]() {
#pragma unroll
                for (int t = 0; t < 3; ++t) {
                    const uint64_t da = dq[t == 2 ? 1 : 0], db = dk[t == 1 ? 1 : 0];
#pragma unroll
                    for (int kb = 0; kb < kHalves; ++kb) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint64_t off = static_cast<uint64_t>((kb * kHalfTileBytes + kk * 32) >> 4);
                            mma_ss(s_tmem, da + off, db + off, idesc_qk, (t | kb | kk) ? 1u : 0u);
                        }
                    }
                }
                mma_commit(&sm.s_full);
                mma_commit(&sm.k_empty);
            };
            auto issue_pv = [&](int j) {
#pragma unroll
                for (int t = 0; t < 3; ++t) {
                    const uint32_t pa = s_tmem + (t == 2 ? 64 : 0);  // P hi in columns 0 - 63, P lo in 64 - 127
                    const uint64_t db = dv[t == 1 ? 1 : 0];
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        mma_ts(o_tmem, pa + kk * 8, db + static_cast<uint64_t>((kk * 2048) >> 4), idesc_pv,
                               (j | t | kk) ? 1u : 0u);
                }
                mma_commit(&sm.o_done);
                mma_commit(&sm.v_empty);
            };
            bool ok = mbar_wait(&sm.q_full, 0) && mbar_wait(&sm.k_full, 0);
            if (ok) {
                tc_fence_after();
                issue_qk();
            }
            for (int j = 0; j < n && ok; ++j) {
                ok = mbar_wait(&sm.p_ready, j & 1) && mbar_wait(&sm.v_full, j & 1);
                if (!ok) break;
                tc_fence_after();
                issue_pv(j);
                if (j + 1 < n) {
                    ok = mbar_wait(&sm.k_full, (j + 1) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk();  // overwrites P(j): the tensor pipe runs its MMAs in order, PV(j) has read it by then
                }
            }
            if (!ok) sm.abort_flag = 1;
        }
        __syncwarp();
    } else {
        // ------------------------------ softmax: thread = query row ------------------------------
        const int row = threadIdx.x;  // row inside the tile, also the TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t s_tmem = tmem + lane_base + kColS;
        const uint32_t o_tmem = tmem + lane_base + kColO;
        const float c = p.q_prescale;  // log2(e) / sqrt(D)
        float m_used = -INFINITY, m_run = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n && ok; ++j) {
            ok = mbar_wait(&sm.s_full, j & 1);
            if (!ok) break;
            tc_fence_after();
            uint32_t r[128];
            tmem_ld128(s_tmem, r);
            tmem_wait_ld();
            if (j == rb) {
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
            // P = exp2(s*c - m_used) in fp32, written as hi + lo: packed hi pairs over columns 0 - 63 of the score
            // buffer, packed lo pairs over columns 64 - 127 (every score is in registers by now)
            float sums[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) sums[a] = 0.f;
            const float neg_m = -m_used;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t ph[16], pl[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = ex2(fmaf(__uint_as_float(r[cc * 32 + 2 * i]), c, neg_m));
                    const float p1 = ex2(fmaf(__uint_as_float(r[cc * 32 + 2 * i + 1]), c, neg_m));
                    sums[(2 * i) & 7] += p0;
                    sums[(2 * i + 1) & 7] += p1;
                    const uint32_t hi = pack_bf16(p0, p1);
                    ph[i] = hi;
                    pl[i] = pack_bf16(p0 - __uint_as_float(hi << 16), p1 - __uint_as_float(hi & 0xffff0000u));
                }
                tmem_st16(s_tmem + cc * 16, ph);
                tmem_st16(s_tmem + 64 + cc * 16, pl);
            }
            l = l * factor + (((sums[0] + sums[1]) + (sums[2] + sums[3])) + ((sums[4] + sums[5]) + (sums[6] + sums[7])));
            if (__any_sync(0xffffffffu, need)) {
                ok = mbar_wait(&sm.o_done, (j - 1) & 1);
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
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_ready);
        }
        // every PV is waited for in order here or by nobody, so the parity names the last one
        if (ok) ok = mbar_wait(&sm.o_done, (n - 1) & 1);
        if (ok) {
            tc_fence_after();
            const int grow = q0 + row;
            const float inv = 1.f / fmaxf(l, 1e-8f);
            const int E = p.H * kD;
            float* Og = static_cast<float*>(p.O) + (static_cast<size_t>(b) * p.N + grow) * E + static_cast<size_t>(h) * kD;
#pragma unroll 1
            for (int cc = 0; cc < kD / 32; ++cc) {
                uint32_t o[32];
                tmem_ld32(o_tmem + cc * 32, o);
                tmem_wait_ld();
                if (grow < p.N) {
#pragma unroll
                    for (int v4 = 0; v4 < 8; ++v4) {
                        float4 w;
                        w.x = __uint_as_float(o[v4 * 4 + 0]) * inv;
                        w.y = __uint_as_float(o[v4 * 4 + 1]) * inv;
                        w.z = __uint_as_float(o[v4 * 4 + 2]) * inv;
                        w.w = __uint_as_float(o[v4 * 4 + 3]) * inv;
                        *reinterpret_cast<float4*>(Og + cc * 32 + v4 * 4) = w;
                    }
                }
            }
            if (grow < p.N) {
                const size_t sidx = (static_cast<size_t>(b) * p.N + grow) * p.H + h;
                if (p.L) p.L[sidx] = l * ex2(m_used - m_run);
                if (p.M) p.M[sidx] = m_run * 0.6931471805599453f;
            }
        } else {
            sm.abort_flag = 1;
        }
    }

    // common exit: every warp arrives here, then the allocating warp releases the tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
    if (threadIdx.x == 0 && sm.abort_flag) report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
}

// View of a [B*N, H*D] bf16 matrix as (x = column, y = row inside the sequence, z = sequence): rows past the end
// of a sequence read as zero.
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

}  // namespace tcf

size_t prefill_f32_scratch_bytes(int B, int N, int H, int D) {
    if (D != 128 && D != 64) return 0;
    return 6ull * static_cast<size_t>(B) * N * H * D * sizeof(__nv_bfloat16);
}

template <int kD>
static int launch_prefill_tc_f32(const PrefillParams& p_in, void* scratch, void* stream) {
    PrefillParams p = p_in;
    if (p.group == 0) {
        const long long pair_bytes = 8LL * p.N * kD;  // hi and lo halves of K and V of one (sequence, head)
        p.group = static_cast<int>(std::max<long long>(1, (32LL << 20) / pair_bytes));
    }
    const int E = p.H * kD;
    const size_t elems = static_cast<size_t>(p.B) * p.N * E;
    const long long ctas = static_cast<long long>((p.N + tcf::kTileM - 1) / tcf::kTileM) * p.H * p.B;
    if (ctas > 0x7fffffffLL) return B2KV_ERR_UNSUPPORTED;
    __nv_bfloat16* half[6];
    for (int i = 0; i < 6; ++i) half[i] = static_cast<__nv_bfloat16*>(scratch) + i * elems;
    CUtensorMap tm[6];
    for (int i = 0; i < 6; ++i)
        if (!tcf::make_map(&tm[i], half[i], p.B, p.N, E)) return B2KV_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const void* src[3] = {p.Q, p.K, p.V};
    const int64_t n4 = static_cast<int64_t>(elems / 4);
    for (int i = 0; i < 3; ++i) {
        tcf::split_kernel<<<static_cast<unsigned>((n4 + 255) / 256), 256, 0, s>>>(
            static_cast<const float4*>(src[i]), reinterpret_cast<uint2*>(half[2 * i]), reinterpret_cast<uint2*>(half[2 * i + 1]),
            n4);
        B2KV_CUDA_TRY(cudaGetLastError());
    }
    constexpr size_t smem = sizeof(tcf::SharedStorage<kD>) + 1024;
    auto kernel = tcf::prefill_tc_f32_kernel<kD>;
    static bool configured[64] = {false};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured[dev] = true;
    }
    kernel<<<static_cast<unsigned>(ctas), tcf::kThreads, smem, s>>>(tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], p);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

int prefill_tensor_core_f32(const PrefillParams& p, int D, void* scratch, size_t scratch_bytes, void* stream) {
    if (scratch == nullptr || scratch_bytes < prefill_f32_scratch_bytes(p.B, p.N, p.H, D) || !aligned16(scratch))
        return B2KV_ERR_UNSUPPORTED;
    if ((static_cast<size_t>(p.B) * p.N * p.H * D) % 8 != 0) return B2KV_ERR_UNSUPPORTED;  // halves stay 16-byte aligned
    if (tensor_map_encoder() == nullptr) return B2KV_ERR_UNSUPPORTED;
    if (D == 128) return launch_prefill_tc_f32<128>(p, scratch, stream);
    if (D == 64) return launch_prefill_tc_f32<64>(p, scratch, stream);
    return B2KV_ERR_UNSUPPORTED;
}

}  // namespace b2kv
