// The tail of a cached generation step: layer normalisation, last-token extraction, softmax over
// the vocabulary and argmax.  fp32 like the reference's buffers (simple-llm/src/gpu/gpu_buffer.py:31-39);
// layer normalisation also takes bf16 rows and parameters (fp32 arithmetic) for a bf16 decoder layer.
//
// Reference kernels (simple-llm/src/gpu/gpu_kernels.py): layernorm :137-249 (one workgroup per row,
// mean by tree reduction, then the variance of (x - mean), then (x - mean) / sqrt(var + eps) * gamma
// + beta), extract_last_tokens :839-887 (row b*S + S - 1 of [B*S, E] to row b of [B, E]), softmax
// :890-992 (max from -1e10, sum of exp(x - max), exp(x - max) / sum).  The arithmetic is the same
// here; what changes is the mapping: rows are small next to the machine (a decode step has B rows), so a
// row is given to 32, 64, 128 or 256 threads by its length, several rows share a CTA, every row is read
// from HBM once (kept in registers when it fits, re-read from L2 otherwise) and reductions are
// warp shuffles.  All of them are HBM-bound: 8 bytes per element for layernorm and softmax.
//
// The head of a step lives here too: the embedding lookup with the position added
// (simple-llm/src/gpu/gpu_kernels.py:384-449, one thread per token looping over the row there;
// here a row is spread over the threads of a CTA in 16-byte chunks).
#include <math.h>

#include "b2kv_common.cuh"

namespace b2kv {

namespace {

constexpr int kCtaThreads = 256;
constexpr int kMaxRegChunks = 8;  // float4 chunks a thread keeps of its row (rows up to 8192 at 256 threads)

struct SumOp {
    __device__ static float apply(float a, float b) { return a + b; }
    __device__ static float identity() { return 0.f; }
};
struct MaxOp {
    __device__ static float apply(float a, float b) { return fmaxf(a, b); }
    __device__ static float identity() { return -1e10f; }  // the reference's starting maximum
};

// Reduction over the kTpr threads that share a row (kTpr consecutive threads of the CTA).
template <typename Op, int kTpr>
__device__ __forceinline__ float row_reduce(float v, float* scratch) {
#pragma unroll
    for (int off = (kTpr < 32 ? kTpr : 32) / 2; off > 0; off >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (kTpr <= 32) return v;
    constexpr int kWarps = kTpr / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = (threadIdx.x / kTpr) * kWarps;  // first warp of this row's group
    __syncthreads();  // scratch may still be read from the previous reduction
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = Op::identity();
#pragma unroll
    for (int w = 0; w < kWarps; ++w) r = Op::apply(r, scratch[first + w]);
    return r;
}

// Four consecutive elements as floats (16 bytes of fp32 or 8 bytes of bf16), and back.
__device__ __forceinline__ float4 load4(const float* p, int i) { return reinterpret_cast<const float4*>(p)[i]; }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p, int i) {
    const uint2 u = reinterpret_cast<const uint2*>(p)[i];
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, int i, float4 v) { reinterpret_cast<float4*>(p)[i] = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, int i, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    reinterpret_cast<uint2*>(p)[i] = u;
}
__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f(float* p, float v) { *p = v; }
__device__ __forceinline__ void from_f(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// mode 0: layernorm (a = gamma, b = beta); mode 1: softmax
template <int kMode, int kTpr, typename T>
__global__ void __launch_bounds__(kCtaThreads) row_kernel(const T* __restrict__ x, const T* __restrict__ ga,
                                                         const T* __restrict__ be, T* __restrict__ y,
                                                         int64_t rows, int size, float eps) {
    __shared__ float scratch[kCtaThreads / 32];
    grid_launch_dependents();
    if (threadIdx.x == 0) grid_dependency_wait();  // the rows come from the kernel before this one
    __syncthreads();
    constexpr int kRowsPerCta = kCtaThreads / kTpr;
    const int t = threadIdx.x % kTpr;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + threadIdx.x / kTpr;
    const bool live = row < rows;  // dead threads still take part in the barriers
    const T* xr = x + (live ? row : 0) * size;
    T* yr = y + (live ? row : 0) * size;
    const bool vec = (size % 4 == 0);  // rows of a 16-byte aligned matrix then start on 16 bytes
    const int chunks = vec ? size / 4 : 0;
    const bool in_regs = vec && chunks <= kMaxRegChunks * kTpr;

    float4 keep[kMaxRegChunks];
    float acc = kMode == 0 ? 0.f : MaxOp::identity();
    // pass 1: sum (layernorm) or maximum (softmax)
    if (in_regs) {
#pragma unroll
        for (int c = 0; c < kMaxRegChunks; ++c) {
            const int i = t + c * kTpr;
            if (live && i < chunks) {
                const float4 v = load4(xr, i);
                keep[c] = v;
                acc = kMode == 0 ? acc + ((v.x + v.y) + (v.z + v.w)) : fmaxf(acc, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
            }
        }
    } else if (live) {
        for (int i = t; i < size; i += kTpr) acc = kMode == 0 ? acc + to_f(xr[i]) : fmaxf(acc, to_f(xr[i]));
    }
    const float first = kMode == 0 ? row_reduce<SumOp, kTpr>(acc, scratch) / static_cast<float>(size)
                                   : row_reduce<MaxOp, kTpr>(acc, scratch);  // mean or maximum
    // pass 2: sum of squared differences, or of exponentials
    acc = 0.f;
    if (in_regs) {
#pragma unroll
        for (int c = 0; c < kMaxRegChunks; ++c) {
            const int i = t + c * kTpr;
            if (live && i < chunks) {
                float4& v = keep[c];
                if (kMode == 0) {
                    v.x -= first, v.y -= first, v.z -= first, v.w -= first;
                    acc += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
                } else {
                    v.x = expf(v.x - first), v.y = expf(v.y - first), v.z = expf(v.z - first), v.w = expf(v.w - first);
                    acc += (v.x + v.y) + (v.z + v.w);
                }
            }
        }
    } else if (live) {
        for (int i = t; i < size; i += kTpr) {
            const float d = to_f(xr[i]) - first;
            acc += kMode == 0 ? d * d : expf(d);
        }
    }
    const float second = row_reduce<SumOp, kTpr>(acc, scratch);
    const float scale = kMode == 0 ? 1.0f / sqrtf(second / static_cast<float>(size) + eps) : second;
    // pass 3: write
    if (in_regs) {
#pragma unroll
        for (int c = 0; c < kMaxRegChunks; ++c) {
            const int i = t + c * kTpr;
            if (live && i < chunks) {
                float4 v = keep[c];
                if (kMode == 0) {
                    const float4 g = load4(ga, i), b = load4(be, i);
                    v.x = v.x * scale * g.x + b.x, v.y = v.y * scale * g.y + b.y;
                    v.z = v.z * scale * g.z + b.z, v.w = v.w * scale * g.w + b.w;
                } else {
                    v.x /= scale, v.y /= scale, v.z /= scale, v.w /= scale;
                }
                store4(yr, i, v);
            }
        }
    } else if (live) {
        for (int i = t; i < size; i += kTpr) {
            const float d = to_f(xr[i]) - first;
            from_f(&yr[i], kMode == 0 ? d * scale * to_f(ga[i]) + to_f(be[i]) : expf(d) / scale);
        }
    }
}

template <int kMode, typename T>
int launch_rows(const T* x, const T* ga, const T* be, T* y, int64_t rows, int size, float eps, cudaStream_t stream) {
    // threads per row by row length (in 16-byte chunks when the row can be vectorised)
    const int work = size % 4 == 0 ? size / 4 : size;
    const int tpr = work <= 64 ? 32 : (work <= 256 ? 64 : (work <= 1024 ? 128 : 256));
    const int64_t ctas = (rows + kCtaThreads / tpr - 1) / (kCtaThreads / tpr);
    if (ctas > 0x7fffffffLL) return B2KV_ERR_UNSUPPORTED;
    const unsigned grid = static_cast<unsigned>(ctas);
    OverlapLaunch launch(grid, kCtaThreads, 0, stream);
    switch (tpr) {
        case 32: B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, row_kernel<kMode, 32, T>, x, ga, be, y, rows, size, eps)); break;
        case 64: B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, row_kernel<kMode, 64, T>, x, ga, be, y, rows, size, eps)); break;
        case 128: B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, row_kernel<kMode, 128, T>, x, ga, be, y, rows, size, eps)); break;
        default: B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, row_kernel<kMode, 256, T>, x, ga, be, y, rows, size, eps)); break;
    }
    return B2KV_OK;
}

// Row b*S + S - 1 of `in` to row b of `out`, 16 bytes per thread when the rows allow it.
__global__ void extract_last_kernel(const float* __restrict__ in, float* __restrict__ out, int B, int S, int E) {
    const int b = blockIdx.y;
    const float* src = in + (static_cast<int64_t>(b) * S + (S - 1)) * E;
    float* dst = out + static_cast<int64_t>(b) * E;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (E % 4 == 0) {
        if (i < E / 4) reinterpret_cast<float4*>(dst)[i] = reinterpret_cast<const float4*>(src)[i];
    } else if (i < E) {
        dst[i] = src[i];
    }
}

// The same for rows of whole 16-byte chunks of any element type.
__global__ void extract_last_chunks_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int S, int chunks) {
    const int b = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < chunks) out[static_cast<int64_t>(b) * chunks + i] = in[(static_cast<int64_t>(b) * S + (S - 1)) * chunks + i];
}

// out[b*S + s, :] = table[ids[b*S + s], :] + pos_enc[start_b + s, :], start_b = seq_pos[b] (or `pos0`).
// One CTA per token; four elements per thread and pass.  A token id outside the table or a position
// outside the encoding is clamped and recorded in the status word instead of being read.
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
embedding_kernel(const T* __restrict__ table, const T* __restrict__ pos_enc, const int32_t* __restrict__ ids,
                 const int32_t* __restrict__ seq_pos, int pos0, T* __restrict__ out, int S, int E, int vocab, int context,
                 int32_t* dev_status) {
    const int64_t tok = blockIdx.x;
    const int b = static_cast<int>(tok / S), s = static_cast<int>(tok - static_cast<int64_t>(b) * S);
    int id = ids[tok];
    int pos = (seq_pos ? seq_pos[b] : pos0) + s;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) report_status(dev_status, B2KV_DEV_BAD_TOKEN);
        id = 0;
    }
    if (pos < 0 || pos >= context) {
        if (threadIdx.x == 0) report_status(dev_status, B2KV_DEV_BAD_POSITION);
        pos = pos < 0 ? 0 : context - 1;
    }
    const T* tr = table + static_cast<int64_t>(id) * E;
    const T* pr = pos_enc + static_cast<int64_t>(pos) * E;
    T* yr = out + tok * E;
    for (int i = threadIdx.x; i < E / 4; i += kCtaThreads) {
        const float4 a = load4(tr, i), c = load4(pr, i);
        store4(yr, i, make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w));
    }
}

// Index of the largest value of each row (the lowest index among equals, like numpy.argmax).
template <typename T>
__global__ void __launch_bounds__(kCtaThreads) argmax_kernel(const T* __restrict__ x, int32_t* __restrict__ out, int V) {
    __shared__ float s_val[kCtaThreads / 32];
    __shared__ int s_idx[kCtaThreads / 32];
    const T* xr = x + static_cast<int64_t>(blockIdx.x) * V;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += kCtaThreads) {
        const float v = Elt<T>::to_float(xr[i]);
        if (v > best || (v == best && i < idx)) best = v, idx = i;
    }
    auto merge = [&](float ov, int oi) {
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    };
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, off), __shfl_xor_sync(0xffffffffu, idx, off));
    if ((threadIdx.x & 31) == 0) s_val[threadIdx.x >> 5] = best, s_idx[threadIdx.x >> 5] = idx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kCtaThreads / 32; ++w) merge(s_val[w], s_idx[w]);
        out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;  // a row of NaN or -inf only: index 0
    }
}

}  // namespace

}  // namespace b2kv

using namespace b2kv;

extern "C" int b2kv_layernorm(const float* x, const float* gamma, const float* beta, float* out, int64_t n_rows, int size,
                              float epsilon, void* stream) {
    if (!x || !gamma || !beta || !out) return B2KV_ERR_BAD_ARG;
    if (n_rows <= 0 || size <= 0) return B2KV_ERR_BAD_ARG;
    if (!aligned16(x) || !aligned16(gamma) || !aligned16(beta) || !aligned16(out)) return B2KV_ERR_ALIGN;
    return launch_rows<0, float>(x, gamma, beta, out, n_rows, size, epsilon, static_cast<cudaStream_t>(stream));
}

extern "C" int b2kv_layernorm_bf16(const void* x, const void* gamma, const void* beta, void* out, int64_t n_rows, int size,
                                   float epsilon, void* stream) {
    if (!x || !gamma || !beta || !out) return B2KV_ERR_BAD_ARG;
    if (n_rows <= 0 || size <= 0) return B2KV_ERR_BAD_ARG;
    if (!aligned16(x) || !aligned16(gamma) || !aligned16(beta) || !aligned16(out)) return B2KV_ERR_ALIGN;
    using T = __nv_bfloat16;
    return launch_rows<0, T>(static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta),
                             static_cast<T*>(out), n_rows, size, epsilon, static_cast<cudaStream_t>(stream));
}

extern "C" int b2kv_softmax(const float* logits, float* probs, int64_t n_rows, int size, void* stream) {
    if (!logits || !probs) return B2KV_ERR_BAD_ARG;
    if (n_rows <= 0 || size <= 0) return B2KV_ERR_BAD_ARG;
    if (!aligned16(logits) || !aligned16(probs)) return B2KV_ERR_ALIGN;
    return launch_rows<1, float>(logits, static_cast<const float*>(nullptr), static_cast<const float*>(nullptr), probs, n_rows, size, 0.f, static_cast<cudaStream_t>(stream));
}

extern "C" int b2kv_extract_last_tokens(const float* in, float* out, int batch_size, int seq_len, int embedding_dim,
                                        void* stream) {
    if (!in || !out) return B2KV_ERR_BAD_ARG;
    if (batch_size <= 0 || seq_len <= 0 || embedding_dim <= 0) return B2KV_ERR_BAD_ARG;
    if (!aligned16(in) || !aligned16(out)) return B2KV_ERR_ALIGN;
    if (batch_size > 65535) return B2KV_ERR_UNSUPPORTED;
    const int per_row = embedding_dim % 4 == 0 ? embedding_dim / 4 : embedding_dim;
    const dim3 grid((per_row + 255) / 256, batch_size);
    extract_last_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, batch_size, seq_len, embedding_dim);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

extern "C" int b2kv_argmax(const float* x, int32_t* out, int n_rows, int size, void* stream) {
    if (!x || !out) return B2KV_ERR_BAD_ARG;
    if (n_rows <= 0 || size <= 0) return B2KV_ERR_BAD_ARG;
    argmax_kernel<float><<<n_rows, kCtaThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, out, size);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

extern "C" int b2kv_argmax_bf16(const void* x, int32_t* out, int n_rows, int size, void* stream) {
    if (!x || !out) return B2KV_ERR_BAD_ARG;
    if (n_rows <= 0 || size <= 0) return B2KV_ERR_BAD_ARG;
    argmax_kernel<__nv_bfloat16><<<n_rows, kCtaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), out, size);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

extern "C" int b2kv_extract_last_tokens_bf16(const void* in, void* out, int batch_size, int seq_len, int embedding_dim,
                                             void* stream) {
    if (!in || !out) return B2KV_ERR_BAD_ARG;
    if (batch_size <= 0 || seq_len <= 0 || embedding_dim <= 0) return B2KV_ERR_BAD_ARG;
    if (!aligned16(in) || !aligned16(out)) return B2KV_ERR_ALIGN;
    if (batch_size > 65535 || embedding_dim % 8 != 0) return B2KV_ERR_UNSUPPORTED;
    const int chunks = embedding_dim / 8;
    const dim3 grid((chunks + 255) / 256, batch_size);
    extract_last_chunks_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(in), static_cast<uint4*>(out), seq_len, chunks);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

extern "C" int b2kv_embedding(const void* table, const void* pos_encoding, const int32_t* input_ids,
                              const int32_t* seq_pos, int pos0, void* out, int batch_size, int seq_len, int embedding_dim,
                              int vocab_size, int context_size, int dtype, int32_t* dev_status, void* stream) {
    if (elt_bytes(dtype) == 0) return B2KV_ERR_UNSUPPORTED;
    if (!table || !pos_encoding || !input_ids || !out) return B2KV_ERR_BAD_ARG;
    if (batch_size <= 0 || seq_len <= 0 || embedding_dim <= 0 || vocab_size <= 0 || context_size <= 0 || pos0 < 0)
        return B2KV_ERR_BAD_ARG;
    if (!aligned16(table) || !aligned16(pos_encoding) || !aligned16(out)) return B2KV_ERR_ALIGN;
    if (embedding_dim % 8 != 0) return B2KV_ERR_UNSUPPORTED;  // rows of whole 16-byte chunks in either type
    const long long tokens = static_cast<long long>(batch_size) * seq_len;
    if (tokens > 0x7fffffffLL) return B2KV_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>(tokens);
    if (dtype == B2KV_DTYPE_F32) {
        embedding_kernel<float><<<grid, kCtaThreads, 0, s>>>(
            static_cast<const float*>(table), static_cast<const float*>(pos_encoding), input_ids, seq_pos, pos0,
            static_cast<float*>(out), seq_len, embedding_dim, vocab_size, context_size, dev_status);
    } else {
        using T = __nv_bfloat16;
        embedding_kernel<T><<<grid, kCtaThreads, 0, s>>>(static_cast<const T*>(table), static_cast<const T*>(pos_encoding),
                                                        input_ids, seq_pos, pos0, static_cast<T*>(out), seq_len,
                                                        embedding_dim, vocab_size, context_size, dev_status);
    }
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}
