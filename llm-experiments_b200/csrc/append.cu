// KV-cache append and gather: pure byte movement with 16-byte vector loads and stores.
//
// Append is the B200 form of the reference's kv_cache_update kernel
// (simple-llm/src/gpu/gpu_kernels.py:2725-2798): one thread there copies one float of K
// and one of V; here one thread copies one 16-byte chunk of each, for any storage type,
// any cache layout given by strides, and optionally through a block table.
#include <algorithm>

#include "b2kv_common.cuh"

namespace b2kv {

struct RowMap {
    const int32_t* seq;          // per-sequence position / length, or null
    int scalar;                  // used when seq is null
    const int32_t* block_table;  // null = contiguous
    int max_blocks, block_size, n_blocks;
    int64_t stride_b, stride_t, stride_h;  // elements; stride_b is the block stride when paged
    int T_max;                             // contiguous: rows per sequence
    int32_t* dev_status;
};

// Element offset of row (b, t) (head 0), or -1 after recording a status code.
__device__ __forceinline__ int64_t row_offset(const RowMap& m, int b, int t) {
    if (m.block_table == nullptr) {
        if (t < 0 || t >= m.T_max) {
            report_status(m.dev_status, B2KV_DEV_BAD_POSITION);
            return -1;
        }
        return static_cast<int64_t>(b) * m.stride_b + static_cast<int64_t>(t) * m.stride_t;
    }
    const int j = t / m.block_size;
    if (t < 0 || j >= m.max_blocks) {
        report_status(m.dev_status, B2KV_DEV_BAD_POSITION);
        return -1;
    }
    const int blk = m.block_table[static_cast<int64_t>(b) * m.max_blocks + j];
    if (blk < 0 || blk >= m.n_blocks) {
        report_status(m.dev_status, B2KV_DEV_BAD_BLOCK);
        return -1;
    }
    return static_cast<int64_t>(blk) * m.stride_b + static_cast<int64_t>(t % m.block_size) * m.stride_t;
}

// One CTA per sequence; chunks_per_row = H*D*es/16, `shift` = log2(elements per chunk).  With
// `advance` the CTA adds one to its sequence's position after every thread has read it, which
// is race-free because no other CTA touches that entry.
__global__ void __launch_bounds__(1024) append_kernel(const uint4* __restrict__ new_k, const uint4* __restrict__ new_v,
                                                      uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                                                      RowMap m, int32_t* seq_rw, int advance, int H, int D,
                                                      int chunks_per_row, int shift) {
    grid_launch_dependents();
    if (threadIdx.x == 0) grid_dependency_wait();  // the new rows and the positions may come from the kernel before this one
    __syncthreads();
    const int b = blockIdx.x;
    const int t = seq_rw ? seq_rw[b] : m.scalar;
    const int64_t base = row_offset(m, b, t);
    if (base >= 0) {
        for (int idx = threadIdx.x; idx < chunks_per_row; idx += blockDim.x) {
            const int e = idx << shift;  // first element of this chunk inside the [H*D] row
            const int h = e / D, d = e - h * D;
            const int64_t dst = (base + static_cast<int64_t>(h) * m.stride_h + d) >> shift;
            const int64_t src = static_cast<int64_t>(b) * chunks_per_row + idx;
            const uint4 kk = new_k[src];
            const uint4 vv = new_v[src];
            k_cache[dst] = kk;
            v_cache[dst] = vv;
        }
    }
    if (advance && seq_rw) {
        __syncthreads();
        if (threadIdx.x == 0 && base >= 0) seq_rw[b] = t + 1;
    }
}

// seq[b] += delta for b < B: the lengths of a ragged cache after a kernel that appended without advancing them.
__global__ void __launch_bounds__(1024) advance_kernel(int32_t* seq, int B, int delta) {
    grid_launch_dependents();
    if (threadIdx.x == 0) grid_dependency_wait();  // the kernel before this one still reads the old lengths
    __syncthreads();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) seq[b] += delta;
}

// Many rows per sequence (a prompt): grid (n_rows, B); rows[b * src_rows_per_seq + src_first + i] goes to position
// first_pos + i of sequence b.  Same addressing as append_kernel; nothing is advanced.
__global__ void __launch_bounds__(512) append_rows_kernel(const uint4* __restrict__ k_rows, const uint4* __restrict__ v_rows,
                                                          uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, RowMap m,
                                                          int src_rows_per_seq, int src_first, int first_pos, int H, int D,
                                                          int chunks_per_row, int shift) {
    const int b = blockIdx.y, i = blockIdx.x;
    const int64_t base = row_offset(m, b, first_pos + i);
    if (base < 0) return;
    const int64_t src0 = (static_cast<int64_t>(b) * src_rows_per_seq + src_first + i) * chunks_per_row;
    for (int idx = threadIdx.x; idx < chunks_per_row; idx += blockDim.x) {
        const int e = idx << shift;
        const int h = e / D, d = e - h * D;
        const int64_t dst = (base + static_cast<int64_t>(h) * m.stride_h + d) >> shift;
        const uint4 kk = k_rows[src0 + idx];
        const uint4 vv = v_rows[src0 + idx];
        k_cache[dst] = kk;
        v_cache[dst] = vv;
    }
}

// grid (ceil(chunks_per_row / 128), T_out, B): out[b, t, :, :] = cache row (b, t) or zero past the length.
__global__ void __launch_bounds__(128) gather_kernel(const uint4* __restrict__ cache, uint4* __restrict__ out, RowMap m,
                                                     int H, int D, int T_out, int chunks_per_row, int shift) {
    const int b = blockIdx.z, t = blockIdx.y;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= chunks_per_row) return;
    const int n = m.seq ? m.seq[b] : m.scalar;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (t < n) {
        const int64_t base = row_offset(m, b, t);
        if (base >= 0) {
            const int e = idx << shift;
            const int h = e / D, d = e - h * D;
            val = cache[(base + static_cast<int64_t>(h) * m.stride_h + d) >> shift];
        }
    }
    out[(static_cast<int64_t>(b) * T_out + t) * chunks_per_row + idx] = val;
}

static int check_common(int B, int H, int D, int dtype, int64_t s0, int64_t st, int64_t sh) {
    const int es = elt_bytes(dtype);
    if (es == 0) return B2KV_ERR_UNSUPPORTED;
    if (B <= 0 || H <= 0 || D <= 0) return B2KV_ERR_BAD_ARG;
    if ((D * es) % 16 != 0) return B2KV_ERR_UNSUPPORTED;
    if (!stride_ok(s0, es) || !stride_ok(st, es) || !stride_ok(sh, es)) return B2KV_ERR_ALIGN;
    return B2KV_OK;
}

static int launch_append(const void* new_k, const void* new_v, void* k_cache, void* v_cache, RowMap m,
                         int32_t* seq_rw, int advance, int B, int H, int D, int dtype, void* stream) {
    if (!new_k || !new_v || !k_cache || !v_cache) return B2KV_ERR_BAD_ARG;
    if (!aligned16(new_k) || !aligned16(new_v) || !aligned16(k_cache) || !aligned16(v_cache)) return B2KV_ERR_ALIGN;
    const int es = elt_bytes(dtype);
    const int chunks = H * D * es / 16;
    const int shift = es == 4 ? 2 : 3;
    int threads = (chunks + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    OverlapLaunch launch(B, threads, 0, stream);
    B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, append_kernel, static_cast<const uint4*>(new_k),
                                     static_cast<const uint4*>(new_v), static_cast<uint4*>(k_cache),
                                     static_cast<uint4*>(v_cache), m, seq_rw, advance, H, D, chunks, shift));
    return B2KV_OK;
}

static int launch_gather(const void* cache, void* out, RowMap m, int B, int H, int D, int T_out, int dtype,
                         void* stream) {
    if (!cache || !out || T_out <= 0) return B2KV_ERR_BAD_ARG;
    if (!aligned16(cache) || !aligned16(out)) return B2KV_ERR_ALIGN;
    if (B > 65535 || T_out > 65535) return B2KV_ERR_UNSUPPORTED;
    const int es = elt_bytes(dtype);
    const int chunks = H * D * es / 16;
    const int shift = es == 4 ? 2 : 3;
    dim3 grid((chunks + 127) / 128, T_out, B);
    gather_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(cache), static_cast<uint4*>(out), m, H, D, T_out, chunks, shift);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

// Rows [b * n_rows + i] of k_rows / v_rows to position i of sequence b of a contiguous cache (a whole prompt).
int append_rows_contiguous(const void* k_rows, const void* v_rows, void* k_cache, void* v_cache, int B, int n_rows, int H,
                           int D, int T_max, int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype,
                           int32_t* dev_status, void* stream) {
    int rc = check_common(B, H, D, dtype, stride_b, stride_t, stride_h);
    if (rc != B2KV_OK) return rc;
    if (!k_rows || !v_rows || !k_cache || !v_cache || n_rows <= 0 || n_rows > T_max) return B2KV_ERR_BAD_ARG;
    if (!aligned16(k_rows) || !aligned16(v_rows) || !aligned16(k_cache) || !aligned16(v_cache)) return B2KV_ERR_ALIGN;
    if (B > 65535) return B2KV_ERR_UNSUPPORTED;
    RowMap m{nullptr, 0, nullptr, 0, 0, 0, stride_b, stride_t, stride_h, T_max, dev_status};
    const int es = elt_bytes(dtype);
    const int chunks = H * D * es / 16;
    const int shift = es == 4 ? 2 : 3;
    int threads = (chunks + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    append_rows_kernel<<<dim3(n_rows, B), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(k_rows), static_cast<const uint4*>(v_rows), static_cast<uint4*>(k_cache),
        static_cast<uint4*>(v_cache), m, n_rows, 0, 0, H, D, chunks, shift);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

int append_rows_paged_from(const void* k_rows, const void* v_rows, void* k_pool, void* v_pool, const int32_t* block_table,
                           int max_blocks, int block_size, int n_blocks, int B, int n_rows, int first_pos,
                           int src_rows_per_seq, int src_first, int H, int D, int64_t stride_blk, int64_t stride_t,
                           int64_t stride_h, int dtype, int32_t* dev_status, void* stream) {
    int rc = check_common(B, H, D, dtype, stride_blk, stride_t, stride_h);
    if (rc != B2KV_OK) return rc;
    if (!k_rows || !v_rows || !k_pool || !v_pool) return B2KV_ERR_BAD_ARG;
    if (!block_table || max_blocks <= 0 || block_size <= 0 || n_blocks <= 0) return B2KV_ERR_BAD_ARG;
    if (n_rows <= 0 || first_pos < 0 || static_cast<long long>(first_pos) + n_rows > static_cast<long long>(max_blocks) * block_size)
        return B2KV_ERR_BAD_ARG;
    if (src_first < 0 || src_first + n_rows > src_rows_per_seq) return B2KV_ERR_BAD_ARG;
    if (!aligned16(k_rows) || !aligned16(v_rows) || !aligned16(k_pool) || !aligned16(v_pool)) return B2KV_ERR_ALIGN;
    if (B > 65535) return B2KV_ERR_UNSUPPORTED;
    RowMap m{nullptr, 0, block_table, max_blocks, block_size, n_blocks, stride_blk, stride_t, stride_h, 0, dev_status};
    const int es = elt_bytes(dtype);
    const int chunks = H * D * es / 16;
    const int shift = es == 4 ? 2 : 3;
    int threads = (chunks + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    append_rows_kernel<<<dim3(n_rows, B), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(k_rows), static_cast<const uint4*>(v_rows), static_cast<uint4*>(k_pool),
        static_cast<uint4*>(v_pool), m, src_rows_per_seq, src_first, first_pos, H, D, chunks, shift);
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

}  // namespace b2kv

using namespace b2kv;

extern "C" {

int b2kv_append(const void* new_k, const void* new_v, void* k_cache, void* v_cache, int32_t* seq_pos, int pos,
                int advance, int B, int H, int D, int T_max, int64_t stride_b, int64_t stride_t, int64_t stride_h,
                int dtype, int32_t* dev_status, void* stream) {
    int rc = check_common(B, H, D, dtype, stride_b, stride_t, stride_h);
    if (rc != B2KV_OK) return rc;
    if (T_max <= 0) return B2KV_ERR_BAD_ARG;
    if (seq_pos == nullptr && (pos < 0 || pos >= T_max)) return B2KV_ERR_BAD_ARG;
    RowMap m{seq_pos, pos, nullptr, 0, 0, 0, stride_b, stride_t, stride_h, T_max, dev_status};
    return launch_append(new_k, new_v, k_cache, v_cache, m, seq_pos, advance, B, H, D, dtype, stream);
}

int b2kv_append_paged(const void* new_k, const void* new_v, void* k_pool, void* v_pool, int32_t* seq_pos, int pos,
                      int advance, const int32_t* block_table, int max_blocks, int block_size, int n_blocks, int B,
                      int H, int D, int64_t stride_blk, int64_t stride_t, int64_t stride_h, int dtype,
                      int32_t* dev_status, void* stream) {
    int rc = check_common(B, H, D, dtype, stride_blk, stride_t, stride_h);
    if (rc != B2KV_OK) return rc;
    if (!block_table || max_blocks <= 0 || block_size <= 0 || n_blocks <= 0) return B2KV_ERR_BAD_ARG;
    if (seq_pos == nullptr && (pos < 0 || pos >= max_blocks * block_size)) return B2KV_ERR_BAD_ARG;
    RowMap m{seq_pos, pos, block_table, max_blocks, block_size, n_blocks, stride_blk, stride_t, stride_h, 0, dev_status};
    return launch_append(new_k, new_v, k_pool, v_pool, m, seq_pos, advance, B, H, D, dtype, stream);
}

int b2kv_advance_lengths(int32_t* seq_lens, int B, int delta, void* stream) {
    if (seq_lens == nullptr || B <= 0) return B2KV_ERR_BAD_ARG;
    const int threads = std::min(1024, (B + 31) / 32 * 32);
    OverlapLaunch launch((B + threads - 1) / threads, threads, 0, stream);
    B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, advance_kernel, seq_lens, B, delta));
    return B2KV_OK;
}

int b2kv_append_rows_paged(const void* k_rows, const void* v_rows, void* k_pool, void* v_pool, const int32_t* block_table,
                           int max_blocks, int block_size, int n_blocks, int B, int n_rows, int first_pos, int H, int D,
                           int64_t stride_blk, int64_t stride_t, int64_t stride_h, int dtype, int32_t* dev_status,
                           void* stream) {
    return append_rows_paged_from(k_rows, v_rows, k_pool, v_pool, block_table, max_blocks, block_size, n_blocks, B, n_rows,
                                  first_pos, n_rows, 0, H, D, stride_blk, stride_t, stride_h, dtype, dev_status, stream);
}

int b2kv_gather(const void* cache, void* out, const int32_t* seq_lens, int len, int B, int H, int D, int T_out,
                int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype, void* stream) {
    int rc = check_common(B, H, D, dtype, stride_b, stride_t, stride_h);
    if (rc != B2KV_OK) return rc;
    RowMap m{seq_lens, len, nullptr, 0, 0, 0, stride_b, stride_t, stride_h, T_out, nullptr};
    return launch_gather(cache, out, m, B, H, D, T_out, dtype, stream);
}

int b2kv_gather_paged(const void* pool, void* out, const int32_t* seq_lens, int len, const int32_t* block_table,
                      int max_blocks, int block_size, int n_blocks, int B, int H, int D, int T_out, int64_t stride_blk,
                      int64_t stride_t, int64_t stride_h, int dtype, int32_t* dev_status, void* stream) {
    int rc = check_common(B, H, D, dtype, stride_blk, stride_t, stride_h);
    if (rc != B2KV_OK) return rc;
    if (!block_table || max_blocks <= 0 || block_size <= 0 || n_blocks <= 0) return B2KV_ERR_BAD_ARG;
    RowMap m{seq_lens, len, block_table, max_blocks, block_size, n_blocks, stride_blk, stride_t, stride_h, 0, dev_status};
    return launch_gather(pool, out, m, B, H, D, T_out, dtype, stream);
}

}  // extern "C"
