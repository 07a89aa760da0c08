/*
 * b2kv - C ABI of the B200 (sm_100a) KV-cache attention kernels.
 *
 * These entry points take the place of the reference's WGSL dispatch
 * (batch_add(ctx, kernel_source, params, buffers, workgroups...),
 * simple-llm/src/gpu/gpu_ops.py:253-316) for the three operations of its KV-cache
 * path.  Every argument is a plain device pointer, an integer or a stream handle;
 * the library allocates nothing, keeps no pointer after a call returns, and
 * launches asynchronously on the stream it is given (stream order takes the place
 * of batch_begin / batch_commit, gpu_ops.py:226-250 and :343-360).
 *
 * Conventions
 *   dtype        B2KV_DTYPE_F32 (the reference's only type) or B2KV_DTYPE_BF16
 *                (storage type of q / k / v / caches / outputs; arithmetic is fp32).
 *   cache layout element (b, t, h, d) lives at  b*stride_b + t*stride_t + h*stride_h + d
 *                (strides in ELEMENTS, d contiguous).  The reference layout
 *                [B*T_max, H*D] (gpu_kernels.py:2791-2796, :2858-2859) is
 *                stride_b = T_max*H*D, stride_t = H*D, stride_h = D; the layout that
 *                streams best on B200, [B, H, T_max, D], is stride_b = H*T_max*D,
 *                stride_h = T_max*D, stride_t = D.
 *   paged layout pools hold blocks of block_size tokens; token t of sequence b lives in
 *                block  block_table[b*max_blocks + t/block_size]  at
 *                blk*stride_blk + (t % block_size)*stride_t + h*stride_h + d.
 *   lengths      seq_lens / seq_pos are int32 device arrays of B entries, or NULL to
 *                use the single host integer (the reference's one current_len).
 *   alignment    every pointer 16-byte aligned, D*sizeof(element) a multiple of 16,
 *                every stride*sizeof(element) a multiple of 16.
 *   stream       a cudaStream_t passed as void* (NULL = the legacy default stream).
 *   overlap      the kernels of a decode step (append, Q/K/V projection, decode, row products,
 *                layernorm, length advance) are launched with programmatic stream
 *                serialisation: each may be scheduled while the kernel before it in the
 *                stream is still running, sets itself up (and streams the first weight
 *                tiles, which no kernel writes), and waits for that kernel to complete
 *                before it reads anything else or writes at all.  Results are those of
 *                plain stream order; b2kv_tune("serial_launches", 1) switches it off.
 *   return       0 on success, a negative B2KV_ERR_* code otherwise; nothing is
 *                launched when an argument check fails.
 *   dev_status   optional int32 device word (NULL to skip).  A kernel that detects a
 *                block-table entry outside [0, n_blocks), a position outside the cache
 *                or a wait that ran out stores a non-zero B2KV_DEV_* code there and
 *                skips the access instead of faulting.  The caller zeroes and reads it.
 */
#ifndef B2KV_H
#define B2KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2KV_DTYPE_F32 0
#define B2KV_DTYPE_BF16 1

#define B2KV_OK 0
#define B2KV_ERR_BAD_ARG (-1)     /* NULL pointer, non-positive dimension, inconsistent sizes */
#define B2KV_ERR_ALIGN (-2)       /* pointer or stride not 16-byte aligned                   */
#define B2KV_ERR_UNSUPPORTED (-3) /* head_dim / dtype / block_size combination not compiled  */
#define B2KV_ERR_WORKSPACE (-4)   /* workspace missing or smaller than *_workspace_bytes     */
#define B2KV_ERR_CUDA (-5)        /* a CUDA runtime call failed; see b2kv_last_cuda_error    */
#define B2KV_ERR_STATIC_LIMIT (-6) /* b2kv_decode_static: the problem needs more scratch than
                                      B2KV_STATIC_SCRATCH_BYTES                               */

#define B2KV_DEV_BAD_BLOCK 1    /* block-table entry outside the pool           */
#define B2KV_DEV_BAD_POSITION 2 /* append position outside [0, T_max)           */
#define B2KV_DEV_WAIT_TIMEOUT 3 /* a bounded wait on a barrier ran out          */
#define B2KV_DEV_BAD_TOKEN 4    /* token id outside the embedding table         */

/* Text for a return code.  Replaces the reference's exception messages at the C level. */
const char* b2kv_strerror(int status);
/* Text of the last CUDA runtime error seen by this library in the calling thread. */
const char* b2kv_last_cuda_error(void);
/* ABI version, bumped when a signature changes. */
int b2kv_version(void);

/*
 * KV-cache append.  Replaces kv_cache_update's dispatch
 * (simple-llm/src/gpu/gpu_kv_cache.py:161-184, kernel gpu_kernels.py:2725-2798):
 * copies new_k / new_v [B, H*D] into the cache rows at position seq_pos[b]
 * (or `pos` for every sequence when seq_pos is NULL).  Bit-exact copy with 16-byte
 * vector stores.  The host owns the single current_len; with per-sequence positions and
 * advance != 0 the kernel adds one to seq_pos[b] after the row is written (the device-side
 * form of "cache.current_len += 1", gpu_kv_cache.py:186).
 */
int b2kv_append(const void* new_k, const void* new_v, void* k_cache, void* v_cache, int32_t* seq_pos, int pos,
                int advance, int B, int H, int D, int T_max, int64_t stride_b, int64_t stride_t, int64_t stride_h,
                int dtype, int32_t* dev_status, void* stream);

/* Paged variant of b2kv_append (block table, no counterpart in the reference: its cache is
 * one contiguous buffer per layer, gpu_kv_cache.py:66-78). */
int b2kv_append_paged(const void* new_k, const void* new_v, void* k_pool, void* v_pool, int32_t* seq_pos, int pos,
                      int advance, const int32_t* block_table, int max_blocks, int block_size, int n_blocks, int B,
                      int H, int D, int64_t stride_blk, int64_t stride_t, int64_t stride_h, int dtype,
                      int32_t* dev_status, void* stream);

/*
 * seq_lens[b] += delta for b < B, in stream order: the length bookkeeping of a ragged cache after an append that did
 * not advance it (b2kv_qkv_append; b2kv_append with advance = 0).  The reference keeps one host-side current_len
 * and adds one in kv_cache_update (simple-llm/src/gpu/gpu_kv_cache.py:186); per-sequence device lengths have no
 * counterpart there.
 */
int b2kv_advance_lengths(int32_t* seq_lens, int B, int delta, void* stream);

/*
 * A whole prompt into a paged cache: rows [b * n_rows + i] of k_rows / v_rows ([B * n_rows, H * D], the layout
 * flash_attention takes its K and V in, simple-llm/src/gpu/gpu_pass_forward.py:497-509) go to position
 * first_pos + i of sequence b through the block table.  No counterpart in the reference (its cache is
 * contiguous and filled one token per kv_cache_update call, gpu_kv_cache.py:113-186); it is what the fused
 * cache write of b2kv_prefill does for a contiguous cache.  No length is advanced.
 */
int b2kv_append_rows_paged(const void* k_rows, const void* v_rows, void* k_pool, void* v_pool, const int32_t* block_table,
                           int max_blocks, int block_size, int n_blocks, int B, int n_rows, int first_pos, int H, int D,
                           int64_t stride_blk, int64_t stride_t, int64_t stride_h, int dtype, int32_t* dev_status,
                           void* stream);

/*
 * Cache gather: writes the logical view out[B, T_out, H, D] (contiguous) of the first
 * seq_lens[b] (or `len`) rows of every sequence, zero beyond.  The reference reads caches
 * back with gpu_buffer_2d_read (simple-llm/src/gpu/gpu_buffer.py:198-208), which only
 * works for its own layout; this is the layout-independent equivalent used for bit-exact
 * append / gather checks.
 */
int b2kv_gather(const void* cache, void* out, const int32_t* seq_lens, int len, int B, int H, int D, int T_out,
                int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype, void* stream);
int b2kv_gather_paged(const void* pool, void* out, const int32_t* seq_lens, int len, const int32_t* block_table,
                      int max_blocks, int block_size, int n_blocks, int B, int H, int D, int T_out, int64_t stride_blk,
                      int64_t stride_t, int64_t stride_h, int dtype, int32_t* dev_status, void* stream);

/*
 * Single-token decode attention over the cache.  Replaces attention_with_kv_cache's
 * dispatch (simple-llm/src/gpu/gpu_kv_cache.py:266-289, kernel gpu_kernels.py:2801-2938):
 * out[b, h, :] = softmax(q[b, h, :] . K[b, 0:n_b, h, :]^T / sqrt(D)) . V[b, 0:n_b, h, :]
 * with n_b = (seq_lens ? seq_lens[b] : len) + len_bias, clamped to [0, T_upper].
 * q, out are [B, H*D].  Sequences with n_b == 0 produce zeros.  The reference's limit of
 * 256 cached tokens (gpu_kv_cache.py:250-257) does not exist here: the cache is
 * processed split-K (flash decoding: the caches of all (sequence, head) pairs are cut into chunks,
 * one large chunk per CTA and small ones that a CTA takes from a counter when it has finished
 * what it had) and the partial results of a (sequence, head) are merged by the CTA that finishes
 * its last piece.  T_upper is a host-side upper bound of every n_b (at most T_max); it
 * bounds the lengths read from the device and the size of the launch.  len_bias lets a caller attend over "length after
 * this step's append" without a separate increment of the device lengths.
 * `workspace` is scratch of at least b2kv_decode_workspace_bytes(...) bytes; it needs no
 * initialisation and carries nothing between calls.
 */
size_t b2kv_decode_workspace_bytes(int B, int H, int D, int T_upper, int dtype);
int b2kv_decode(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* seq_lens, int len,
                int len_bias, int B, int H, int D, int T_upper, int64_t stride_b, int64_t stride_t, int64_t stride_h,
                int dtype, void* workspace, size_t workspace_bytes, int32_t* dev_status, void* stream);
int b2kv_decode_paged(const void* q, const void* k_pool, const void* v_pool, void* out, const int32_t* seq_lens,
                      int len, int len_bias, const int32_t* block_table, int max_blocks, int block_size, int n_blocks,
                      int B, int H, int D, int T_upper, int64_t stride_blk, int64_t stride_t, int64_t stride_h,
                      int dtype, void* workspace, size_t workspace_bytes, int32_t* dev_status, void* stream);

/*
 * Decode attention of the head-split configuration fused with the all-gather of its outputs.
 * No counterpart in the reference (which is single-device).  Rank r of `world` ranks holds heads
 * [r*H_local, (r+1)*H_local) of every sequence.  The decode kernel itself stores each output row - from
 * the warp of the CTA that finishes the row - straight into the [B, H_total*D] output buffers of ALL
 * ranks (peer_out[w], peer-mapped device memory, plain stores over NVLink) at this rank's head offset;
 * the last CTA of the launch to finish then writes `epoch` into word `rank` of every rank's flag array
 * (peer_flags[w]).  A final one-warp kernel waits, with
 * a bound of about two seconds, until all `world` words of this rank's own flags (my_flags) have
 * reached `epoch`; after it, peer_out[rank] holds the outputs of all heads, in stream order.
 * (my_flags == NULL queues no wait kernel: the caller then orders the consumption itself.)
 *   peer_out, peer_flags  device arrays of `world` pointers (the same on every rank up to
 *                         address translation); flags are uint32[world], zeroed once.
 *   counter, counter_target  not used any more (the CTAs count themselves in on a word of the
 *                         workspace); kept so that callers need not change.  epoch = number of
 *                         this call, starting at 1.
 * Use two output buffers alternately (by epoch parity): a rank may be one call ahead of a peer
 * that still reads the previous result.  A wait that runs out sets B2KV_DEV_WAIT_TIMEOUT in
 * dev_status and returns; nothing spins for ever.
 */
int b2kv_decode_allgather(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens, int len,
                          int len_bias, int B, int H_local, int D, int T_upper, int64_t stride_b, int64_t stride_t,
                          int64_t stride_h, int dtype, void* workspace, size_t workspace_bytes, void* const* peer_out,
                          uint32_t* const* peer_flags, const uint32_t* my_flags, uint32_t* counter,
                          uint32_t counter_target, int rank, int world, int H_total, uint32_t epoch,
                          int32_t* dev_status, void* stream);

/*
 * Decode attention over a SLICE of every sequence's tokens, for the sequence-split
 * (context-parallel) configuration in which each rank holds part of a long cache; no counterpart
 * in the reference.  b2kv_decode_partial is b2kv_decode except that it leaves, per (sequence, head),
 * the unnormalised row and its softmax statistics in partial_out (float [B*H, D + 2]: D sums,
 * then the maximum in the log2 domain, -inf for an empty slice, then the sum of weights).
 * b2kv_merge_partials combines R such arrays (parts [R, B*H, D + 2], e.g. all-gathered from R ranks)
 * into the normalised output [B, H*D] of type dtype.
 */
int b2kv_decode_partial(const void* q, const void* k_cache, const void* v_cache, float* partial_out,
                        const int32_t* seq_lens, int len, int len_bias, int B, int H, int D, int T_upper,
                        int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype, void* workspace,
                        size_t workspace_bytes, int32_t* dev_status, void* stream);
int b2kv_merge_partials(const float* parts, int R, int B, int H, int D, void* out, int dtype, void* stream);

/*
 * b2kv_decode without a workspace argument.  It has no counterpart in the reference, whose
 * dispatch layer creates a fresh uniform buffer for every operation
 * (simple-llm/src/gpu/gpu_ops.py:184-203, :298) and so always allocates.
 *
 * Who needs it: a caller that may not allocate device memory at the moment it decodes.  An
 * inference server that handed every free byte of HBM to its KV-cache pool at start-up has
 * nothing left for cudaMalloc to give; a decode loop with a latency budget cannot afford
 * cudaMalloc either, because it synchronises the whole device and takes a process-wide lock.
 * Such callers still pass q, the caches and out, but the split-K partials go to an array
 * of B2KV_STATIC_SCRATCH_BYTES bytes that is part of the library image: every GPU whose
 * context loads the library holds that much memory until the process exits.  The call itself
 * performs no cudaMalloc / cudaFree and calls no allocating routine.
 *
 * Limits and rules:
 *   - Shapes whose partials do not fit are refused with B2KV_ERR_STATIC_LIMIT before anything is
 *     launched; use b2kv_decode with your own workspace for those.  The partials take
 *     2 * (10 * CTAs + 2) + B * H slots of (D + 2) * 4 bytes (two per chunk of work that the
 *     launch may cut the caches into, one per (sequence, head)), plus 8 bytes per (sequence,
 *     head) for the tickets and 8 for the chunk counter, where CTAs is the persistent grid:
 *     the SM count times the resident CTAs per SM of the compiled variant (two for 256-byte
 *     rows, at most four for any row size), and never more than the tiles of work.  The
 *     benchmark shape (B=64, H=32, D=128, bf16; 296 CTAs on a 148-SM B200) needs 7972 slots
 *     = 4.1 MB and fits; B=4096 with the same heads does not.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current).  Make that first call before starting
 *     any stream capture on that device.
 *   - All calls on one device share the one array and it keeps whatever the previous call left
 *     in it.  Nothing in it has to start at zero: a call writes every partial before any CTA
 *     reads it, and the per-(sequence, head) tickets that decide who merges carry the number of
 *     the launch, so what an earlier call left behind never counts.  But two calls that overlap
 *     on the GPU (different streams, no ordering between them) race on it: keep calls on one
 *     device in stream order.
 *   - Contiguous caches only (no block table).  Results are bit-identical to b2kv_decode.
 */
#define B2KV_STATIC_SCRATCH_BYTES (32u << 20)
int b2kv_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* seq_lens,
                       int len, int len_bias, int B, int H, int D, int T_upper, int64_t stride_b, int64_t stride_t,
                       int64_t stride_h, int dtype, int32_t* dev_status, void* stream);

/*
 * Causal flash-attention prefill.  Replaces flash_attention's dispatch
 * (simple-llm/src/gpu/gpu_pass_forward.py:557-588, kernel gpu_kernels.py:499-770).
 * Q, K, V, O are [B*N, H*D]; L and M (float, [B*N*H], index b*N*H + row*H + h, either may
 * be NULL) receive the softmax row sums and row maxima of the scaled scores as the
 * reference kernel writes them (gpu_kernels.py:762-768).  Key j is visible to query i when
 * j <= i.  When k_cache / v_cache are non-NULL the kernel also writes K / V rows 0..N-1 of
 * every sequence into the caches (same dtype, layout given by the cache strides), which
 * the reference can only do one token at a time through kv_cache_update.
 * bf16 with D == 128 or 64 runs on the tcgen05 tensor cores; other shapes run on a SIMT kernel.
 * A tensor-core kernel whose bounded barrier wait ran out stores B2KV_DEV_WAIT_TIMEOUT in dev_status
 * (the output of that launch is then incomplete).
 */
int b2kv_prefill(const void* Q, const void* K, const void* V, void* O, float* L, float* M, void* k_cache,
                 void* v_cache, int64_t stride_b, int64_t stride_t, int64_t stride_h, int T_max, int B, int N, int H,
                 int D, int dtype, int32_t* dev_status, void* stream);

/*
 * b2kv_prefill with a scratch buffer, which lets fp32 prompts (the reference's storage type) of head_dim 128 or 64 run
 * on the tensor cores as well: Q, K and V are split into two bfloat16 halves each (x = hi + lo, 16 mantissa bits kept)
 * in the scratch, every product becomes three MMAs into fp32 accumulators (the dropped lo * lo term is below 2^-16
 * relative), softmax and outputs stay fp32; results agree with the fp32 oracle within rtol 1e-4 and atol 3e-5
 * on outputs of order one (the SIMT kernel, which b2kv_prefill takes for fp32, holds atol 1e-5).  b2kv_prefill_workspace_bytes gives the scratch size, 0 where scratch buys nothing (bf16
 * prompts, other head_dims, prompts shorter than 128 tokens): the call then is b2kv_prefill.  The scratch needs no
 * initialisation and carries nothing between calls.  With a cache the K / V rows are written by a copy kernel behind the
 * attention.
 */
size_t b2kv_prefill_workspace_bytes(int B, int N, int H, int D, int dtype);
int b2kv_prefill_ws(const void* Q, const void* K, const void* V, void* O, float* L, float* M, void* k_cache, void* v_cache,
                    int64_t stride_b, int64_t stride_t, int64_t stride_h, int T_max, int B, int N, int H, int D, int dtype,
                    void* workspace, size_t workspace_bytes, int32_t* dev_status, void* stream);

/*
 * b2kv_prefill into a PAGED cache (no counterpart in the reference, whose cache is contiguous): the prompt's K / V
 * rows 0..N-1 of sequence b go to the pool blocks that block_table[b, :] names, addressed as in b2kv_append_paged.
 * On the tensor-core path (bf16, D == 128 or 64) the attention kernel stores every whole block itself from its
 * shared-memory tiles when block_size is a multiple of 8 that divides 128 or is a multiple of 128; a last, partly
 * filled block, other block sizes and the SIMT path are written by a copy kernel behind the attention.  No row past
 * N - 1 is written and no length is advanced.  A table entry outside [0, n_blocks) is skipped and recorded in
 * dev_status (B2KV_DEV_BAD_BLOCK).
 */
int b2kv_prefill_paged(const void* Q, const void* K, const void* V, void* O, float* L, float* M, void* k_pool, void* v_pool,
                       const int32_t* block_table, int max_blocks, int block_size, int n_blocks, int64_t stride_blk,
                       int64_t stride_t, int64_t stride_h, int B, int N, int H, int D, int dtype, int32_t* dev_status,
                       void* stream);

/*
 * The tail of a cached generation step, fp32 like the reference's buffers.  Each replaces one
 * dispatch of simple-llm/src/gpu/gpu_pass_forward.py:
 *   b2kv_layernorm            layernorm :140-176 (WGSL src/gpu/gpu_kernels.py:137-249): per row of
 *                             [n_rows, size], (x - mean) / sqrt(var + epsilon) * gamma + beta, var = mean
 *                             of (x - mean)^2; epsilon is GPUConfig.layernorm_epsilon (gpu_types.py:197).
 *   b2kv_extract_last_tokens  extract_last_tokens :285-328 (WGSL :839-887): row b*seq_len + seq_len - 1
 *                             of [batch_size*seq_len, embedding_dim] to row b of [batch_size, embedding_dim].
 *   b2kv_softmax              softmax :462-494 (WGSL :890-992): exp(x - max) / sum over each row.
 *   b2kv_argmax               greedy choice of the next token, int32 index per row (lowest index among
 *                             equal maxima); the reference does this on the host after reading the
 *                             probabilities back (src/generate.py).
 * Pointers are device pointers, 16-byte aligned; the calls are asynchronous on `stream`.
 */
int b2kv_layernorm(const float* x, const float* gamma, const float* beta, float* out, int64_t n_rows, int size,
                   float epsilon, void* stream);
/* b2kv_layernorm on bf16 rows and bf16 gamma / beta (fp32 arithmetic): extension for bf16 decoder layers. */
int b2kv_layernorm_bf16(const void* x, const void* gamma, const void* beta, void* out, int64_t n_rows, int size,
                        float epsilon, void* stream);
int b2kv_extract_last_tokens(const float* in, float* out, int batch_size, int seq_len, int embedding_dim, void* stream);
int b2kv_softmax(const float* logits, float* probs, int64_t n_rows, int size, void* stream);
int b2kv_argmax(const float* x, int32_t* out, int n_rows, int size, void* stream);
/* b2kv_extract_last_tokens and b2kv_argmax on bf16 rows (embedding_dim a multiple of 8): extensions for a bf16
 * decoder whose hidden rows and logits are bf16. */
int b2kv_extract_last_tokens_bf16(const void* in, void* out, int batch_size, int seq_len, int embedding_dim, void* stream);
int b2kv_argmax_bf16(const void* x, int32_t* out, int n_rows, int size, void* stream);

/*
 * Embedding lookup with the positional encoding added.  Replaces embedding's dispatch
 * (simple-llm/src/gpu/gpu_pass_forward.py:84-137, kernel src/gpu/gpu_kernels.py:384-449):
 *   out[b*seq_len + s, :] = table[input_ids[b*seq_len + s], :] + pos_encoding[start_b + s, :]
 * table is [vocab_size, embedding_dim], pos_encoding [context_size, embedding_dim], out [batch_size*seq_len,
 * embedding_dim], all of `dtype` (fp32 as in the reference, or bf16 with the sum rounded once); input_ids int32.
 * The reference always starts at position 0 (start_b = 0: pass seq_pos = NULL, pos0 = 0).  Extension for a cached
 * decode step, whose one new token per sequence sits at that sequence's current length: start_b = seq_pos[b]
 * (int32 device array, e.g. the cache's lengths) or the host integer pos0.  embedding_dim a multiple of 8.  A token
 * id outside the table or a position outside the encoding is clamped and recorded in dev_status
 * (B2KV_DEV_BAD_TOKEN / B2KV_DEV_BAD_POSITION).
 */
int b2kv_embedding(const void* table, const void* pos_encoding, const int32_t* input_ids, const int32_t* seq_pos, int pos0,
                   void* out, int batch_size, int seq_len, int embedding_dim, int vocab_size, int context_size, int dtype,
                   int32_t* dev_status, void* stream);

/*
 * Q / K / V projection of one decode step fused with the cache append (bf16 storage, fp32 accumulate).
 * Replaces, for the rows of one decode step, the three matmul dispatches of the attention block
 * (simple-llm/src/wgpu_backend.py:812-831; gpu_pass_forward.py:35-82, C = A @ B) followed by
 * kv_cache_update (gpu_kv_cache.py:113-186):
 *   q_out[b, :]                = x[b, :] @ wq
 *   k_cache row (b, position)  = x[b, :] @ wk      (same for v_cache with wv)
 * x is [B, E], the weights are [E, E] row-major ([in, out], as the reference stores them), q_out is
 * [B, E]; position = seq_pos[b] when seq_pos is non-NULL, else `pos`; the cache is addressed with the
 * strides of b2kv_append.  E = H * D, E a multiple of 128, B <= 128.  The lengths are not advanced.
 */
int b2kv_qkv_append(const void* x, const void* wq, const void* wk, const void* wv, void* q_out, void* k_cache,
                    void* v_cache, const int32_t* seq_pos, int pos, int B, int E, int H, int D, int T_max,
                    int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype, int32_t* dev_status, void* stream);

/*
 * out[b, :] = act(x[b, :] @ w + bias) + residual[b, :] for the few rows of a decode step: x [B, K], w [K, N]
 * row-major, bias [N] (nullable), residual (nullable) and out [B, N]; activation 0 = none, 1 = the reference's GELU
 * x * sigmoid(1.702 x) (src/gpu/gpu_kernels.py:285-293); bf16 with fp32 accumulation, B <= 128, K and N multiples
 * of 128.  Replaces the reference's matmul dispatch (simple-llm/src/gpu/gpu_pass_forward.py:35-82, C = A @ B)
 * for the attention output projection and the MLP of a cached decode step (src/wgpu_backend.py:857-930), together
 * with the bias_add (:211-248), gelu (:179-209) and residual_add (:250-283) dispatches that follow it there.
 * Same kernel as b2kv_qkv_append (the weights are streamed once through the tensor cores).
 */
int b2kv_matmul_rows(const void* x, const void* w, const void* bias, const void* residual, void* out, int B, int K, int N,
                     int activation, int dtype, void* stream);

/*
 * out = act(a @ w + bias) + residual for any number of rows: a [M, K], w [K, N] row-major ([in, out], as the
 * reference stores its weights), bias [N] (nullable), residual (nullable) and out [M, N]; activation as in
 * b2kv_matmul_rows; bf16 with fp32 accumulation, K and N multiples of 8.  Replaces the reference's matmul
 * dispatch (simple-llm/src/gpu/gpu_pass_forward.py:35-82, C = A @ B; kernel src/gpu/gpu_kernels.py:10-134) for
 * the prompt-side projections either side of flash_attention (src/wgpu_backend.py:812-930), with the bias_add
 * (:211-248), gelu (:179-209) and residual_add (:250-283) dispatches that follow it there.  A persistent
 * tensor-core kernel over 128 x 256 output tiles; for at most 128 rows b2kv_matmul_rows streams the weights
 * faster.  A bounded barrier wait that ran out stores B2KV_DEV_WAIT_TIMEOUT in dev_status (the output of that
 * launch is then incomplete).
 */
int b2kv_matmul(const void* a, const void* w, const void* bias, const void* residual, void* out, int M, int K, int N,
                int activation, int dtype, int32_t* dev_status, void* stream);

/*
 * Tuning hook for experiments (process-global and unsynchronised: set knobs before launching work, never while
 * another thread is inside a b2kv call): sets an integer knob by name ("decode_variant",
 * "decode_grid_per_sm", "decode_l2_keep", "decode_no_tensor_map", "decode_dynamic_chunks": small chunks of the
 * decode's work handed out on demand, 0 = for long launches only, 1 = always, 2 = never,
 * "prefill_force_simt", "prefill_variant": 2 = CTA-pair prefill kernel for bf16, D = 128,
 * N a multiple of 256, "prefill_f32_simt": 1 = b2kv_prefill_ws never takes the
 * split-bfloat16 tensor-core kernel, "prefill_unfused_paged": 1 = b2kv_prefill_paged always
 * fills the pool with the copy kernel, "prefill_test_expire": 1 = test hook, the softmax warps of the one-CTA tensor-core prefill
 * behave as if their first bounded wait had run out (the launch then ends after about two seconds with
 * B2KV_DEV_WAIT_TIMEOUT in dev_status), "matmul_splits": ranges of input features per tile in b2kv_matmul_rows,
 * "serial_launches": 1 = plain stream order for every launch (see "overlap" at the top),
 * "gemm_variant": 1 = one CTA per output tile, 2 / 3 = CTA pairs with 64 / 128 input features per
 * ring stage in b2kv_matmul);
 * returns B2KV_ERR_BAD_ARG
 * for an unknown name.  Defaults are chosen per shape when a knob is 0.  No counterpart in
 * the reference beyond the tile-size fields of GPUConfig (gpu_types.py:69-121).
 */
int b2kv_tune(const char* name, int value);

#ifdef __cplusplus
}
#endif

#endif /* B2KV_H */
