/*
 * CPU oracle (C + OpenMP) for the KV-cache attention path.  TEST INFRASTRUCTURE ONLY.
 *
 * A restatement of the reference's arithmetic for this path, used as the checker
 * for the CUDA kernels at sizes where the numpy oracle (kv_oracle.py) is too slow,
 * and as the timed CPU baseline of the benchmark.  The product library never links
 * or loads it.
 *
 * What each function follows (paths inside the reference project):
 *   kvo_append        simple-llm/src/gpu/gpu_kernels.py:2784-2796  (row copy, index math)
 *   kvo_decode        simple-llm/src/gpu_test.py:2328-2367         (per (b,h): scores =
 *                     q.K^T * 1/sqrt(D); max-subtracted exp; divide by the sum; weights.V)
 *                     and the shader simple-llm/src/gpu/gpu_kernels.py:2846-2936
 *   kvo_prefill       simple-llm/src/gpu_test.py:794-810 (dense causal softmax; masked
 *                     entries are exactly zero after exp(-1e10 - m)) with the L / M
 *                     statistics and their layout of gpu_kernels.py:762-768
 *
 * Accumulation: dot products and sums are carried in double and rounded to float
 * once; the reference accumulates in float.  The difference is far inside the
 * tolerances used (1e-4 relative for fp32).  Storage types: 0 = float32,
 * 1 = bfloat16 bits in uint16 (an extension; the reference is float32 only).
 * Element (b, t, h, d) of a cache lives at  b*sb + t*st + h*sh + d  (elements), so
 * the reference layout [B*T_max, H*D] is sb = T_max*H*D, st = H*D, sh = D.
 * With a block table, b*sb + t*st is replaced by  blk*sblk + (t % bs)*st  with
 * blk = block_table[b*max_blocks + t/bs].
 *
 * Parity pin: see the header of kv_oracle.py; tests/test_oracle.py checks this file
 * against the fixtures produced from the reference's own test code.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float load_elt(const void* base, int64_t idx, int dtype) {
    if (dtype == 0) return ((const float*)base)[idx];
    uint32_t u = ((uint32_t)((const uint16_t*)base)[idx]) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline size_t elt_size(int dtype) { return dtype == 0 ? 4 : 2; }

/* sum_d qf[d] * row[d], carried in double. */
static inline double dot_row(const float* qf, const void* base, int64_t off, int D, int dtype) {
    double dot = 0.0;
    if (dtype == 0) {
        const float* r = (const float*)base + off;
#pragma omp simd reduction(+ : dot)
        for (int d = 0; d < D; ++d) dot += (double)qf[d] * (double)r[d];
    } else {
        const uint16_t* r = (const uint16_t*)base + off;
#pragma omp simd reduction(+ : dot)
        for (int d = 0; d < D; ++d) {
            uint32_t u = ((uint32_t)r[d]) << 16;
            float f;
            memcpy(&f, &u, 4);
            dot += (double)qf[d] * (double)f;
        }
    }
    return dot;
}

/* acc[d] += e * row[d]. */
static inline void axpy_row(double* acc, double e, const void* base, int64_t off, int D, int dtype) {
    if (dtype == 0) {
        const float* r = (const float*)base + off;
#pragma omp simd
        for (int d = 0; d < D; ++d) acc[d] += e * (double)r[d];
    } else {
        const uint16_t* r = (const uint16_t*)base + off;
#pragma omp simd
        for (int d = 0; d < D; ++d) {
            uint32_t u = ((uint32_t)r[d]) << 16;
            float f;
            memcpy(&f, &u, 4);
            acc[d] += e * (double)f;
        }
    }
}

int kvo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void kvo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Row offset (in elements) of token t of sequence b, contiguous or paged. */
static inline int64_t row_base(int b, int64_t t, int64_t sb, int64_t st, const int32_t* block_table,
                               int max_blocks, int block_size, int64_t sblk) {
    if (!block_table) return (int64_t)b * sb + t * st;
    int64_t blk = block_table[(int64_t)b * max_blocks + t / block_size];
    return blk * sblk + (t % block_size) * st;
}

/* new_k/new_v [B, H*D] -> cache rows at pos[b] (pos_arr) or at the one position pos. */
void kvo_append(const void* new_k, const void* new_v, void* k_cache, void* v_cache, const int32_t* pos_arr,
                int pos, int B, int H, int D, int64_t sb, int64_t st, int64_t sh, int dtype,
                const int32_t* block_table, int max_blocks, int block_size, int64_t sblk) {
    size_t es = elt_size(dtype);
    for (int b = 0; b < B; ++b) {
        int64_t t = pos_arr ? pos_arr[b] : pos;
        int64_t base = row_base(b, t, sb, st, block_table, max_blocks, block_size, sblk);
        for (int h = 0; h < H; ++h) {
            const char* sk = (const char*)new_k + ((size_t)b * H * D + (size_t)h * D) * es;
            const char* sv = (const char*)new_v + ((size_t)b * H * D + (size_t)h * D) * es;
            memcpy((char*)k_cache + (size_t)(base + h * sh) * es, sk, D * es);
            memcpy((char*)v_cache + (size_t)(base + h * sh) * es, sv, D * es);
        }
    }
}

/* q [B, H*D] (dtype), out float [B, H*D]; lens_arr[b] (or the one length len) valid rows. */
void kvo_decode(const void* q, const void* k_cache, const void* v_cache, float* out, const int32_t* lens_arr,
                int len, int B, int H, int D, int64_t sb, int64_t st, int64_t sh, int dtype,
                const int32_t* block_table, int max_blocks, int block_size, int64_t sblk) {
    const float scale = (float)(1.0 / sqrt((double)D));
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; ++b) {
        for (int h = 0; h < H; ++h) {
            int64_t n = lens_arr ? lens_arr[b] : len;
            float* o = out + ((size_t)b * H + h) * D;
            for (int d = 0; d < D; ++d) o[d] = 0.0f;
            if (n <= 0) continue;
            float* qf = (float*)malloc(sizeof(float) * D);
            float* s = (float*)malloc(sizeof(float) * n);
            double* acc = (double*)calloc(D, sizeof(double));
            for (int d = 0; d < D; ++d) qf[d] = load_elt(q, ((int64_t)b * H + h) * D + d, dtype);
            float m = -INFINITY;
            for (int64_t t = 0; t < n; ++t) {
                int64_t base = row_base(b, t, sb, st, block_table, max_blocks, block_size, sblk) + h * sh;
                s[t] = (float)dot_row(qf, k_cache, base, D, dtype) * scale;
                if (s[t] > m) m = s[t];
            }
            double total = 0.0;
            for (int64_t t = 0; t < n; ++t) {
                double e = exp((double)s[t] - (double)m);
                total += e;
                int64_t base = row_base(b, t, sb, st, block_table, max_blocks, block_size, sblk) + h * sh;
                axpy_row(acc, e, v_cache, base, D, dtype);
            }
            for (int d = 0; d < D; ++d) o[d] = (float)(acc[d] / total);
            free(qf);
            free(s);
            free(acc);
        }
    }
}

/* Q, K, V [B*N, H*D] (dtype) -> O float [B*N, H*D]; L, M float [B*N*H] at b*N*H + row*H + h
 * (either may be NULL).  Causal: key j is visible to query i when j <= i. */
void kvo_prefill(const void* Q, const void* K, const void* V, float* O, float* L, float* M, int B, int N, int H,
                 int D, int dtype) {
    const float scale = (float)(1.0 / sqrt((double)D));
    const int64_t E = (int64_t)H * D;
#pragma omp parallel
    {
        float* s = (float*)malloc(sizeof(float) * (size_t)N);
        float* qf = (float*)malloc(sizeof(float) * (size_t)D);
        double* acc = (double*)malloc(sizeof(double) * (size_t)D);
#pragma omp for collapse(3) schedule(dynamic, 8)
        for (int b = 0; b < B; ++b) {
            for (int h = 0; h < H; ++h) {
                for (int i = 0; i < N; ++i) {
                    int64_t qoff = ((int64_t)b * N + i) * E + (int64_t)h * D;
                    for (int d = 0; d < D; ++d) qf[d] = load_elt(Q, qoff + d, dtype);
                    float m = -INFINITY;
                    for (int j = 0; j <= i; ++j) {
                        int64_t koff = ((int64_t)b * N + j) * E + (int64_t)h * D;
                        s[j] = (float)dot_row(qf, K, koff, D, dtype) * scale;
                        if (s[j] > m) m = s[j];
                    }
                    double total = 0.0;
                    for (int d = 0; d < D; ++d) acc[d] = 0.0;
                    for (int j = 0; j <= i; ++j) {
                        double e = exp((double)s[j] - (double)m);
                        total += e;
                        int64_t voff = ((int64_t)b * N + j) * E + (int64_t)h * D;
                        axpy_row(acc, e, V, voff, D, dtype);
                    }
                    double denom = total > 1e-8 ? total : 1e-8;
                    for (int d = 0; d < D; ++d) O[qoff + d] = (float)(acc[d] / denom);
                    int64_t sidx = (int64_t)b * N * H + (int64_t)i * H + h;
                    if (L) L[sidx] = (float)total;
                    if (M) M[sidx] = m;
                }
            }
        }
        free(s);
        free(qf);
        free(acc);
    }
}
