// Single-token decode attention over the KV cache: split-K flash decoding for sm_100a.
//
// The reference kernel (simple-llm/src/gpu/gpu_kernels.py:2801-2938) gives one workgroup
// to each (sequence, head), keeps the whole score vector in workgroup memory (hence its
// 256-token limit) and reads K rows uncoalesced.  Here all (sequence, head) caches of the batch
// are laid end to end in one token space of H * sum(n_b) tokens, which is cut into one equal
// share per CTA of a persistent grid (cuts rounded to whole tiles inside a (sequence, head)), so
// ragged batches stay balanced without any scheduling traffic.  A share may cover the tail of
// one (sequence, head), several whole ones and the head of another; every piece is a work
// item.  Inside a CTA one producer warp streams K/V tiles from HBM into a ring of
// shared-memory stages with bulk copies (TMA, untiled) that complete on mbarriers, and the
// consumer warps fold each tile into an online softmax held in registers.  The producer
// runs ahead across item boundaries, so the copy queue never drains between items.  An item
// that is its whole (sequence, head) writes the output row itself; otherwise it leaves one partial
// (m, l, acc[D]) in the workspace and takes a ticket for its pair, and the CTA that takes the
// pair's last ticket merges the partials and writes the row (nobody waits for another CTA, no
// second launch).  The forms whose merge has more to do (outputs stored into every rank's buffer,
// unnormalised rows for the sequence split) still merge in a small second kernel.
//
// Arithmetic: storage type fp32 or bf16, all math in fp32; scores are kept in the log2
// domain (q is pre-multiplied by log2(e)/sqrt(D)) so that exp is a single ex2.
//
// HBM traffic per launch is the K and V rows of the attended tokens, once:
// sum_b n_b * H * D * 2 * sizeof(element), plus q, out and the partials.
#include <math.h>
#include <string.h>

#include <atomic>
#include <chrono>

#include "b2kv_common.cuh"
#include "tma_map.cuh"

namespace b2kv {

constexpr int kFlagFirst = 1;  // first tile of an item: reset the running softmax, take q
constexpr int kFlagLast = 2;   // last tile of an item: merge the warps and store the partial
constexpr int kFlagDone = 4;   // no more work for this CTA
constexpr int kFlagWhole = 8;  // the item is its whole (sequence, head): no other CTA holds a piece of it

struct StageMeta {
    int slot;   // partial-result slot of the item this tile belongs to
    int ntok;   // valid rows in the tile
    int flags;
    int pieces;          // pieces with tokens that the item's (sequence, head) was cut into, over all CTAs
    long long pair_off;  // where the (sequence, head) starts in the token space
    int len;             // its length
    int bh;              // sequence * H + head
};

// Fused all-gather: instead of writing an output row to a local buffer, the split kernel's merging warps
// store it straight into the output buffers of all ranks (peer memory over NVLink) at this rank's head
// offset, and the last CTA of the launch to finish raises this rank's flag on every rank.
struct GatherInfo {
    void* const* peer_out;        // device array [world]: each rank's [B, h_total * D] output buffer (null = off)
    uint32_t* const* peer_flags;  // device array [world]: each rank's flag words, one per source rank
    const uint32_t* my_flags;     // this rank's own flag words (what the wait kernel watches)
    unsigned int* counter;        // (not used any more: the CTAs count themselves in on a word of the workspace)
    unsigned int counter_target;
    int rank, world, h_total;
    uint32_t epoch;               // value written to the flags by this call
};

struct DecodeParams {
    const void* q;
    const void* k;
    const void* v;
    float* ws_acc;  // [slots, D]
    float* ws_ml;   // [slots, 2]
    const int32_t* seq_lens;
    const int32_t* block_table;
    int32_t* dev_status;
    int len_scalar, len_bias;
    int B, H, T_upper;
    int n_slots;  // partial-result slots in the workspace: two per chunk of the token space
    int max_blocks, block_size, n_blocks;
    int run_len;  // tokens that one bulk copy may cover (contiguous in memory)
    int l2_evict_first;  // 1: K/V copies carry the evict-first L2 policy (each row is read once)
    int use_tensor_map;  // 1: rows of a head are not adjacent in memory (reference layout): a tile is one tiled
                         // TMA load through the kernel's tensor maps instead of one bulk copy per row
    int64_t stride_b, stride_t, stride_h;
    float q_prescale;
    GatherInfo gather;
    float* partial_out;  // non-null: the merge kernel writes (unnormalised row, max, sum) instead of the output
    // Merge inside the split kernel (plain decode only): the CTA that finishes the last piece of a (sequence, head)
    // merges the pair's partials and writes the output row, so that no second launch is needed.
    int merge_inside;                // 1: the split kernel writes the output rows itself; 0: the merge kernel does
    void* fused_out;                 // output [B, H*D] of the storage type for the merge inside, unless the rows go
                                     // to the ranks' buffers (gather.peer_out)
    unsigned long long* ws_done;     // CTAs of the launch that have finished, tagged like ws_counter (fused gather)
    unsigned long long* ws_tickets;  // [B*H]: (low 40 bits of the call number << 24) | pieces of the pair finished in that call
    unsigned long long call_id;      // unique per launch call, 48 bits, never 0: tickets left by other calls never count
                                     // (a finished pair's ticket goes back to 0, for launches replayed from a graph)
    int dynamic_chunks;              // 0: by the size of the batch, 1: always, 2: never hand out small chunks on demand
    unsigned long long* ws_counter;  // (low 40 bits of the call number << 24) | chunks handed out so far in that call;
                                     // back to 0 when the last CTA has asked
};

__device__ __forceinline__ int seq_len_of(const DecodeParams& p, int b) {
    int n = (p.seq_lens ? p.seq_lens[b] : p.len_scalar) + p.len_bias;
    return min(max(n, 0), p.T_upper);
}

// How a launch cuts the batch's token space into chunks (see "work split" below).
struct Geometry {
    long long total;  // tokens in the token space
    long long sa;     // tokens per advance chunk (a multiple of the tile)
    long long a_end;  // where the small chunks begin: min(n_static * sa, total)
    long long sb;     // tokens per small chunk (a multiple of the tile)
    int n_static;     // advance chunks = CTAs
    int n_chunks;     // n_static + small chunks
};

template <typename T, int D, int TILE_T, int STAGES, int NCW>
struct DecodeCfg {
    static constexpr int kRowBytes = D * static_cast<int>(sizeof(T));
    static constexpr int kTileBytes = TILE_T * kRowBytes;
    // K tile, V tile, q row; stages start on 128-byte boundaries (tiled TMA destinations need that)
    static constexpr int kStageBytes = (2 * kTileBytes + kRowBytes + 127) / 128 * 128;
    static constexpr int kChunksPerRow = kRowBytes / 16;
    static constexpr int kLanesPerRow = kChunksPerRow < 32 ? kChunksPerRow : 32;
    static constexpr int kChunksPerLane = kChunksPerRow / kLanesPerRow;
    static constexpr int kRowsPerPass = 32 / kLanesPerRow;
    static constexpr int kRowsPerWarp = TILE_T / NCW;
    static constexpr int kPasses = kRowsPerWarp / kRowsPerPass;
    static constexpr int kBatch = kPasses < 8 ? kPasses : 8;
    static constexpr int kEpc = Elt<T>::kPerChunk;
    static constexpr int kAcc = kChunksPerLane * kEpc;
    static constexpr int kMergeFloats = NCW * (D + 2);
    static constexpr int kThreads = (NCW + 2) * 32;  // consumer warps, the copy warp, the merging warp
    static constexpr size_t kSmemBytes = static_cast<size_t>(STAGES) * kStageBytes + (2 * STAGES + 4) * sizeof(uint64_t) +
                                         (STAGES + 2) * sizeof(StageMeta) + 2 * kMergeFloats * sizeof(float) + sizeof(Geometry) + 8 + 128;
    // CTAs that the shared memory of an SM holds, three at most: the register budget is set to let them in
    static constexpr int kCtasPerSm = (232448 / (kSmemBytes + 1024)) < 1 ? 1 : ((232448 / (kSmemBytes + 1024)) > 3 ? 3 : static_cast<int>(232448 / (kSmemBytes + 1024)));
    static_assert(kRowBytes % 16 == 0, "rows must be whole 16-byte chunks");
    static_assert(kChunksPerRow >= 2, "a row must span at least two lanes");
    static_assert(TILE_T % NCW == 0 && kRowsPerWarp % kRowsPerPass == 0 && kPasses % kBatch == 0, "tile split");
};

// --------------------------------------------------------------------------------------
// work split: chunks of the batch's token space, one large one per CTA and small ones on demand
// --------------------------------------------------------------------------------------
//
// The caches of all (sequence, head) pairs laid end to end are one token space of H * sum_b n_b tokens.
// CTAs that share an SM, and SMs among themselves, do not stream at the same rate (finishing times of equal
// shares were measured 8 % either side of their mean), so equal shares leave most of the machine idle at the
// end.  The first three quarters of the space are therefore dealt out as one chunk per CTA (chunk g = CTA g),
// and the rest as small chunks (a thirty-second of a CTA's equal share) that a CTA takes from a counter when
// it has finished what it had.  Chunk numbers grow with the position in the token space.  Every cut adds a
// piece that has to be merged, so a launch whose equal shares are short (less than 256 tiles: there small chunks
// were measured to cost more than they even out, 227 against 170 us at 79 tiles per CTA) is dealt out whole, as
// equal shares.  Interleaved runs at 319 tiles per CTA: 675 us against 695 us for equal shares (long run,
// power-capped clocks).  Nor do small chunks pay where sequences are long against them: four sequences of
// 131072 tokens and 32 heads ran 1.40 against 1.20 ms, a pair's hundred pieces being merged by one warp at the end.

constexpr int kStaticNum = 3, kStaticDen = 4;  // part of the token space dealt out in advance
constexpr int kChunksPerShare = 32;            // small chunks that an equal share would be cut into
constexpr int kMinChunkTiles = 8;              // a small chunk lasts long enough for the merging warp to keep up
constexpr int kMinDynamicTiles = 256;          // equal shares shorter than this many tiles are dealt out whole
constexpr int kMaxPiecesPerPair = 16;          // ... and so is a batch whose longest sequence spans more small chunks

// Most chunks of any batch for a grid of `n_ctas` (the small part is at most a quarter of the space plus what
// rounding adds, a small chunk at least a thirty-second of an equal share).
__host__ __device__ constexpr int max_chunks(int n_ctas) { return n_ctas * (2 + kChunksPerShare * (kStaticDen - kStaticNum) / kStaticDen) + 2; }

// Every thread of the calling warp takes part (the lengths are summed across the lanes).
__device__ __forceinline__ Geometry geometry_of(const DecodeParams& p, int n_ctas, int tile, int lane) {
    long long sum = 0;
    int longest = 0;
    for (int b = lane; b < p.B; b += 32) {
        const int n = seq_len_of(p, b);
        sum += n;
        longest = max(longest, n);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, off);
        longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, off));
    }
    Geometry ge;
    ge.total = sum * p.H;
    const long long per = (ge.total + n_ctas - 1) / n_ctas;  // an equal share
    ge.sb = ((per + kChunksPerShare - 1) / kChunksPerShare + tile - 1) / tile * tile;
    if (ge.sb < static_cast<long long>(kMinChunkTiles) * tile) ge.sb = static_cast<long long>(kMinChunkTiles) * tile;
    // Small chunks only where they pay: not in a short launch (their extra pieces and requests cost more than they
    // even out), and not where a (sequence, head) would be cut into many of them (its pieces are merged by one
    // warp, one after the other, at the very end).
    const bool on_demand = p.dynamic_chunks == 1 ||
                           (p.dynamic_chunks == 0 && per >= static_cast<long long>(kMinDynamicTiles) * tile &&
                            ge.sb * kMaxPiecesPerPair >= longest);
    ge.sa = ((on_demand ? (per * kStaticNum + kStaticDen - 1) / kStaticDen : per) + tile - 1) / tile * tile;
    if (ge.sa < tile) ge.sa = tile;
    ge.n_static = n_ctas;
    ge.a_end = min(static_cast<long long>(n_ctas) * ge.sa, ge.total);
    ge.n_chunks = n_ctas + static_cast<int>((ge.total - ge.a_end + ge.sb - 1) / ge.sb);
    return ge;
}

__device__ __forceinline__ void chunk_range(const Geometry& ge, long long g, long long& start, long long& end) {
    if (g < ge.n_static) {
        start = min(g * ge.sa, ge.a_end);
        end = min(start + ge.sa, ge.a_end);
    } else {
        start = min(ge.a_end + (g - ge.n_static) * ge.sb, ge.total);
        end = min(start + ge.sb, ge.total);
    }
}

// The chunk that holds position `pos` (< total) of the token space.
__device__ __forceinline__ long long chunk_of(const Geometry& ge, long long pos) {
    return pos < ge.a_end ? pos / ge.sa : ge.n_static + (pos - ge.a_end) / ge.sb;
}

// Where the piece of a (sequence, head) inside chunk g leaves its partial result: a chunk holds at most two
// pieces of pairs that other chunks share, the pair that began before the chunk and the pair that goes on after it.
__device__ __forceinline__ int piece_slot(long long g, long long chunk_start, long long pair_off) {
    return static_cast<int>(2 * g + (pair_off >= chunk_start ? 1 : 0));
}

// The piece [t_begin, t_end) of a (sequence, head) of `len` tokens at `pair_off` in the token
// space that the share [start, end) owns.  Cuts inside the pair are rounded up to whole tiles
// (relative to the pair's first token); the neighbouring share rounds the same cut the same way.
__device__ __forceinline__ void piece_of(long long start, long long end, long long pair_off, int len, int tile,
                                         int& t_begin, int& t_end) {
    long long lo = 0, hi = len;
    if (pair_off < start) lo = (start - pair_off + tile - 1) / tile * tile;
    if (pair_off + len > end) hi = (end - pair_off + tile - 1) / tile * tile;
    if (hi > len) hi = len;
    if (lo > hi) lo = hi;
    t_begin = static_cast<int>(lo);
    t_end = static_cast<int>(hi);
}

// Finds the sequence b whose tokens contain position `pos` of the token space, 32 sequences per
// step (warp scan of the lengths).  Every thread of the calling warp takes part and gets the result.
__device__ __forceinline__ void locate_sequence(const DecodeParams& p, long long pos, int lane, int& b,
                                                long long& tok_before, int& len_b) {
    long long before = 0;
    b = p.B;
    for (int b0 = 0; b0 < p.B; b0 += 32) {
        const int len = (b0 + lane < p.B) ? seq_len_of(p, b0 + lane) : 0;
        long long incl = len;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const long long up = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += up;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, (before + incl) * p.H > pos);
        if (hit != 0u) {
            const int l0 = __ffs(hit) - 1;
            b = b0 + l0;
            tok_before = before + __shfl_sync(0xffffffffu, incl - len, l0);
            len_b = __shfl_sync(0xffffffffu, len, l0);
            return;
        }
        before += __shfl_sync(0xffffffffu, incl, 31);
    }
}

// Counters in the workspace (the chunk counter, the tickets of the pairs) carry the launch's number above their
// count, so that whatever another launch or an uninitialised workspace left there never counts: the first CTAs to
// arrive put the launch's number in (one compare-and-swap each; a CTA that loses sees the number and goes on),
// everybody counts with a plain atomic add, which needs no retries however many CTAs come at once and is a
// single round trip to L2 once the number is in.  Returns the count with this arrival included.  claim_chunk takes the next small chunk from the launch's counter (a number
// past the last chunk: none is left).
__device__ __forceinline__ long long tagged_count(unsigned long long* word, unsigned long long call_id) {
    const unsigned long long tag = (call_id % ((1ull << 40) - 1ull) + 1ull) << 24;
    // Count first: where the launch's number is in already (every arrival but a word's first few), that is all.
    unsigned long long old = atomicAdd(word, 1ull);
    if ((old & ~0xffffffull) == tag) return static_cast<long long>(old & 0xffffffull) + 1;
    // It was not (this arrival counted on whatever the word held): put it in, or find it put in, and count again.
    unsigned long long seen = old + 1ull;
    while ((seen & ~0xffffffull) != tag) {
        old = atomicCAS(word, seen, tag);
        if (old == seen) break;
        seen = old;
    }
    return static_cast<long long>(atomicAdd(word, 1ull) & 0xffffffull) + 1;  // this request included
}

__device__ __forceinline__ long long claim_chunk(const DecodeParams& p, const Geometry& ge) {
    const long long asked = tagged_count(p.ws_counter, p.call_id);
    // Every CTA asks until it is turned away: small chunks + CTAs requests in all.  The last one leaves a zero (a
    // launch replayed from a CUDA graph carries the number it was captured with and must not count on).
    if (asked == static_cast<long long>(ge.n_chunks - ge.n_static) + ge.n_static) *p.ws_counter = 0ull;
    return ge.n_static + asked - 1;
}

// --------------------------------------------------------------------------------------
// producer warp
// --------------------------------------------------------------------------------------

template <typename Cfg, typename T, int D, int TILE_T, int STAGES>
__device__ __forceinline__ void decode_producer(const DecodeParams& p, const CUtensorMap* tm_k,
                                                const CUtensorMap* tm_v, uint8_t* stages, uint64_t* full,
                                                uint64_t* empty, StageMeta* meta, Geometry* geo, int lane) {
    const char* kbase = static_cast<const char*>(p.k);
    const char* vbase = static_cast<const char*>(p.v);
    const char* qbase = static_cast<const char*>(p.q);
    int stage = 0;
    uint32_t phase = 0;
    long long fills = 0;  // stages filled so far (for the drain after a failed wait)
    bool ok = true;

    const uint64_t l2_policy = l2_policy_evict_first();
    const Geometry ge = geometry_of(p, gridDim.x, TILE_T, lane);
    if (lane == 0) *geo = ge;  // (published to the other warps with the first stage's barrier)
    const bool on_demand = ge.n_chunks > ge.n_static;

    // Where a chunk begins: its range and the first (sequence, head) that it touches.
    struct ChunkStart {
        long long c_start, c_end;
        long long tok_before;  // tokens of the sequences that precede b
        int b, len_b, h;
    };
    auto chunk_start = [&](long long g) {
        ChunkStart cs;
        chunk_range(ge, g, cs.c_start, cs.c_end);
        cs.b = p.B;
        cs.tok_before = 0;
        cs.len_b = 0;
        if (cs.c_start < cs.c_end) locate_sequence(p, cs.c_start, lane, cs.b, cs.tok_before, cs.len_b);
        cs.h = (cs.b < p.B) ? static_cast<int>((cs.c_start - cs.tok_before * p.H) / cs.len_b) : 0;
        return cs;
    };

    // this CTA's chunks: its own advance chunk, then small ones as long as the counter has some
    ChunkStart coming = chunk_start(blockIdx.x);
    for (long long chunk = blockIdx.x; ok && chunk < ge.n_chunks;) {
        const long long c_start = coming.c_start, c_end = coming.c_end;
        long long tok_before = coming.tok_before;
        int b = coming.b, len_b = coming.len_b, h = coming.h;
        // The chunk after this one is asked for, and its beginning looked up, once this one's first tile is on its
        // way: the request is a round trip to L2 and the look-up a few hundred instructions, which at
        // the head of a chunk would hold its copies back (2.5 us per chunk, measured).  Every CTA asks until it is
        // turned away, so the launch's last request is known by its number and puts the counter back to zero (for
        // a launch replayed from a CUDA graph).
        long long chunk_next = ge.n_chunks;
        bool asked = !on_demand;
        int tiles_issued = 0;
        auto ask = [&]() {
            if (asked) return;
            if (lane == 0) chunk_next = claim_chunk(p, ge);
            chunk_next = __shfl_sync(0xffffffffu, chunk_next, 0);
            asked = true;
            if (chunk_next < ge.n_chunks) coming = chunk_start(chunk_next);
        };

        while (ok && b < p.B) {
            const long long pair_off = tok_before * p.H + static_cast<long long>(h) * len_b;
            if (pair_off >= c_end) break;
            int t_begin, t_end;
            piece_of(c_start, c_end, pair_off, len_b, TILE_T, t_begin, t_end);
            // how many chunks hold a piece with tokens of this pair (the merge counts them in)
            int pieces = 0;
            {
                const long long g_first = chunk_of(ge, pair_off), g_last = chunk_of(ge, pair_off + len_b - 1);
                for (long long g = g_first + lane; g <= g_last; g += 32) {
                    long long s0, s1;
                    chunk_range(ge, g, s0, s1);
                    int t0, t1;
                    piece_of(s0, s1, pair_off, len_b, TILE_T, t0, t1);
                    pieces += (t0 < t1) ? 1 : 0;
                }
    #pragma unroll
                for (int off = 16; off >= 1; off >>= 1) pieces += __shfl_xor_sync(0xffffffffu, pieces, off);
            }
            // a pair in one piece has a slot of its own (used when a merge kernel follows), a piece of several is one
            // of its chunk's two
            const int bh = b * p.H + h;
            int slot = pieces == 1 ? p.n_slots - p.B * p.H + bh : piece_slot(chunk, c_start, pair_off);
            if (t_begin < t_end && (slot < 0 || slot >= p.n_slots)) {
                report_status(p.dev_status, B2KV_DEV_BAD_POSITION);  // cannot happen: sized on the host
                t_end = t_begin;
                slot = 0;
            }

            for (int t0 = t_begin; t0 < t_end; t0 += TILE_T) {
                const int ntok = min(TILE_T, t_end - t0);
                if (tiles_issued++ == 1) ask();
                // paged: this lane's block of the tile is looked up before the wait for a free stage, so that the table's
                // latency falls into that wait and not between a stage coming free and its copies going out
                int blk_ahead = -1;
                if (p.block_table != nullptr && !p.use_tensor_map) {
                    const int tok = t0 + lane * p.run_len;
                    if (tok < t0 + ntok) blk_ahead = p.block_table[static_cast<int64_t>(b) * p.max_blocks + tok / p.block_size];
                }
                if (!mbar_wait(&empty[stage], phase ^ 1u)) {
                    ok = false;
                    break;
                }
                uint8_t* sbase = stages + static_cast<size_t>(stage) * Cfg::kStageBytes;
                const bool first = (t0 == t_begin);
                if (lane == 0) {
                    StageMeta mt;
                    mt.slot = slot;
                    mt.ntok = ntok;
                    mt.flags = (first ? kFlagFirst : 0) | (t0 + TILE_T >= t_end ? kFlagLast : 0) | (pieces == 1 ? kFlagWhole : 0);
                    mt.pieces = pieces;
                    mt.pair_off = pair_off;
                    mt.len = len_b;
                    mt.bh = bh;
                    meta[stage] = mt;
                    // a tiled load always delivers the whole box (rows past the end arrive as zeros or as
                    // the next rows of the cache; the consumers use the first ntok only)
                    const uint32_t rows = p.use_tensor_map ? static_cast<uint32_t>(TILE_T) : static_cast<uint32_t>(ntok);
                    const uint32_t bytes = 2u * rows * Cfg::kRowBytes + (first ? Cfg::kRowBytes : 0);
                    mbar_arrive_expect_tx(&full[stage], bytes);
                }
                __syncwarp();
                if (first && lane == 31) {
                    bulk_g2s(sbase + 2 * Cfg::kTileBytes,
                             qbase + (static_cast<size_t>(b) * p.H + h) * Cfg::kRowBytes, Cfg::kRowBytes, &full[stage]);
                }
                if (p.use_tensor_map) {
                    if (lane == 0) tma_load_4d(sbase, tm_k, &full[stage], 0, t0, h, b);
                    if (lane == 1) tma_load_4d(sbase + Cfg::kTileBytes, tm_v, &full[stage], 0, t0, h, b);
                    ++fills;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    continue;
                }
                const int nruns = (ntok + p.run_len - 1) / p.run_len;
                for (int r = lane; r < nruns; r += 32) {
                    const int tok = t0 + r * p.run_len;
                    const int cnt = min(p.run_len, t0 + ntok - tok);
                    int64_t off;
                    if (p.block_table == nullptr) {
                        off = static_cast<int64_t>(b) * p.stride_b + static_cast<int64_t>(tok) * p.stride_t;
                    } else {
                        int blk = r == lane ? blk_ahead : p.block_table[static_cast<int64_t>(b) * p.max_blocks + tok / p.block_size];
                        if (blk < 0 || blk >= p.n_blocks) {
                            report_status(p.dev_status, B2KV_DEV_BAD_BLOCK);
                            blk = 0;  // stay inside the pool; the status word tells the caller
                        }
                        off = static_cast<int64_t>(blk) * p.stride_b +
                              static_cast<int64_t>(tok % p.block_size) * p.stride_t;
                    }
                    off = (off + static_cast<int64_t>(h) * p.stride_h) * static_cast<int64_t>(sizeof(T));
                    const uint32_t bytes = static_cast<uint32_t>(cnt) * Cfg::kRowBytes;
                    const int dst = (tok - t0) * Cfg::kRowBytes;
                    if (p.l2_evict_first) {
                        bulk_g2s_hint(sbase + dst, kbase + off, bytes, &full[stage], l2_policy);
                        bulk_g2s_hint(sbase + Cfg::kTileBytes + dst, vbase + off, bytes, &full[stage], l2_policy);
                    } else {
                        bulk_g2s(sbase + dst, kbase + off, bytes, &full[stage]);
                        bulk_g2s(sbase + Cfg::kTileBytes + dst, vbase + off, bytes, &full[stage]);
                    }
                }
                ++fills;
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            // next (sequence, head); empty sequences own no tokens and are skipped
            if (++h == p.H) {
                h = 0;
                tok_before += len_b;
                do {
                    ++b;
                    len_b = (b < p.B) ? seq_len_of(p, b) : 0;
                } while (b < p.B && len_b == 0);
            }
        }
        ask();
        chunk = chunk_next;
    }

    if (ok && mbar_wait(&empty[stage], phase ^ 1u)) {
        if (lane == 0) {
            StageMeta mt;
            mt.slot = 0;
            mt.ntok = 0;
            mt.flags = kFlagDone;
            mt.pieces = 0;
            mt.pair_off = 0;
            mt.len = 0;
            mt.bh = 0;
            meta[stage] = mt;
            mbar_arrive(&full[stage]);
        }
        return;
    }
    // A wait ran out: tell the host, then make sure no copy of ours is still in flight
    // towards this CTA's shared memory before the warp leaves.
    report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
    for (long long f = max(0ll, fills - STAGES); f < fills; ++f)
        (void)mbar_wait(&full[f % STAGES], static_cast<uint32_t>((f / STAGES) & 1));
}

// Where a finished output element goes when the split kernel writes the rows itself: the local output, or -
// fused all-gather - the buffer of every rank at this rank's heads (plain peer stores over NVLink).
template <typename T, int D>
__device__ __forceinline__ void store_output(const DecodeParams& p, int bh, int d, T val) {
    if (p.gather.peer_out == nullptr) {
        static_cast<T*>(p.fused_out)[static_cast<size_t>(bh) * D + d] = val;
        return;
    }
    const int b = bh / p.H, h = bh - b * p.H;
    const size_t col = (static_cast<size_t>(b) * p.gather.h_total + static_cast<size_t>(p.gather.rank) * p.H + h) * D + d;
    for (int w = 0; w < p.gather.world; ++w) static_cast<T*>(p.gather.peer_out[w])[col] = val;
}

// --------------------------------------------------------------------------------------
// consumer warps
// --------------------------------------------------------------------------------------

template <typename Cfg, typename T, int D, int TILE_T, int STAGES, int NCW>
__device__ __forceinline__ void decode_consumer(const DecodeParams& p, uint8_t* stages, uint64_t* full,
                                                uint64_t* empty, uint64_t* hand_full, uint64_t* hand_empty,
                                                const StageMeta* meta, StageMeta* hand_meta, float* merge, int warp,
                                                int lane) {
    constexpr int LPR = Cfg::kLanesPerRow;
    constexpr int CPL = Cfg::kChunksPerLane;
    constexpr int EPC = Cfg::kEpc;
    constexpr int NACC = Cfg::kAcc;
    constexpr int RPP = Cfg::kRowsPerPass;
    constexpr int BATCH = Cfg::kBatch;
    const int g = lane / LPR;  // which of the RPP rows of a pass this lane works on
    const int j = lane % LPR;  // which 16-byte chunk(s) of the row

    float acc[NACC], qf[NACC];
    float m = -INFINITY, l = 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        acc[i] = 0.f;
        qf[i] = 0.f;
    }

    // Sequences without tokens own no work item: their output rows are zeros, written here (the CTAs share them out).
    if (p.merge_inside) {
        const int row_elems = p.H * D;
        for (int b = blockIdx.x; b < p.B; b += gridDim.x) {
            if (seq_len_of(p, b) != 0) continue;
            for (int i = warp * 32 + lane; i < row_elems; i += NCW * 32)
                store_output<T, D>(p, b * p.H + i / D, i % D, Elt<T>::from_float(0.f));
        }
        if (p.gather.peer_out != nullptr) __threadfence_system();  // (before this CTA counts itself in)
    }

    int stage = 0;
    uint32_t phase = 0;
    uint32_t item = 0;  // finished items so far: item i is handed over in merge buffer i & 1

    while (true) {
        if (!mbar_wait(&full[stage], phase)) {
            report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
            return;
        }
        const StageMeta mt = meta[stage];
        if (mt.flags & kFlagDone) {
            // tell the merging warp that nothing follows (same hand-over as an item)
            const int buf = item & 1;
            if (!mbar_wait(&hand_empty[buf], ((item >> 1) & 1u) ^ 1u)) {
                report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
                return;
            }
            if (warp == 0 && lane == 0) hand_meta[buf] = mt;
            __syncwarp();
            if (lane == 0) mbar_arrive(&hand_full[buf]);
            return;
        }
        const uint8_t* Ks = stages + static_cast<size_t>(stage) * Cfg::kStageBytes;
        const uint8_t* Vs = Ks + Cfg::kTileBytes;

        if (mt.flags & kFlagFirst) {
            m = -INFINITY;
            l = 0.f;
#pragma unroll
            for (int c = 0; c < CPL; ++c) {
                const uint4 qc = *reinterpret_cast<const uint4*>(Ks + 2 * Cfg::kTileBytes + (c * LPR + j) * 16);
                Elt<T>::widen(qc, &qf[c * EPC]);
            }
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                qf[i] *= p.q_prescale;
                acc[i] = 0.f;
            }
        }

        // Rows go to the warps in turn, RPP at a time (pass i of warp w: rows (i * NCW + w) * RPP ...), so that the
        // few rows of a short tile - the end of a (sequence, head) or of a share - are spread over all the warps.
        const int row0 = warp * RPP;
        if (row0 < mt.ntok) {
#pragma unroll 1
            for (int ib = 0; ib < Cfg::kPasses; ib += BATCH) {
                float s[BATCH];
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = row0 + (ib + i) * (NCW * RPP) + g;
                    float part = 0.f;
                    if (r < mt.ntok) {
#pragma unroll
                        for (int c = 0; c < CPL; ++c) {
                            const uint4 kc =
                                *reinterpret_cast<const uint4*>(Ks + r * Cfg::kRowBytes + (c * LPR + j) * 16);
                            float kf[EPC];
                            Elt<T>::widen(kc, kf);
#pragma unroll
                            for (int e = 0; e < EPC; ++e) part = fmaf(qf[c * EPC + e], kf[e], part);
                        }
                    }
                    s[i] = part;
                }
#pragma unroll
                for (int off = LPR / 2; off >= 1; off >>= 1) {
#pragma unroll
                    for (int i = 0; i < BATCH; ++i) s[i] += __shfl_xor_sync(0xffffffffu, s[i], off);
                }
                float m_new = m;
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = row0 + (ib + i) * (NCW * RPP) + g;
                    if (r >= mt.ntok) s[i] = -INFINITY;
                    m_new = fmaxf(m_new, s[i]);
                }
                // every row of this lane group masked so far: keep exp2 arguments finite
                const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                const float corr = exp2f(m - m_use);
                l *= corr;
#pragma unroll
                for (int i = 0; i < NACC; ++i) acc[i] *= corr;
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = row0 + (ib + i) * (NCW * RPP) + g;
                    if (r < mt.ntok) {
                        const float pr = exp2f(s[i] - m_use);
                        l += pr;
#pragma unroll
                        for (int c = 0; c < CPL; ++c) {
                            const uint4 vc =
                                *reinterpret_cast<const uint4*>(Vs + r * Cfg::kRowBytes + (c * LPR + j) * 16);
                            float vf[EPC];
                            Elt<T>::widen(vc, vf);
#pragma unroll
                            for (int e = 0; e < EPC; ++e) acc[c * EPC + e] = fmaf(pr, vf[e], acc[c * EPC + e]);
                        }
                    }
                }
                m = m_new;
            }
        }

        // all reads of this stage are done: hand it back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);
        if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
        }

        if (mt.flags & kFlagLast) {
            // merge the RPP lane groups of this warp
#pragma unroll
            for (int off = LPR; off < 32; off <<= 1) {
                const float m_o = __shfl_xor_sync(0xffffffffu, m, off);
                const float l_o = __shfl_xor_sync(0xffffffffu, l, off);
                const float m_n = fmaxf(m, m_o);
                const float m_u = (m_n == -INFINITY) ? 0.f : m_n;
                const float a = exp2f(m - m_u), bsc = exp2f(m_o - m_u);
                l = l * a + l_o * bsc;
#pragma unroll
                for (int i = 0; i < NACC; ++i) {
                    const float o = __shfl_xor_sync(0xffffffffu, acc[i], off);
                    acc[i] = acc[i] * a + o * bsc;
                }
                m = m_n;
            }
            // Hand the warp's partial to the merging warp and go on with the next tile: what follows an item (the
            // sum over the warps, the store, and for a piece the fence, the ticket and perhaps the merge of all the
            // pair's pieces: 3 - 4 us of latencies) then costs the stream nothing.  The buffer is free once the
            // merging warp has read what item - 2 left in it.
            const int buf = item & 1;
            if (!mbar_wait(&hand_empty[buf], ((item >> 1) & 1u) ^ 1u)) {
                report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
                return;
            }
            float* mb = merge + buf * Cfg::kMergeFloats + warp * (D + 2);
            if (g == 0) {
#pragma unroll
                for (int c = 0; c < CPL; ++c)
#pragma unroll
                    for (int e = 0; e < EPC; ++e) mb[(c * LPR + j) * EPC + e] = acc[c * EPC + e];
                if (j == 0) {
                    mb[D] = m;
                    mb[D + 1] = l;
                }
            }
            if (warp == 0 && lane == 0) hand_meta[buf] = mt;
            __syncwarp();
            if (lane == 0) mbar_arrive(&hand_full[buf]);
            ++item;
        }
    }
}

// --------------------------------------------------------------------------------------
// merging warp: finishes the items that the consumer warps hand over
// --------------------------------------------------------------------------------------

template <typename Cfg, typename T, int D, int TILE_T, int NCW>
__device__ __forceinline__ void decode_merger(const DecodeParams& p, uint64_t* hand_full, uint64_t* hand_empty,
                                              const StageMeta* hand_meta, const float* merge,
                                              const Geometry* geo, int lane) {
    constexpr int CPM = (D + 31) / 32;  // output columns per lane: lane, lane + 32, ...
    for (uint32_t item = 0;; ++item) {
        const int buf = item & 1;
        // Bounded like every wait; it also ends this warp should the consumer warps have given up.
        if (!mbar_wait(&hand_full[buf], (item >> 1) & 1u)) {
            report_status(p.dev_status, B2KV_DEV_WAIT_TIMEOUT);
            return;
        }
        const StageMeta mt = hand_meta[buf];
        if (mt.flags & kFlagDone) {
            // Fused all-gather: this CTA's rows are on their way to the ranks.  Fence them, count the CTA in; the
            // last CTA of the launch raises this rank's flag on every rank (and leaves the count at zero for a
            // launch replayed from a graph).
            if (p.merge_inside && p.gather.peer_out != nullptr) {
                __threadfence_system();
                __syncwarp();
                if (lane == 0 && tagged_count(p.ws_done, p.call_id) == static_cast<long long>(gridDim.x)) {
                    __threadfence_system();
                    for (int w = 0; w < p.gather.world; ++w) {
                        volatile uint32_t* flag = p.gather.peer_flags[w] + p.gather.rank;
                        *flag = p.gather.epoch;
                    }
                    __threadfence_system();
                    *p.ws_done = 0ull;
                }
            }
            return;
        }
        const float* mr = merge + buf * Cfg::kMergeFloats;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < NCW; ++w) m_all = fmaxf(m_all, mr[w * (D + 2) + D]);
        const float m_u = (m_all == -INFINITY) ? 0.f : m_all;
        float wgt[NCW];
        float l_all = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; ++w) {
            wgt[w] = exp2f(mr[w * (D + 2) + D] - m_u);
            l_all += wgt[w] * mr[w * (D + 2) + D + 1];
        }
        float o[CPM];
#pragma unroll
        for (int i = 0; i < CPM; ++i) {
            const int d = lane + 32 * i;
            o[i] = 0.f;
            if (d < D) {
#pragma unroll
                for (int w = 0; w < NCW; ++w) o[i] += wgt[w] * mr[w * (D + 2) + d];
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&hand_empty[buf]);  // the buffer and its description may be written again

        if (p.merge_inside && (mt.flags & kFlagWhole)) {
            // the whole (sequence, head) was this one item: its row is final
            // (divided, not multiplied by a reciprocal: bit for bit what the merge kernel gives)
#pragma unroll
            for (int i = 0; i < CPM; ++i) {
                const int d = lane + 32 * i;
                if (d < D) store_output<T, D>(p, mt.bh, d, Elt<T>::from_float(o[i] / l_all));
            }
            continue;
        }
#pragma unroll
        for (int i = 0; i < CPM; ++i) {
            const int d = lane + 32 * i;
            if (d < D) p.ws_acc[static_cast<size_t>(mt.slot) * D + d] = o[i];
        }
        if (lane == 0) {
            p.ws_ml[static_cast<size_t>(mt.slot) * 2] = m_all;
            p.ws_ml[static_cast<size_t>(mt.slot) * 2 + 1] = l_all;
        }
        if (!p.merge_inside) continue;  // a merge kernel follows this launch
        // One piece of several.  Publish it (fence), take a ticket for the pair: the CTA that takes the pair's last
        // ticket finds every piece in the workspace and merges them.  Nobody waits for another CTA.
        __threadfence();
        __syncwarp();
        const int bh = mt.bh;
        int last = 0;
        if (lane == 0) last = tagged_count(p.ws_tickets + bh, p.call_id) == static_cast<long long>(mt.pieces) ? 1 : 0;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last == 0) continue;
        __threadfence();
        const Geometry ge = *geo;
        const long long g_first = chunk_of(ge, mt.pair_off), g_last = chunk_of(ge, mt.pair_off + mt.len - 1);
        // The weighted sums, piece after piece (a fixed order), the loads of four chunks in flight together (a long
        // pair may come in a hundred pieces; a chunk without a piece of this pair counts with weight 0).  Up to four
        // chunks - the usual case - are one round trip to L2: their maxima come with the same loads.
        constexpr int kAhead = 4;
        float part[kAhead][CPM], pm[kAhead], pl[kAhead];
        bool live[kAhead];
        auto load_pieces = [&](long long g0) {
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const long long g = g0 + u;
                live[u] = false;
                pm[u] = -INFINITY, pl[u] = 0.f;
#pragma unroll
                for (int i = 0; i < CPM; ++i) part[u][i] = 0.f;
                if (g > g_last) continue;
                long long s0, s1;
                chunk_range(ge, g, s0, s1);
                int t0, t1;
                piece_of(s0, s1, mt.pair_off, mt.len, TILE_T, t0, t1);
                if (t0 >= t1) continue;
                live[u] = true;
                const size_t sl = static_cast<size_t>(piece_slot(g, s0, mt.pair_off));
                pm[u] = __ldcg(&p.ws_ml[sl * 2]);
                pl[u] = __ldcg(&p.ws_ml[sl * 2 + 1]);
#pragma unroll
                for (int i = 0; i < CPM; ++i) {
                    const int d = lane + 32 * i;
                    if (d < D) part[u][i] = __ldcg(&p.ws_acc[sl * D + d]);
                }
            }
        };
        float m_g = -INFINITY, l_g = 0.f, og[CPM];
#pragma unroll
        for (int i = 0; i < CPM; ++i) og[i] = 0.f;
        auto add_pieces = [&]() {
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                if (!live[u]) continue;
                const float wg = exp2f(pm[u] - m_g);
                l_g += wg * pl[u];
#pragma unroll
                for (int i = 0; i < CPM; ++i) og[i] += wg * part[u][i];
            }
        };
        if (g_last - g_first < kAhead) {
            load_pieces(g_first);
#pragma unroll
            for (int u = 0; u < kAhead; ++u) m_g = fmaxf(m_g, pm[u]);
            add_pieces();
        } else {
            // the pieces' common maximum first: the lanes share the chunks out
            for (long long g = g_first + lane; g <= g_last; g += 32) {
                long long s0, s1;
                chunk_range(ge, g, s0, s1);
                int t0, t1;
                piece_of(s0, s1, mt.pair_off, mt.len, TILE_T, t0, t1);
                if (t0 < t1) m_g = fmaxf(m_g, __ldcg(&p.ws_ml[static_cast<size_t>(piece_slot(g, s0, mt.pair_off)) * 2]));
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) m_g = fmaxf(m_g, __shfl_xor_sync(0xffffffffu, m_g, off));
            for (long long g0 = g_first; g0 <= g_last; g0 += kAhead) {
                load_pieces(g0);
                add_pieces();
            }
        }
#pragma unroll
        for (int i = 0; i < CPM; ++i) {
            const int d = lane + 32 * i;
            if (d < D) store_output<T, D>(p, bh, d, Elt<T>::from_float(og[i] / l_g));
        }
        // Every piece of the pair has come in, so nobody touches its ticket again in this launch: leave
        // it at zero.  A launch replayed from a CUDA graph carries the number it was captured with, and
        // must not count on top of its own earlier run.
        __syncwarp();
        if (lane == 0) p.ws_tickets[bh] = 0ull;
    }
}

// --------------------------------------------------------------------------------------
// kernel
// --------------------------------------------------------------------------------------

template <typename T, int D, int TILE_T, int STAGES, int NCW>
__global__ void __launch_bounds__((NCW + 2) * 32, DecodeCfg<T, D, TILE_T, STAGES, NCW>::kCtasPerSm)
decode_split_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v) {
    using Cfg = DecodeCfg<T, D, TILE_T, STAGES, NCW>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint64_t* full = reinterpret_cast<uint64_t*>(stages + static_cast<size_t>(STAGES) * Cfg::kStageBytes);
    uint64_t* empty = full + STAGES;
    // finished items go from the consumer warps to the merging warp through two buffers
    uint64_t* hand_full = empty + STAGES;   // [2] the eight warps' partials of an item are in the buffer
    uint64_t* hand_empty = hand_full + 2;   // [2] the merging warp has read the buffer
    StageMeta* meta = reinterpret_cast<StageMeta*>(hand_empty + 2);
    StageMeta* hand_meta = meta + STAGES;   // [2] the item in each buffer
    float* merge = reinterpret_cast<float*>(hand_meta + 2);
    Geometry* geo = reinterpret_cast<Geometry*>(merge + 2 * Cfg::kMergeFloats);  // how the token space is cut

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NCW);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&hand_full[s], NCW);
            mbar_init(&hand_empty[s], 1);
        }
        fence_mbar_init();
        // The lengths, the queries and the newest cache rows may come from the kernel before this one.  One thread
        // waits for it and the others sleep at the barrier: a CTA that is launched ahead of time shares its SM
        // with CTAs of that kernel and must not take issue slots from them.
        grid_dependency_wait();
    }
    __syncthreads();
    if (warp == NCW) {
        decode_producer<Cfg, T, D, TILE_T, STAGES>(p, &tm_k, &tm_v, stages, full, empty, meta, geo, lane);
    } else if (warp == NCW + 1) {
        decode_merger<Cfg, T, D, TILE_T, NCW>(p, hand_full, hand_empty, hand_meta, merge, geo, lane);
    } else {
        decode_consumer<Cfg, T, D, TILE_T, STAGES, NCW>(p, stages, full, empty, hand_full, hand_empty, meta, hand_meta, merge,
                                                        warp, lane);
    }
}

// One CTA per (sequence, head), one thread per output column.  Recomputes which shares of the
// split kernel's grid (`n_ctas`, tile `tile`) hold a piece of this pair and merges their partials.
template <typename T, int D>
__global__ void __launch_bounds__(D < 32 ? 32 : D) decode_combine_kernel(const DecodeParams p, T* __restrict__ out,
                                                                       int n_ctas, int tile) {
    __shared__ long long sh_before;
    __shared__ Geometry sh_geo;
    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh - b * p.H;
    const int d = threadIdx.x;
    if (threadIdx.x < 32) {
        const Geometry ge = geometry_of(p, n_ctas, tile, threadIdx.x);
        long long before = 0;
        for (int i = threadIdx.x; i < b; i += 32) before += seq_len_of(p, i);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) before += __shfl_xor_sync(0xffffffffu, before, off);
        if (threadIdx.x == 0) {
            sh_before = before;
            sh_geo = ge;
        }
    }
    __syncthreads();
    const int n = seq_len_of(p, b);
    float m_all = -INFINITY, l_all = 0.f, o = 0.f;
    if (d < D && n > 0) {
        const Geometry ge = sh_geo;
        const long long pair_off = sh_before * p.H + static_cast<long long>(h) * n;
        const long long g_first = chunk_of(ge, pair_off), g_last = chunk_of(ge, pair_off + n - 1);
        // first pass: the pieces and their common maximum; second pass: the weighted sums.  A pair in one piece
        // has a slot of its own, a piece of several is one of its chunk's two.
        int pieces = 0;
        for (long long g = g_first; g <= g_last; ++g) {
            long long s0, s1;
            chunk_range(ge, g, s0, s1);
            int t0, t1;
            piece_of(s0, s1, pair_off, n, tile, t0, t1);
            pieces += (t0 < t1) ? 1 : 0;
        }
        const size_t own = static_cast<size_t>(p.n_slots - p.B * p.H + bh);
        for (long long g = g_first; g <= g_last; ++g) {
            long long s0, s1;
            chunk_range(ge, g, s0, s1);
            int t0, t1;
            piece_of(s0, s1, pair_off, n, tile, t0, t1);
            if (t0 < t1) m_all = fmaxf(m_all, p.ws_ml[(pieces == 1 ? own : static_cast<size_t>(piece_slot(g, s0, pair_off))) * 2]);
        }
        for (long long g = g_first; g <= g_last; ++g) {
            long long s0, s1;
            chunk_range(ge, g, s0, s1);
            int t0, t1;
            piece_of(s0, s1, pair_off, n, tile, t0, t1);
            if (t0 < t1) {
                const size_t slot = pieces == 1 ? own : static_cast<size_t>(piece_slot(g, s0, pair_off));
                const float wgt = exp2f(p.ws_ml[slot * 2] - m_all);
                l_all += wgt * p.ws_ml[slot * 2 + 1];
                o += wgt * p.ws_acc[slot * D + d];
            }
        }
    }
    if (p.partial_out != nullptr) {
        // sequence-split mode: this rank saw only a slice of the tokens; hand the unnormalised row and
        // its (max, sum) to the cross-rank merge.  Layout [B*H, D + 2]; max is in the log2 domain.
        float* row = p.partial_out + static_cast<size_t>(bh) * (D + 2);
        if (d < D) row[d] = o;
        if (d == 0) {
            row[D] = m_all;
            row[D + 1] = l_all;
        }
        return;
    }
    if (d < D) out[static_cast<size_t>(bh) * D + d] = Elt<T>::from_float(n > 0 ? o / l_all : 0.f);
}

// Waits (bounded) until every rank's flag has reached `epoch`: lane w watches rank w.  The flags
// are written by kernels running on other GPUs, never by a kernel queued behind this one.
__global__ void gather_wait_kernel(const uint32_t* flags, int world, uint32_t epoch, int32_t* dev_status) {
    const int w = threadIdx.x;
    if (w >= world) return;
    const volatile uint32_t* flag = flags + w;
    for (uint32_t it = 0; it < (1u << 21); ++it) {
        if (static_cast<int32_t>(*flag - epoch) >= 0) {
            __threadfence_system();
            return;
        }
        __nanosleep(it < 64 ? 100 : 1000);
    }
    report_status(dev_status, B2KV_DEV_WAIT_TIMEOUT);
}

// --------------------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------------------

// Tokens per K (or V) tile for a row of `row_bytes` in the generic configuration: 8 KB tiles,
// so that several CTAs (twelve or more consumer warps) fit on one SM; the consumers, not the
// copy engine, are what has to keep up with HBM.
constexpr int default_tile(int row_bytes) {
    int t = 8192 / row_bytes;
    return t > 128 ? 128 : (t < 8 ? 8 : t);
}

// Most CTAs per SM that a launch uses: the grid is persistent, more would only add partials.
constexpr int kMaxCtasPerSm = 4;

// Partial-result slots for a grid of `n_ctas`: two per chunk (a chunk shares at most its first and its last
// (sequence, head) with other chunks) and one per (sequence, head) for pairs in one piece.
static size_t partial_slots(int n_ctas, int B, int H) {
    return 2 * static_cast<size_t>(max_chunks(n_ctas)) + static_cast<size_t>(B) * H;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Number of this launch for the tickets of the merge inside the split kernel: 48 bits, never 0, starting from a
// value that no earlier process is likely to have left in a reused workspace.
static unsigned long long next_call_id() {
    static std::atomic<unsigned long long> counter{
        (static_cast<unsigned long long>(std::chrono::steady_clock::now().time_since_epoch().count()) * 0x9E3779B97F4A7C15ull) >> 8};
    unsigned long long id = (counter.fetch_add(1) + 1) & ((1ull << 48) - 1);
    return id == 0 ? 1 : id;
}

template <typename T, int D, int TILE_T, int STAGES, int NCW>
static int launch_decode(DecodeParams p, void* out, void* workspace, size_t workspace_bytes, void* stream) {
    using Cfg = DecodeCfg<T, D, TILE_T, STAGES, NCW>;
    auto kernel = decode_split_kernel<T, D, TILE_T, STAGES, NCW>;
    static bool configured[64] = {false};
    static int ctas_per_sm[64] = {0};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        B2KV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(Cfg::kSmemBytes)));
        int occ = 0;
        B2KV_CUDA_TRY(
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, Cfg::kThreads, Cfg::kSmemBytes));
        if (occ < 1) return B2KV_ERR_UNSUPPORTED;
        ctas_per_sm[dev] = occ;
        configured[dev] = true;
    }
    int per_sm = tune_get("decode_grid_per_sm");
    if (per_sm <= 0 || per_sm > ctas_per_sm[dev]) per_sm = ctas_per_sm[dev];
    if (per_sm > kMaxCtasPerSm) per_sm = kMaxCtasPerSm;
    const int grid_full = device_sm_count() * per_sm;
    // no more CTAs than tiles of work (upper bound from T_upper)
    const long long tiles_upper = static_cast<long long>(p.B) * p.H * ((p.T_upper + TILE_T - 1) / TILE_T);
    int grid = static_cast<int>(tiles_upper < grid_full ? tiles_upper : grid_full);
    if (grid < 1) grid = 1;
    const size_t slots = partial_slots(grid, p.B, p.H);
    if (slots > 0x7fffffffull) return B2KV_ERR_UNSUPPORTED;
    p.n_slots = static_cast<int>(slots);
    p.l2_evict_first = tune_get("decode_l2_keep") ? 0 : 1;
    p.dynamic_chunks = tune_get("decode_dynamic_chunks");

    // a bulk copy may cover several rows only when rows are adjacent in memory
    if (p.stride_t == D) {
        p.run_len = p.block_table ? (p.block_size < TILE_T ? p.block_size : TILE_T) : TILE_T;
        if (p.block_table && (TILE_T % p.run_len) != 0) p.run_len = 1;
        if (p.block_table && p.block_size > TILE_T && (p.block_size % TILE_T) != 0) p.run_len = 1;
    } else {
        p.run_len = 1;
    }

    const size_t acc_bytes = align_up(slots * D * sizeof(float), 256);
    const size_t ml_bytes = align_up(slots * 2 * sizeof(float), 8);
    const size_t ticket_bytes = static_cast<size_t>(p.B) * p.H * sizeof(unsigned long long);
    const size_t need = acc_bytes + ml_bytes + ticket_bytes + 2 * sizeof(unsigned long long);
    if (workspace == nullptr || workspace_bytes < need) return B2KV_ERR_WORKSPACE;
    p.ws_acc = static_cast<float*>(workspace);
    p.ws_ml = reinterpret_cast<float*>(static_cast<char*>(workspace) + acc_bytes);
    p.ws_tickets = reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + acc_bytes + ml_bytes);
    p.ws_counter = p.ws_tickets + static_cast<size_t>(p.B) * p.H;
    p.ws_done = p.ws_counter + 1;
    // The decode merges inside the split kernel, with the fused all-gather's peer stores too; the sequence split,
    // whose merge leaves unnormalised partials, keeps the merge kernel.
    const bool fused_merge = p.partial_out == nullptr && (p.gather.peer_out != nullptr || !tune_get("decode_merge_kernel"));
    p.merge_inside = fused_merge ? 1 : 0;
    p.fused_out = fused_merge ? out : nullptr;
    p.call_id = next_call_id();

    // Row-strided contiguous caches (the reference layout): one tiled TMA load per tile.  The maps
    // bound the token coordinate by T_upper, which no attended row exceeds.
    CUtensorMap tm_k, tm_v;
    memset(&tm_k, 0, sizeof(tm_k));
    memset(&tm_v, 0, sizeof(tm_v));
    p.use_tensor_map = 0;
    if (p.block_table == nullptr && p.run_len == 1 && !tune_get("decode_no_tensor_map") && D <= 256) {
        const int dt = sizeof(T) == 4 ? B2KV_DTYPE_F32 : B2KV_DTYPE_BF16;
        if (make_cache_tensor_map(&tm_k, p.k, dt, D, p.T_upper, p.H, p.B, p.stride_b, p.stride_t, p.stride_h, D, TILE_T,
                                  CU_TENSOR_MAP_SWIZZLE_NONE) &&
            make_cache_tensor_map(&tm_v, p.v, dt, D, p.T_upper, p.H, p.B, p.stride_b, p.stride_t, p.stride_h, D, TILE_T,
                                  CU_TENSOR_MAP_SWIZZLE_NONE))
            p.use_tensor_map = 1;
    }

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    OverlapLaunch launch(grid, Cfg::kThreads, Cfg::kSmemBytes, s);
    B2KV_CUDA_TRY(cudaLaunchKernelEx(&launch.cfg, kernel, p, tm_k, tm_v));
    B2KV_CUDA_TRY(cudaGetLastError());
    if (!fused_merge) {
        decode_combine_kernel<T, D><<<p.B * p.H, D < 32 ? 32 : D, 0, s>>>(p, static_cast<T*>(out), grid, TILE_T);
        B2KV_CUDA_TRY(cudaGetLastError());
    }
    if (p.gather.peer_out != nullptr && p.gather.my_flags != nullptr) {
        gather_wait_kernel<<<1, 32, 0, s>>>(p.gather.my_flags, p.gather.world, p.gather.epoch, p.dev_status);
        B2KV_CUDA_TRY(cudaGetLastError());
    }
    return B2KV_OK;
}

template <typename T, int D>
static int dispatch_variant(const DecodeParams& p, void* out, void* ws, size_t ws_bytes, void* stream) {
    constexpr int kRow = D * static_cast<int>(sizeof(T));
    // Variants of the ring for the headline row size (256 bytes: bf16 head_dim 128, fp32 head_dim 64);
    // other row sizes use the default (8 KB tiles, 4 stages, 4 consumer warps).
    if constexpr (kRow == 256) {
        switch (tune_get("decode_variant")) {
            case 1: return launch_decode<T, D, 64, 3, 4>(p, out, ws, ws_bytes, stream);
            case 2: return launch_decode<T, D, 32, 3, 4>(p, out, ws, ws_bytes, stream);
            case 3: return launch_decode<T, D, 64, 4, 8>(p, out, ws, ws_bytes, stream);
            case 4: return launch_decode<T, D, 128, 3, 8>(p, out, ws, ws_bytes, stream);
            case 5: return launch_decode<T, D, 32, 6, 4>(p, out, ws, ws_bytes, stream);
            case 6: return launch_decode<T, D, 64, 3, 8>(p, out, ws, ws_bytes, stream);
            case 7: return launch_decode<T, D, 16, 6, 4>(p, out, ws, ws_bytes, stream);
            case 8: return launch_decode<T, D, 32, 4, 8>(p, out, ws, ws_bytes, stream);
            case 9: return launch_decode<T, D, 32, 4, 4>(p, out, ws, ws_bytes, stream);
            case 10: return launch_decode<T, D, 32, 5, 4>(p, out, ws, ws_bytes, stream);
            case 11: return launch_decode<T, D, 16, 4, 4>(p, out, ws, ws_bytes, stream);
            case 12: return launch_decode<T, D, 32, 2, 4>(p, out, ws, ws_bytes, stream);
            case 13: return launch_decode<T, D, 64, 2, 16>(p, out, ws, ws_bytes, stream);
            case 14: return launch_decode<T, D, 128, 2, 16>(p, out, ws, ws_bytes, stream);
            case 15: return launch_decode<T, D, 64, 3, 16>(p, out, ws, ws_bytes, stream);
            case 16: return launch_decode<T, D, 128, 2, 8>(p, out, ws, ws_bytes, stream);
            case 17: return launch_decode<T, D, 64, 2, 8>(p, out, ws, ws_bytes, stream);
            // Default: 16 KB tiles and 8 consumer warps; six stages per SM either as two CTAs of three stages (fewer
            // CTAs, fewer pieces to merge: 2 - 3 % faster on contiguous caches, 643 against 653 us at the benchmark
            // shape) or, through a block table, as three CTAs of two (three copy warps per SM for the many short
            // copies: 683 against 706 us with 16-token blocks).
            default:
                if (p.block_table != nullptr) return launch_decode<T, D, 64, 2, 8>(p, out, ws, ws_bytes, stream);
                return launch_decode<T, D, 64, 3, 8>(p, out, ws, ws_bytes, stream);
        }
    } else {
        return launch_decode<T, D, default_tile(kRow), 4, 4>(p, out, ws, ws_bytes, stream);
    }
}

template <typename T>
static int dispatch_dim(const DecodeParams& p, int D, void* out, void* ws, size_t ws_bytes, void* stream) {
    switch (D) {
        case 16: return dispatch_variant<T, 16>(p, out, ws, ws_bytes, stream);
        case 32: return dispatch_variant<T, 32>(p, out, ws, ws_bytes, stream);
        case 64: return dispatch_variant<T, 64>(p, out, ws, ws_bytes, stream);
        case 128: return dispatch_variant<T, 128>(p, out, ws, ws_bytes, stream);
        case 256: return dispatch_variant<T, 256>(p, out, ws, ws_bytes, stream);
        default: return B2KV_ERR_UNSUPPORTED;
    }
}

// Argument checks shared by every decode entry point; nothing touches the device here.
static int decode_check_args(const void* q, const void* k, const void* v, const void* out, bool out_optional,
                             const int32_t* block_table, int max_blocks, int block_size, int n_blocks, int B, int H,
                             int D, int T_upper, int64_t s0, int64_t st, int64_t sh, int dtype, const void* workspace) {
    const int es = elt_bytes(dtype);
    if (es == 0) return B2KV_ERR_UNSUPPORTED;
    if (!q || !k || !v || (!out && !out_optional)) return B2KV_ERR_BAD_ARG;
    if (B <= 0 || H <= 0 || D <= 0 || T_upper <= 0) return B2KV_ERR_BAD_ARG;
    if (static_cast<long long>(B) * H > 0x7fffffffLL / 4) return B2KV_ERR_UNSUPPORTED;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(workspace))
        return B2KV_ERR_ALIGN;
    if (!stride_ok(s0, es) || !stride_ok(st, es) || !stride_ok(sh, es)) return B2KV_ERR_ALIGN;
    if (st < D && st != 0) return B2KV_ERR_BAD_ARG;
    if (block_table && (max_blocks <= 0 || block_size <= 0 || n_blocks <= 0 ||
                        static_cast<long long>(max_blocks) * block_size < T_upper))
        return B2KV_ERR_BAD_ARG;
    return B2KV_OK;
}

static int decode_entry(const void* q, const void* k, const void* v, void* out, const int32_t* seq_lens, int len,
                        int len_bias, const int32_t* block_table, int max_blocks, int block_size, int n_blocks, int B,
                        int H, int D, int T_upper, int64_t s0, int64_t st, int64_t sh, int dtype, void* workspace,
                        size_t workspace_bytes, int32_t* dev_status, void* stream, const GatherInfo* gather = nullptr,
                        float* partial_out = nullptr) {
    const int rc = decode_check_args(q, k, v, out, gather != nullptr, block_table, max_blocks, block_size, n_blocks, B, H,
                                     D, T_upper, s0, st, sh, dtype, workspace);
    if (rc != B2KV_OK) return rc;
    DecodeParams p{};
    p.q = q;
    p.k = k;
    p.v = v;
    p.seq_lens = seq_lens;
    p.block_table = block_table;
    p.dev_status = dev_status;
    p.len_scalar = len;
    p.len_bias = len_bias;
    p.B = B;
    p.H = H;
    p.T_upper = T_upper;
    p.max_blocks = max_blocks;
    p.block_size = block_size;
    p.n_blocks = n_blocks;
    p.stride_b = s0;
    p.stride_t = st;
    p.stride_h = sh;
    p.q_prescale = static_cast<float>(1.4426950408889634 / sqrt(static_cast<double>(D)));
    if (gather != nullptr) p.gather = *gather;
    p.partial_out = partial_out;
    if (dtype == B2KV_DTYPE_F32) return dispatch_dim<float>(p, D, out, workspace, workspace_bytes, stream);
    return dispatch_dim<__nv_bfloat16>(p, D, out, workspace, workspace_bytes, stream);
}

}  // namespace b2kv

using namespace b2kv;

extern "C" {

size_t b2kv_decode_workspace_bytes(int B, int H, int D, int T_upper, int dtype) {
    const int es = elt_bytes(dtype);
    if (B <= 0 || H <= 0 || D <= 0 || T_upper <= 0 || es == 0 || (D * es) % 16 != 0) return 0;
    // An upper bound of what any compiled variant will ask for: the largest grid a launch uses.
    (void)T_upper;
    const size_t slots = partial_slots(device_sm_count() * kMaxCtasPerSm, B, H);
    return align_up(slots * D * sizeof(float), 256) + align_up(slots * 2 * sizeof(float), 8) +
           static_cast<size_t>(B) * H * sizeof(unsigned long long) + 2 * sizeof(unsigned long long) + 256;
}

int b2kv_decode(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* seq_lens, int len,
                int len_bias, int B, int H, int D, int T_upper, int64_t stride_b, int64_t stride_t, int64_t stride_h,
                int dtype, void* workspace, size_t workspace_bytes, int32_t* dev_status, void* stream) {
    return decode_entry(q, k_cache, v_cache, out, seq_lens, len, len_bias, nullptr, 0, 0, 0, B, H, D, T_upper,
                        stride_b, stride_t, stride_h, dtype, workspace, workspace_bytes, dev_status, stream);
}

int b2kv_decode_paged(const void* q, const void* k_pool, const void* v_pool, void* out, const int32_t* seq_lens,
                      int len, int len_bias, const int32_t* block_table, int max_blocks, int block_size, int n_blocks,
                      int B, int H, int D, int T_upper, int64_t stride_blk, int64_t stride_t, int64_t stride_h,
                      int dtype, void* workspace, size_t workspace_bytes, int32_t* dev_status, void* stream) {
    if (!block_table) return B2KV_ERR_BAD_ARG;
    return decode_entry(q, k_pool, v_pool, out, seq_lens, len, len_bias, block_table, max_blocks, block_size,
                        n_blocks, B, H, D, T_upper, stride_blk, stride_t, stride_h, dtype, workspace, workspace_bytes,
                        dev_status, stream);
}

}  // extern "C"

namespace b2kv {

// Merges R partial results of every (sequence, head): parts[r][bh][0..D) unnormalised row,
// [D] max (log2 domain, -inf when the slice held no token), [D+1] sum.  One CTA per (sequence, head).
template <typename T>
__global__ void merge_partials_kernel(const float* __restrict__ parts, int R, int BH, int D, T* __restrict__ out) {
    const int bh = blockIdx.x;
    const size_t stride_r = static_cast<size_t>(BH) * (D + 2);
    const float* base = parts + static_cast<size_t>(bh) * (D + 2);
    float m_all = -INFINITY;
    for (int r = 0; r < R; ++r) m_all = fmaxf(m_all, base[r * stride_r + D]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float l_all = 0.f, o = 0.f;
        if (m_all != -INFINITY) {
            for (int r = 0; r < R; ++r) {
                const float m_r = base[r * stride_r + D];
                if (m_r == -INFINITY) continue;
                const float w = exp2f(m_r - m_all);
                l_all += w * base[r * stride_r + D + 1];
                o += w * base[r * stride_r + d];
            }
        }
        out[static_cast<size_t>(bh) * D + d] = Elt<T>::from_float(l_all > 0.f ? o / l_all : 0.f);
    }
}

}  // namespace b2kv

extern "C" int b2kv_decode_partial(const void* q, const void* k_cache, const void* v_cache, float* partial_out,
                                   const int32_t* seq_lens, int len, int len_bias, int B, int H, int D, int T_upper,
                                   int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype, void* workspace,
                                   size_t workspace_bytes, int32_t* dev_status, void* stream) {
    if (!partial_out || !aligned16(partial_out)) return partial_out ? B2KV_ERR_ALIGN : B2KV_ERR_BAD_ARG;
    GatherInfo none{};
    return decode_entry(q, k_cache, v_cache, partial_out, seq_lens, len, len_bias, nullptr, 0, 0, 0, B, H, D, T_upper,
                        stride_b, stride_t, stride_h, dtype, workspace, workspace_bytes, dev_status, stream, &none,
                        partial_out);
}

extern "C" int b2kv_merge_partials(const float* parts, int R, int B, int H, int D, void* out, int dtype, void* stream) {
    if (!parts || !out || R <= 0 || B <= 0 || H <= 0 || D <= 0) return B2KV_ERR_BAD_ARG;
    if (elt_bytes(dtype) == 0) return B2KV_ERR_UNSUPPORTED;
    const int threads = D < 32 ? 32 : (D > 256 ? 256 : D);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == B2KV_DTYPE_F32)
        merge_partials_kernel<float><<<B * H, threads, 0, s>>>(parts, R, B * H, D, static_cast<float*>(out));
    else
        merge_partials_kernel<__nv_bfloat16><<<B * H, threads, 0, s>>>(parts, R, B * H, D, static_cast<__nv_bfloat16*>(out));
    B2KV_CUDA_TRY(cudaGetLastError());
    return B2KV_OK;
}

extern "C" int b2kv_decode_allgather(const void* q, const void* k_cache, const void* v_cache, const int32_t* seq_lens,
                                     int len, int len_bias, int B, int H_local, int D, int T_upper, int64_t stride_b,
                                     int64_t stride_t, int64_t stride_h, int dtype, void* workspace,
                                     size_t workspace_bytes, void* const* peer_out, uint32_t* const* peer_flags,
                                     const uint32_t* my_flags, uint32_t* counter, uint32_t counter_target, int rank,
                                     int world, int H_total, uint32_t epoch, int32_t* dev_status, void* stream) {
    if (!peer_out || !peer_flags) return B2KV_ERR_BAD_ARG;
    if (world < 1 || world > 32 || rank < 0 || rank >= world || H_total != H_local * world) return B2KV_ERR_BAD_ARG;
    GatherInfo g{peer_out, peer_flags, my_flags, counter, counter_target, rank, world, H_total, epoch};
    return decode_entry(q, k_cache, v_cache, nullptr, seq_lens, len, len_bias, nullptr, 0, 0, 0, B, H_local, D, T_upper,
                        stride_b, stride_t, stride_h, dtype, workspace, workspace_bytes, dev_status, stream, &g);
}

// --------------------------------------------------------------------------------------
// Decode without any allocation by the caller: the split-K partials live in an array that is
// part of the library image.
// --------------------------------------------------------------------------------------

// Partials of b2kv_decode_static.  File scope, so every GPU whose context loads this library
// holds these B2KV_STATIC_SCRATCH_BYTES until the process exits.  In host code this name is only
// a host-side stand-in for the device array, never a device address: the address is obtained
// with cudaGetSymbolAddress below and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_decode_static_scratch[B2KV_STATIC_SCRATCH_BYTES];

// Device address of the array for the current device, looked up once per device.
static int decode_static_scratch(void** out) {
    static void* addr[64] = {nullptr};
    int dev = 0;
    B2KV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B2KV_ERR_UNSUPPORTED;
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        B2KV_CUDA_TRY(cudaGetSymbolAddress(&p, g_decode_static_scratch));
        if (p == nullptr) return B2KV_ERR_CUDA;
        addr[dev] = p;
    }
    *out = addr[dev];
    return B2KV_OK;
}

extern "C" int b2kv_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                  const int32_t* seq_lens, int len, int len_bias, int B, int H, int D, int T_upper,
                                  int64_t stride_b, int64_t stride_t, int64_t stride_h, int dtype,
                                  int32_t* dev_status, void* stream) {
    // argument checks first, so that a bad call is refused without touching the device
    int rc = decode_check_args(q, k_cache, v_cache, out, false, nullptr, 0, 0, 0, B, H, D, T_upper, stride_b, stride_t,
                               stride_h, dtype, nullptr);
    if (rc != B2KV_OK) return rc;
    if (D != 16 && D != 32 && D != 64 && D != 128 && D != 256) return B2KV_ERR_UNSUPPORTED;
    void* scratch = nullptr;
    rc = decode_static_scratch(&scratch);
    if (rc != B2KV_OK) return rc;
    // Nothing needs clearing: every partial that a merge reads is written by the same call first, and the
    // tickets carry the number of the launch.
    rc = decode_entry(q, k_cache, v_cache, out, seq_lens, len, len_bias, nullptr, 0, 0, 0, B, H, D, T_upper, stride_b,
                      stride_t, stride_h, dtype, scratch, static_cast<size_t>(B2KV_STATIC_SCRATCH_BYTES), dev_status,
                      stream);
    return rc == B2KV_ERR_WORKSPACE ? B2KV_ERR_STATIC_LIMIT : rc;
}

