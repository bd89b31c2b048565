// Split-KV decode attention (one query token per stream) for sm_100a.
//
// Replaces, for the n_q == 1 call of MiniCPMModel::forward_step (src/minicpm.cpp:813-846 ->
// :708-710), what ggml's CPU backend does in ggml_compute_forward_flash_attn_ext_f16_one_chunk
// plus ggml_flash_attn_ext_reduce_partials (third_party/ggml/src/ggml-cpu/ops.cpp:8109-8345,
// 8637-8705) and what ggml-cuda does in flash_attn_ext_vec + flash_attn_combine_results with its
// stream-k style work split (third_party/ggml/src/ggml-cuda/fattn-vec.cuh:19-507,
// fattn-common.cuh:728-779, 923-975).
//
// Design (HBM-bound kernel; the cache is read exactly once):
//   work  = the 64-row K/V tiles of every (stream, kv head) pair of the launch, laid end to end
//           in one list (stream-major, then kv head, then position).  The list is cut into equal
//           runs, one per CTA of a one-wave grid, whatever the streams' lengths are: a CTA's run
//           may start in the middle of one pair and end in the middle of another.  The cut is
//           computed on the device from the lengths as they are at launch time, so nothing in
//           the launch depends on the position but its grid size.  Launches with short runs
//           split every pair on its own instead (no CTA crosses from one pair into the next),
//           and f16 launches of few pairs run one thread-block cluster per pair: see
//           cut_work_list and the cluster mode in launch_decode;
//   copy  = a producer warp streams its run of tiles into a shared-memory ring (4 stages for f16,
//           6 for q8_0) signalled on mbarriers, straight across pair boundaries: f16 K and V tiles
//           by bulk-tensor copies (cp.async.bulk.tensor, 128-byte swizzle), a q8_0 tile (bytes and
//           scales of K and V, one span of the cache) by one bulk copy;
//   math  = four consumer warps, 16 rows of each tile.  Q (pre-scaled by scale*log2 e) is split as
//           hi + lo in f16 and the two parts occupy rows 0-7 and 8-15 of the m16n8k16 A operand,
//           so one MMA yields the hi and lo products and their sum carries ~22 bits of Q.  The
//           same trick carries the softmax weights P through the P.V MMA.  Accumulation is f32;
//   merge = at the end of each pair's part of the run the warps are merged through shared memory
//           (the ring stage of the tile consumed last).  A pair that lies inside one run is
//           written out directly; otherwise the (max, sum, acc[64]) partials go to one of the
//           CTA's two workspace slots and the last CTA of the pair to finish folds them (a ticket
//           counter per pair, taken when the run ends, decides who is last); in cluster mode they
//           go to the first CTA of the pair's cluster through distributed shared memory.
// q8_0 K/V: a stored byte is q + 128 and becomes an f16 tensor-core operand with one byte permute
// (the subnormal (q + 128) * 2^-24); the 128 comes out of the accumulators, the per-block scales are
// applied in f32 to the per-block score accumulators (K) and folded into the softmax weights (V),
// so Q is never quantised.
#include "kv_cache.cuh"

#include <algorithm>
#include <cstdlib>

using namespace vox;

namespace {

constexpr int kConsumerWarps = 4;
constexpr int kThreads       = (kConsumerWarps + 1) * 32;
constexpr int kPartialStride = 66;  // max, sum, acc[64]
constexpr int kMaxGqa        = 8;   // query heads per kv head (rows 0-7 of the A operand)

// Developer build (-DVOX_ATTN_DEVELOPER): every CTA notes the time (globaltimer, ns) at which it passes a few points
// of its life, launches of even and odd layers apart (two consecutive launches are then on record together);
// vox_debug_decode_trace copies the notes out.  Compiled out of the product library.
#ifdef VOX_ATTN_DEVELOPER
constexpr int kTraceCtas = 1024, kTracePoints = 8;
__device__ unsigned long long g_decode_trace[2][kTraceCtas][kTracePoints];
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define DECODE_TRACE(point) do { if (blockIdx.x < kTraceCtas) g_decode_trace[p.layer & 1][blockIdx.x][point] = global_ns(); } while (0)
#else
#define DECODE_TRACE(point)
#endif

struct DecodeParams {
    const uint8_t * q;
    size_t          q_nb_head, q_nb_stream;
    const int32_t * kv_len;
    int             kv_len_const;
    float *         partial;   // [2 * gridDim.x][gqa][kPartialStride]
    float *         dst;
    int             n_streams, n_kv_heads, n_heads, gqa, layer, max_len;
    int             run_min;   // fewest tiles a CTA's run holds (bounds the partials per pair)
    float           scale_log2;
    int *           status;
    int *           counters;  // one ticket counter per (stream, kv head), zero between launches
    // Fused append (k_new non-null): kv_len[stream] counts the row that arrives with this call; the CTA
    // whose run holds the pair's last tile converts the row, stores it into the cache and uses it.
    const uint8_t * k_new;
    const uint8_t * v_new;
    size_t          new_nb_head, new_nb_stream;
    uint8_t *       k_rows;    // this layer's K rows (f16 plane; q8_0: the K bytes of the layer's first tile, see kv_cache.cuh)
    uint8_t *       v_rows;
    uint8_t *       k_scales;  // q8_0: the K scales of the layer's first tile
    uint8_t *       v_scales;
    size_t          nb_pos, nb_head, nb_stream, sb_pos, sb_head, sb_stream;
    // q8_0: the tiles of this layer (one contiguous span per 64 rows of a pair, see kQ8TileBytes) and the strides of a
    // pair and of a stream
    const uint8_t * q8_tiles;
    size_t          q8_nb_head, q8_nb_stream;
    // Non-zero: the lengths and the cache rows this launch reads were not written by the kernel just before
    // it on the stream (only Q and the arriving row were), so the first tiles are requested before the
    // programmatic-dependency wait, while that kernel is still draining.
    int             early;
    int             early_tiles;  // tiles of a run requested before the dependency wait (at most the ring's depth)
    // Cluster mode (cluster > 0): the grid is one thread-block cluster of `cluster` CTAs per pair; the CTAs of a cluster
    // split the pair's tiles among them and hand their partial results to the first CTA through distributed shared
    // memory.  The ring then has n_stages stages and the memory of the rest holds the partials.
    int             cluster, n_stages;
    // Non-null: [stream][32] (cos, sin) pairs; Q and the arriving K row are rotated as they are read
    // (element i with element i + 32: the reference's ggml_rope_ext, GGML_ROPE_TYPE_NEOX).
    const float2 *  rope;
    // Non-null: a permutation of the streams; position i of the work list belongs to stream order[i]
    const int32_t * order;
    // Non-null: additive f16 mask of the single query row, [n_kv] per (head % mask_ne2, stream % mask_ne3)
    // (the operator's mask tensor for n_q == 1, third_party/ggml/src/ggml-cpu/ops.cpp:8233-8237)
    const uint8_t * mask;
    size_t          mask_nb_head, mask_nb_stream;
    int             mask_ne2, mask_ne3;
};

__device__ __forceinline__ int clamp_len(const DecodeParams & p, int len) { return max(0, min(len, p.max_len)); }
__device__ __forceinline__ int tiles_of(int len) { return (len + kKvTile - 1) / kKvTile; }

// Where a warp stands in the work list: tile `t` of kv head `kvh` of the stream at list position `i`.
struct Walk {
    int i, stream, len, tiles, kvh, t;
};

__device__ __forceinline__ void walk_load(const DecodeParams & p, Walk & w) {
    w.stream = p.order ? p.order[w.i] : w.i;
    w.len    = clamp_len(p, p.kv_len ? p.kv_len[w.stream] : p.kv_len_const);
    w.tiles  = tiles_of(w.len);
}
// to tile 0 of the next pair that has any rows (the caller knows there is one)
__device__ __forceinline__ void walk_next_pair(const DecodeParams & p, Walk & w) {
    w.t = 0;
    if (++w.kvh < p.n_kv_heads) return;
    w.kvh = 0;
    do {
        ++w.i;
        walk_load(p, w);
    } while (w.tiles == 0 && w.i + 1 < p.n_streams);
}

// The cut of the work list, computed by every warp for itself (32 lanes, each summing a block of the
// streams; the lengths stay in L1 for the other warps of the CTA).
//
// Flat cut: the tiles of all pairs laid end to end, `run` tiles per CTA, CTA b from tile f0 = b * run on.  A run may
// start in the middle of one pair and end in the middle of another.
//
// Aligned cut, taken for launches whose runs are short: a CTA that crosses from one pair into the next loads Q
// twice, merges its warps twice and usually folds two pairs, one after the other, at the very end of the launch,
// which costs about as much as three or four more tiles (measured: 32 streams x 2048 rows 14.9 -> 11.6 us per launch,
// x 4096 rows 19.4 -> 16.7 us).  So when every pair can be split into parts of at most r tiles for some r up to a
// quarter (and at most `slack` tiles) above the flat run, with no more parts than the grid has CTAs, each pair is split
// on its own into ceil(tiles / r) nearly equal parts and a CTA works on one part of one pair.  Staging the next pair's
// Q rows in shared memory ahead of time was tried for the flat cut and changed nothing: the cost is in the second
// merge and in two folds one after the other, not in the load.
//
// What the flat cut leaves on the table: CTAs that are given equal shares do not finish together (per-CTA timelines of
// a launch of 256 streams x 4096 rows: the last tile of a CTA anywhere between 59 and 82 us after the start, by SM
// rather than by what the CTA reads; 28 to 41 us on the ragged serving launch).  Dealing out only four fifths of the
// list as runs and leaving the rest as a pool of 4-tile chunks that CTAs take as they finish (an atomic counter, the
// chunk announced to the consumer warps through the ring stage of its first tile) was built and measured: 20 % slower
// (63 against 50 us on the serving launch).  Every chunk pays a Q load, a merge of the warps and a partial of its own,
// and with the tickets of a CTA taken together at its end all folds of the launch land in its last microseconds.
//
// Returns the number of tiles of this CTA (0: nothing to do) and where they start (w).  For the bookkeeping of cut
// pairs: flat cut -> aligned = false, run, f0; aligned cut -> aligned = true and part b0 .. b1 = the CTAs of this
// CTA's pair.
constexpr int kClusterMaxRun = 24;  // cluster mode: longest part of a pair, in tiles, that the bound may lead to
constexpr int kAlignedMaxRun = 64;  // beyond this a second Q load, merge and fold are small against the run itself
struct Cut {
    int  n_tiles, run, f0, b0, b1;
    bool aligned, any_empty;
};
// ceil(x / r) for 0 <= x, 1 <= r, x < 2^20, without an integer division: (x + r - 0.5) / r lies at least 0.5 / r away
// from an integer, far more than the error of the approximate quotient
__device__ __forceinline__ int ceil_div_small(int x, int r) { return __float2int_rd(__fdividef((float) (x + r) - 0.5f, (float) r)); }

__device__ __forceinline__ Cut cut_work_list(const DecodeParams & p, int lane, int slack, Walk & w) {
    constexpr int kKeep = 8;  // a lane keeps the tile counts of its streams in registers up to 8 (256 streams)
    const int n = p.n_streams, per = (n + 31) >> 5;
    const int lo = min(n, lane * per), hi = min(n, lo + per);
    const int HK = p.n_kv_heads, grid = (int) gridDim.x, b = (int) blockIdx.x;
    auto load_tiles = [&](int i) {
        const int s = p.order ? p.order[i] : i;
        return tiles_of(clamp_len(p, p.kv_len ? p.kv_len[s] : p.kv_len_const));
    };
    int kept[kKeep];
#pragma unroll
    for (int k = 0; k < kKeep; ++k) kept[k] = lo + k < hi ? load_tiles(lo + k) : 0;
    auto tiles_at = [&](int i) {  // i in [lo, hi)
        int v = 0;
        if (i - lo < kKeep) {
#pragma unroll
            for (int k = 0; k < kKeep; ++k) v = i - lo == k ? kept[k] : v;
        } else {
            v = load_tiles(i);
        }
        return v;
    };
    Cut  c;
    int  sum   = 0;
    bool empty = false;
#pragma unroll
    for (int k = 0; k < kKeep; ++k) {
        sum += kept[k];
        empty |= lo + k < hi && kept[k] == 0;
    }
    for (int i = lo + kKeep; i < hi; ++i) {
        const int tl = load_tiles(i);
        sum += tl;
        empty |= tl == 0;
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31) * HK;
    c.any_empty     = __any_sync(0xffffffffu, empty);
    c.run           = max(p.run_min, (total + grid - 1) / grid);
    c.f0            = b * c.run;
    c.aligned       = false;
    c.b0 = c.b1 = b;
    c.n_tiles       = 0;
    w.i = w.kvh = w.t = 0;

    if (c.run <= kAlignedMaxRun && total < (1 << 20)) {
        // crossing into a second pair costs a CTA about as much as `slack` tiles
        const int r_max = c.run + max(1, min(slack, c.run >> 2));
        for (int r = c.run; r <= r_max && !c.aligned; ++r) {
            int parts = 0;
#pragma unroll
            for (int k = 0; k < kKeep; ++k) parts += ceil_div_small(kept[k], r);
            for (int i = lo + kKeep; i < hi; ++i) parts += ceil_div_small(load_tiles(i), r);
            int pincl = parts;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, pincl, o);
                if (lane >= o) pincl += y;
            }
            const int all = __shfl_sync(0xffffffffu, pincl, 31) * HK;
            if (all > grid) continue;
            c.aligned = true;
            if (b >= all) return c;  // more CTAs than parts
            const int      pexcl = pincl - parts;
            const unsigned owner = __ballot_sync(0xffffffffu, b >= pexcl * HK && b < pincl * HK);
            const int      src   = __ffs(owner) - 1;
            int start = 0, count = 0, b0 = 0, b1 = 0;
            if (lane == src) {
                int acc = pexcl * HK;
                for (int i = lo; i < hi; ++i) {
                    const int tl = tiles_at(i), np = ceil_div_small(tl, r);
                    if (b < acc + np * HK) {
                        const int rem = b - acc, kvh = rem / np, j = rem - kvh * np;
                        w.i = i; w.kvh = kvh;
                        start = (j * tl) / np;
                        count = ((j + 1) * tl) / np - start;
                        b0 = b - j; b1 = b0 + np - 1;
                        break;
                    }
                    acc += np * HK;
                }
            }
            w.i       = __shfl_sync(0xffffffffu, w.i, src);
            w.kvh     = __shfl_sync(0xffffffffu, w.kvh, src);
            w.t       = __shfl_sync(0xffffffffu, start, src);
            c.n_tiles = __shfl_sync(0xffffffffu, count, src);
            c.b0      = __shfl_sync(0xffffffffu, b0, src);
            c.b1      = __shfl_sync(0xffffffffu, b1, src);
            walk_load(p, w);
            return c;
        }
    }

    if (c.f0 >= total) return c;
    c.n_tiles = min(total, c.f0 + c.run) - c.f0;
    const int      excl  = incl - sum;
    const unsigned owner = __ballot_sync(0xffffffffu, c.f0 >= excl * HK && c.f0 < incl * HK);
    const int      src   = __ffs(owner) - 1;
    if (lane == src) {
        int acc = excl;
        for (int i = lo; i < hi; ++i) {
            const int tl = tiles_at(i);
            if (c.f0 < (acc + tl) * HK) {
                const int rem = c.f0 - acc * HK;
                w.i = i; w.kvh = rem / tl; w.t = rem % tl;
                break;
            }
            acc += tl;
        }
    }
    w.i   = __shfl_sync(0xffffffffu, w.i, src);
    w.kvh = __shfl_sync(0xffffffffu, w.kvh, src);
    w.t   = __shfl_sync(0xffffffffu, w.t, src);
    walk_load(p, w);
    return c;
}

// Shared-memory ring: per stage one 64-row K tile and one 64-row V tile.
//   f16 : 2 x 8 KB (128-byte rows, 128-byte swizzle)                       -> 16 KB, 4 stages
//   q8_0: 2 x 4 KB bytes (64-byte rows, 64-byte swizzle) + 2 x 256 B scales, one span of the cache -> 9 KB (1 KB aligned), 6 stages
template <bool Q8> struct Ring {
    static constexpr int kStages     = Q8 ? 6 : 4;
    // q8_0 tiles are half the bytes and its arithmetic chain is longer: one more CTA hides it.  Measured per 256-stream
    // launch (one tile per pass): 4 CTAs x 96 registers x 5 stages 45.6 us; 5 x 72 x 4: 48.1 us; 3 x 105 x 6: 48.2 us.
    // Stages are held while their tile is worked on, so depth pays: 4 CTAs x 6 stages (the most that fits) 43.8 -> 42.5 us.
    static constexpr int kCtasPerSm  = Q8 ? 4 : 3;
    static constexpr int kDataBytes  = Q8 ? kKvTile * 64 : kKvTile * 128;
    static constexpr int kStageBytes = Q8 ? 9 * 1024 : 2 * kDataBytes;
    static constexpr int kTxBytes    = Q8 ? kQ8TileBytes : 2 * kDataBytes;
    static constexpr int kSmemBytes  = kStages * kStageBytes + 1024;
    // the warps of a CTA are merged through the stage of the tile they consumed last
    static_assert(kStageBytes >= kConsumerWarps * kMaxGqa * kPartialStride * 4, "a stage must hold the warps' partials");
};

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float half_lo(uint32_t x) { return __half2float(__ushort_as_half((unsigned short) (x & 0xffffu))); }
__device__ __forceinline__ float half_hi(uint32_t x) { return __half2float(__ushort_as_half((unsigned short) (x >> 16))); }

// Bytes of a q8_0 tile -> f16 tensor-core operands without arithmetic.  The tiles hold u = q + 128 (1..255); a byte
// in the low half of a 16-bit word whose high half is zero is the (subnormal) f16 number u * 2^-24, which mma.sync
// takes as it is.  `selector` picks which two bytes of the word go to the two halves (PRMT, 4 = a zero byte).  The
// products then carry (q + 128) * 2^-24: the factor goes into the step that consumes the accumulator anyway, and the
// 128 comes out of the accumulator as 128 times the sum of the other operand, taken once (K: the row sums of Q per
// 32-value block, known when Q is loaded; V: the running sums of the weights).
constexpr float kTwo24 = 16777216.0f, kTwoM24 = 1.0f / 16777216.0f;
__device__ __forceinline__ uint32_t u8_pair_to_half2(uint32_t bytes, uint32_t selector) { return __byte_perm(bytes, 0u, selector); }
// product of two packed pairs of halves, as bits
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2 *>(&a), *reinterpret_cast<const __half2 *>(&b));
    return *reinterpret_cast<const uint32_t *>(&r);
}

// The row that arrives with this call, stored by the producer warp (lane l holds elements 2l, 2l+1 of K
// and of V; converted exactly as kv_append_kernel converts them) before it requests the tile that
// contains the row: the bulk copy then delivers the new row like any other.  The proxy fence orders
// these generic-proxy stores before the async-proxy read of the copy issued after the warp barrier.
template <bool Q8>
__device__ __forceinline__ void store_arriving_row(float2 kk, float2 vv, uint8_t * k_pair, uint8_t * v_pair, uint8_t * ks_pair,
                                                   uint8_t * vs_pair, size_t nb_pos, int pos, int lane) {
    if constexpr (!Q8) {
        *reinterpret_cast<uint32_t *>(k_pair + (size_t) pos * nb_pos + lane * 4) = pack_half2(kk.x, kk.y);
        *reinterpret_cast<uint32_t *>(v_pair + (size_t) pos * nb_pos + lane * 4) = pack_half2(vv.x, vv.y);
    } else {
        char2 qk, qv;
        float dk, dv;
        q8_0_quantize_pair(kk.x, kk.y, qk, dk);
        q8_0_quantize_pair(vv.x, vv.y, qv, dv);
        const size_t tile = q8_tile_off(pos);
        *reinterpret_cast<uchar2 *>(k_pair + tile + q8_byte_off(pos, 2 * lane)) = q8_0_biased(qk);
        *reinterpret_cast<uchar2 *>(v_pair + tile + q8_byte_off(pos, 2 * lane)) = q8_0_biased(qv);
        if ((lane & 15) == 0) {
            *reinterpret_cast<__half *>(ks_pair + tile + q8_scale_off(pos, lane >> 4)) = __float2half_rn(dk);
            *reinterpret_cast<__half *>(vs_pair + tile + q8_scale_off(pos, lane >> 4)) = __float2half_rn(dv);
        }
    }
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncwarp();
}

// Cluster mode: distributed shared memory.  The address of `addr` (of this CTA's shared memory) in the CTA of rank
// `rank`, stores to such an address, an arrival on a barrier of that CTA that publishes this thread's (and, after a
// CTA barrier, its CTA's) earlier stores, and the bounded wait that goes with it.
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void dsmem_st2(uint32_t addr, float a, float b) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void dsmem_arrive(uint32_t bar) {
    asm volatile("fence.acq_rel.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 15u) == 0 && clock64() - t0 > kWaitCycles) return false;
    }
}

__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

// The fold of NP pairs at once by one thread (head hh of each pair, output columns d0 .. d0+3): the partials of a pair
// (runs b0 .. b1 of the launch; the run that holds the pair's first tile wrote its slot 1, the others their slot 0) are
// read W at a time, the loads of a batch issued together (each is a round trip to L2, and a pair may have been cut 17
// ways).  pend[k] = stream, kv head, b0, b1.
template <int NP, int W>
__device__ __forceinline__ void fold_pairs(const DecodeParams & p, const int (*pend)[4], int k0, int hh, int d0) {
    int   b0[NP], b1[NP];
    float M[NP], L[NP], acc[NP][4];
    int   span = 0;
#pragma unroll
    for (int k = 0; k < NP; ++k) {
        b0[k] = pend[k0 + k][2];
        b1[k] = pend[k0 + k][3];
        span  = max(span, b1[k] - b0[k] + 1);
        M[k] = -INFINITY; L[k] = 0.0f;
        acc[k][0] = acc[k][1] = acc[k][2] = acc[k][3] = 0.0f;
    }
    for (int c = 0; c < span; c += W) {
        float  mc[NP][W], lc[NP][W];
        float2 lo[NP][W], hi[NP][W];
#pragma unroll
        for (int k = 0; k < NP; ++k)
#pragma unroll
            for (int u = 0; u < W; ++u) {
                const int     cc = min(b0[k] + c + u, b1[k]);
                const float * pc = p.partial + ((size_t) cc * 2 + (cc == b0[k] ? 1 : 0)) * p.gqa * kPartialStride + hh * kPartialStride;
                mc[k][u] = b0[k] + c + u <= b1[k] ? __ldcg(pc) : -INFINITY;
                lc[k][u] = __ldcg(pc + 1);
                lo[k][u] = __ldcg(reinterpret_cast<const float2 *>(pc + 2 + d0));
                hi[k][u] = __ldcg(reinterpret_cast<const float2 *>(pc + 4 + d0));
            }
        // the running maximum is raised partial by partial, in list order: the arithmetic (and so every bit of the
        // result) does not depend on W, i.e. not on whether this CTA happened to fold one pair or two
#pragma unroll
        for (int k = 0; k < NP; ++k)
#pragma unroll
            for (int u = 0; u < W; ++u) {
                if (mc[k][u] == -INFINITY) continue;  // past the pair's last partial, or a partial that saw nothing
                const float Mn = fmaxf(M[k], mc[k][u]);
                const float fo = exp2f(M[k] - Mn);  // M == -inf: 0
                const float fw = exp2f(mc[k][u] - Mn);
                M[k]      = Mn;
                L[k]      = L[k] * fo + lc[k][u] * fw;
                acc[k][0] = acc[k][0] * fo + lo[k][u].x * fw;
                acc[k][1] = acc[k][1] * fo + lo[k][u].y * fw;
                acc[k][2] = acc[k][2] * fo + hi[k][u].x * fw;
                acc[k][3] = acc[k][3] * fo + hi[k][u].y * fw;
            }
    }
#pragma unroll
    for (int k = 0; k < NP; ++k) {
        const int   stream = pend[k0 + k][0], head = pend[k0 + k][1] * p.gqa + hh;
        const float inv    = L[k] > 0.0f ? 1.0f / L[k] : 0.0f;
        *reinterpret_cast<float4 *>(p.dst + ((size_t) stream * p.n_heads + head) * kHeadDim + d0) =
            make_float4(acc[k][0] * inv, acc[k][1] * inv, acc[k][2] * inv, acc[k][3] * inv);
    }
}

template <bool Q8>
__global__ void __launch_bounds__(kThreads, Ring<Q8>::kCtasPerSm)
decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const DecodeParams p) {
    using R = Ring<Q8>;
    constexpr int kStages = R::kStages;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * kStages];
    __shared__ uint64_t xbar;  // cluster mode, first CTA of a cluster: the CTAs of the pair have delivered their partials
    __shared__ int      abort_flag;
    __shared__ int      fold_flag;
    // pairs this run holds a part of (at most two: one that began in an earlier run, one that goes on in a later
    // one): stream, kv head, first and last run of the pair.  Their tickets are taken together when the run ends.
    __shared__ int      pending[2][4];
    __shared__ int      n_pending;
    __shared__ int      cut_note[5];  // what thread 0 needs of the cut when it records a cut pair (kept out of the registers)

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *      smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) DECODE_TRACE(0);

    // set-up that reads nothing the previous kernel of the stream wrote: done while that kernel drains
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
    if (tid == 0) {
        abort_flag = 0;
        fold_flag  = 0;
        n_pending  = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumerWarps);
        }
        fence_mbar_init();
    }
    if constexpr (!Q8) {
        if (tid == kConsumerWarps * 32) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
        }
    }
    const int n_stages = kStages == 4 ? p.n_stages : kStages;  // only the f16 kernel gives ring stages up (cluster mode)
    Walk      w;
    int       n_tiles = 0, parts = 1, rank = 0;
    bool      any_empty = false;
    // (q8_0 launches do not use the cluster mode: with two of its six ring stages given up for the partials the kernel
    // was slower than with tickets, 13.7 against 11.7 us at 32 streams x 2048 rows.)
    constexpr bool kClusterMode = !Q8;
    if (kClusterMode && p.cluster > 0) {
        // One cluster per pair: no list to cut.  The pair's tiles are split into nearly equal parts of four tiles or
        // more, one per CTA of the cluster as far as they go; the other CTAs of the cluster have nothing to do.
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
        const int pair = (int) blockIdx.x / p.cluster;
        w.i = pair / p.n_kv_heads; w.kvh = pair - w.i * p.n_kv_heads;
        walk_load(p, w);
        parts   = max(1, min(p.cluster, w.tiles >> 2));
        w.t     = rank < parts ? (rank * w.tiles) / parts : 0;
        n_tiles = rank < parts ? ((rank + 1) * w.tiles) / parts - w.t : 0;
        if (tid == 0) mbar_init(smem_u32(&xbar), parts);
        fence_mbar_init();
        __syncthreads();
        // every CTA's barrier is initialised before anyone can reach it
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (!p.early) {
            pdl_wait();
            pdl_launch_dependents();
        }
        if (tid == 0) DECODE_TRACE(1);
        if (rank >= parts) {
            if (p.early) {  // every CTA of the grid passes the dependency wait
                pdl_wait();
                pdl_launch_dependents();
            }
            return;
        }
        if (w.tiles == 0) {  // nothing visible: the result is zeros (ops.cpp:8333); rank 0 is the only part
            if (p.early) {
                pdl_wait();
                pdl_launch_dependents();
            }
            if (warp < kConsumerWarps) {
                float4 * out = reinterpret_cast<float4 *>(p.dst + ((size_t) w.stream * p.n_heads + (size_t) w.kvh * p.gqa) * kHeadDim);
                for (int j = tid; j < p.gqa * kHeadDim / 4; j += kConsumerWarps * 32) out[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            return;
        }
    } else {
    __syncthreads();
    // Dependency wait.  Every thread passes it before it triggers the launch of the next kernel, and
    // CTA 0 always passes it, so a kernel that starts early can rely on everything before its
    // predecessor being complete.
    if (!p.early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const Cut cut = cut_work_list(p, lane, Q8 ? 3 : 4, w);
    n_tiles   = cut.n_tiles;
    any_empty = cut.any_empty;
    if (tid == 0) {
        cut_note[0] = cut.aligned; cut_note[1] = cut.f0; cut_note[2] = cut.run; cut_note[3] = cut.b0; cut_note[4] = cut.b1;
        DECODE_TRACE(1);
    }
    if (n_tiles == 0 && blockIdx.x != 0) return;  // more CTAs than runs: nothing to do
    }

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer
        // All lanes walk the run (the arriving row is converted by the whole warp); lane 0 issues the copies.
        bool waited = !p.early;
        int  issued = 0;
        for (int it = 0; it < n_tiles; ++it) {
            const bool append_here = p.k_new != nullptr && w.t == w.tiles - 1;  // the arriving row lies in the pair's last tile
            if (!waited && (append_here || it >= p.early_tiles)) {  // the first tiles were requested while the previous kernel drained
                pdl_wait();
                pdl_launch_dependents();
                waited = true;
            }
            if (append_here) {
                const int raw = p.kv_len[w.stream];
                if (raw > p.max_len) {  // the stream has outgrown its rows: nothing is written
                    if (lane == 0) atomicOr(p.status, kStatusBadState);
                } else {
                    const size_t src = (size_t) w.stream * p.new_nb_stream + (size_t) w.kvh * p.new_nb_head + lane * 8;
                    float2       kk  = *reinterpret_cast<const float2 *>(p.k_new + src);
                    const float2 vv  = *reinterpret_cast<const float2 *>(p.v_new + src);
                    if (p.rope != nullptr) {
                        // lane l holds elements 2l, 2l+1; their partners (32 further, or 32 back) sit in lane l ^ 16.
                        // Separate multiplies and adds, in the operand order of the reference's rotate_pairs.
                        const float2 * tb = p.rope + (size_t) w.stream * (kHeadDim / 2) + 2 * (lane & 15);
                        const float2   r0 = tb[0], r1 = tb[1];
                        const float    ox = __shfl_xor_sync(0xffffffffu, kk.x, 16), oy = __shfl_xor_sync(0xffffffffu, kk.y, 16);
                        if (lane < 16) {  // x0 = mine, x1 = partner: x0*cos - x1*sin
                            kk.x = __fsub_rn(__fmul_rn(kk.x, r0.x), __fmul_rn(ox, r0.y));
                            kk.y = __fsub_rn(__fmul_rn(kk.y, r1.x), __fmul_rn(oy, r1.y));
                        } else {          // x0 = partner, x1 = mine: x0*sin + x1*cos
                            kk.x = __fadd_rn(__fmul_rn(ox, r0.y), __fmul_rn(kk.x, r0.x));
                            kk.y = __fadd_rn(__fmul_rn(oy, r1.y), __fmul_rn(kk.y, r1.x));
                        }
                    }
                    const size_t pair = (size_t) w.stream * p.nb_stream + (size_t) w.kvh * p.nb_head;
                    store_arriving_row<Q8>(kk, vv, p.k_rows + pair, p.v_rows + pair, p.k_scales + pair, p.v_scales + pair, p.nb_pos, w.len - 1, lane);
                }
            }
            int good = 1;
            if (lane == 0) {
                const int s = it % n_stages;
                if (it >= n_stages && !mbar_wait_bounded(empty0 + 8 * s, ((it / n_stages) - 1) & 1)) {
                    atomicOr(p.status, kStatusTimeout);
                    atomicExch(&abort_flag, 1);
                    good = 0;
                }
                if (good && *reinterpret_cast<volatile int *>(&abort_flag)) good = 0;
                if (good) {
                    const uint32_t sb  = smem_base + s * R::kStageBytes;
                    const uint32_t bar = full0 + 8 * s;
                    const int      pos = w.t * kKvTile;
                    mbar_expect_tx(bar, R::kTxBytes);
                    if constexpr (Q8) {  // the tile is one span of the cache, already in the layout of the stage
                        const uint8_t * src = p.q8_tiles + (size_t) w.stream * p.q8_nb_stream + (size_t) w.kvh * p.q8_nb_head + (size_t) w.t * kQ8TileBytes;
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(sb),
                                     "l"(src), "r"((uint32_t) kQ8TileBytes), "r"(bar)
                                     : "memory");
                    } else {
                        tma_load_5d(sb, &map_k, bar, 0, pos, w.kvh, w.stream, p.layer);
                        tma_load_5d(sb + R::kDataBytes, &map_v, bar, 0, pos, w.kvh, w.stream, p.layer);
                    }
                }
            }
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) break;
            if (lane == 0 && it == 0) DECODE_TRACE(6);
            issued = it + 1;
            if (++w.t == w.tiles && it + 1 < n_tiles) walk_next_pair(p, w);
        }
        if (!waited) {
            pdl_wait();
            pdl_launch_dependents();
        }
#ifdef VOX_ATTN_DEVELOPER
        if (lane == 0 && blockIdx.x < kTraceCtas) {  // which SM the CTA ran on
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            g_decode_trace[p.layer & 1][blockIdx.x][7] = smid + 1;
        }
#endif
        if (lane == 0 && *reinterpret_cast<volatile int *>(&abort_flag)) {
            // consumers gave up: let the copies already issued land before the CTA retires
            for (int i = max(0, issued - n_stages); i < issued; ++i)
                mbar_wait_bounded(full0 + 8 * (i % n_stages), (i / n_stages) & 1);
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    if (p.early) {  // Q is written by the kernel before this one
        pdl_wait();
        pdl_launch_dependents();
    }
    if (tid == 0) DECODE_TRACE(2);
    if (blockIdx.x == 0 && any_empty) {
        // a stream with no visible rows has no tile in the list: its result is zeros (ops.cpp:8333)
        for (int i = 0; i < p.n_streams; ++i) {
            const int len = clamp_len(p, p.kv_len ? p.kv_len[i] : p.kv_len_const);
            if (len > 0) continue;
            float4 * out = reinterpret_cast<float4 *>(p.dst + (size_t) i * p.n_heads * kHeadDim);
            for (int j = tid; j < p.n_heads * kHeadDim / 4; j += kConsumerWarps * 32) out[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }

    // per-lane ldmatrix row/chunk selectors (see the fragment layouts of mma.m16n8k16)
    const int k_row = 16 * warp + ((lane >> 4) << 3) + (lane & 7), k_chk = (lane >> 3) & 1;
    const int v_row = 16 * warp + (((lane >> 3) & 1) << 3) + (lane & 7), v_chk = lane >> 4;

    // q8_0: byte offsets inside a stage that do not change from tile to tile.  Row 16*warp + 8j + g of the K bytes:
    // 16-byte chunk (2b + t/2) ^ ((row / 2) % 4), where 8j drops out of the swizzle term and b only flips bit 1 of the
    // chunk, so block 1 is the same offset with bit 5 flipped and j adds 512; likewise the two chunk pairs of V.
    const uint32_t k_off = (16 * warp + g) * 64 + ((((t >> 1)) ^ ((g >> 1) & 3)) << 4) + ((t & 1) << 3);
    const uint32_t v_off = v_row * 64 + ((v_chk ^ ((v_row >> 1) & 3)) << 4);
    const uint32_t s_off = (16 * warp + 2 * t) * 4;  // scales of positions 8j + 2t, 8j + 2t + 1: + 32j

    bool ok = true;
    int  it = 0;                 // tiles of the run consumed so far
    int  cstage = 0, cphase = 0; // ring stage and barrier phase of the next tile to consume
    int  last_stage = 0;         // stage of the tile consumed last
    while (it < n_tiles && ok) {
        const int seg    = min(w.tiles - w.t, n_tiles - it);  // tiles of this pair inside the run
        if (seg <= 0) {  // the lengths moved under the launch: the cut no longer matches them
            if (tid == 0) atomicOr(p.status, kStatusBadState);
            break;
        }
        const int stream = w.stream, kvh = w.kvh, c1 = w.len;

        // Q fragments of the four k-steps: rows 0-7 = hi part of the group's heads, rows 8-15 = lo part.
        // The 64 head dimensions may be fed to the MMAs in any order as long as K uses the same one:
        //   f16 : k-step c covers d = 16c .. 16c+15 in natural order (K fragments come from ldmatrix);
        //   q8_0: k-step s covers the 8 bytes per lane that one 64-bit shared load returns,
        //         d = 32*(s/2) + 8t + 4*(s%2) + {0,1,2,3}, so that k-steps 0,1 / 2,3 stay inside one
        //         32-value quantisation block and the block scale can be applied to their accumulator.
        uint32_t qa[4][4];
        float    q_bias[2] = {0.0f, 0.0f};  // q8_0: what the +128 of the K bytes contributes to a score, per 32-value block
        {
            const int     head = kvh * p.gqa + min(g, p.gqa - 1);
            const float * qrow = reinterpret_cast<const float *>(p.q + (size_t) stream * p.q_nb_stream + (size_t) head * p.q_nb_head);
            const float   live = g < p.gqa ? p.scale_log2 : 0.0f;
            float xs[4][4];  // k-step c: elements d0, d0+1, d1, d1+1
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int d0 = Q8 ? 32 * (c >> 1) + 8 * t + 4 * (c & 1) : 16 * c + 2 * t;
                const int d1 = Q8 ? d0 + 2 : d0 + 8;
                const float2 x = *reinterpret_cast<const float2 *>(qrow + d0);
                const float2 y = *reinterpret_cast<const float2 *>(qrow + d1);
                xs[c][0] = x.x; xs[c][1] = x.y; xs[c][2] = y.x; xs[c][3] = y.y;
            }
            if (p.rope != nullptr) {
                // in both orders k-steps c and c+2 hold each other's partners (d and d + 32)
                const float2 * tb = p.rope + (size_t) stream * (kHeadDim / 2);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int d0 = Q8 ? 8 * t + 4 * c : 16 * c + 2 * t;
                    const int d1 = Q8 ? d0 + 2 : d0 + 8;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 r  = tb[(e < 2 ? d0 : d1) + (e & 1)];
                        const float  x0 = xs[c][e], x1 = xs[c + 2][e];
                        xs[c][e]     = __fsub_rn(__fmul_rn(x0, r.x), __fmul_rn(x1, r.y));
                        xs[c + 2][e] = __fadd_rn(__fmul_rn(x0, r.y), __fmul_rn(x1, r.x));
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float h0, l0, h1, l1, h2, l2, h3, l3;
                split_hi_lo(xs[c][0] * live, h0, l0);
                split_hi_lo(xs[c][1] * live, h1, l1);
                split_hi_lo(xs[c][2] * live, h2, l2);
                split_hi_lo(xs[c][3] * live, h3, l3);
                qa[c][0] = pack_half2(h0, h1);
                qa[c][1] = pack_half2(l0, l1);
                qa[c][2] = pack_half2(h2, h3);
                qa[c][3] = pack_half2(l2, l3);
                if constexpr (Q8) q_bias[c >> 1] += ((h0 + l0) + (h1 + l1)) + ((h2 + l2) + (h3 + l3));
            }
            if constexpr (Q8) {
                // k-steps 2b, 2b+1 hold the lane's share of block b: summed over the four lanes of a head, times 128 * 2^-24,
                // that is what the bias of the K bytes adds to every score of the block
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    q_bias[b] += __shfl_xor_sync(0xffffffffu, q_bias[b], 1);
                    q_bias[b] += __shfl_xor_sync(0xffffffffu, q_bias[b], 2);
                    q_bias[b] *= 128.0f * kTwoM24;
                }
            }
        }
        float o[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        // q8_0: sums of the V-scaled weights (accumulator tile of the product with ones: [0] = [1] = head g with the
        // scales of block 0, [2] = [3] = with those of block 1)
        float v_bias[4] = {0.0f, 0.0f, 0.0f, 0.0f};

        // Tiles per pass of a consumer warp: one.  Two (both cache types were tried: two independent tiles in one pass
        // give the scheduler something to overlap the dependency chains with) measured the same or slower: f16 50.6
        // against 49.9 us per 256-stream launch (it holds two ring stages at a time), q8_0 43.8 against 43.9 us at four
        // CTAs per SM, where the 96 registers a thread may have cannot keep both chains in flight.
#ifndef VOX_DECODE_U_F16
#define VOX_DECODE_U_F16 1
#endif
#ifndef VOX_DECODE_U_Q8
#define VOX_DECODE_U_Q8 1
#endif
        constexpr int U = Q8 ? VOX_DECODE_U_Q8 : VOX_DECODE_U_F16;
        for (int i = 0; i < seg && ok; i += U) {
            int  st[U], p0[U];
            bool have[U], act[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                have[u] = i + u < seg;
                st[u]   = cstage + u < n_stages ? cstage + u : cstage + u - n_stages;
                p0[u]   = (w.t + i + u) * kKvTile + 16 * warp;
                act[u]  = have[u] && p0[u] < c1;
                if (have[u] && !mbar_wait_bounded(full0 + 8 * st[u], cstage + u < n_stages ? cphase : cphase ^ 1)) {
                    *reinterpret_cast<volatile int *>(&abort_flag) = 1;
                    ok = false;
                }
            }
            if (!ok) break;
            if (tid == 0 && it == 0 && i == 0) DECODE_TRACE(3);
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_DECODE_NOMATH)  // developer build: the copy structure alone
            if (false) {
#else
            if (act[0]) {
#endif
                float sv[U][2][2];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t kb = smem_base + st[u] * R::kStageBytes;
                    if (!act[u]) {
                        sv[u][0][0] = sv[u][0][1] = sv[u][1][0] = sv[u][1][1] = -INFINITY;
                        continue;
                    }
                    if constexpr (!Q8) {
                        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4(kb + k_row * 128 + (((2 * c + k_chk) ^ (k_row & 7)) << 4), b0, b1, b2, b3);
                            mma_16816(sc[0], qa[c], b0, b1);
                            mma_16816(sc[1], qa[c], b2, b3);
                        }
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            sv[u][j][0] = sc[j][0] + sc[j][2];
                            sv[u][j][1] = sc[j][1] + sc[j][3];
                        }
                    } else {
                        const uint32_t ksc = kb + 2 * R::kDataBytes;
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            // one accumulator per 32-value block; the hi rows start at minus the bias of the block
                            float     sc[2][4] = {{-q_bias[0], -q_bias[0], 0.f, 0.f}, {-q_bias[1], -q_bias[1], 0.f, 0.f}};
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_ABL_NOK)
                            if (false)
#endif
#pragma unroll
                            for (int b = 0; b < 2; ++b) {
                                const uint2 raw = lds64(kb + ((k_off ^ (b << 5)) + 512 * j));
                                mma_16816(sc[b], qa[2 * b], u8_pair_to_half2(raw.x, 0x4140), u8_pair_to_half2(raw.x, 0x4342));
                                mma_16816(sc[b], qa[2 * b + 1], u8_pair_to_half2(raw.y, 0x4140), u8_pair_to_half2(raw.y, 0x4342));
                            }
                            // scales of positions 8j+2t and 8j+2t+1, both blocks: four consecutive halves
                            const uint2 ds = lds64(ksc + s_off + 32 * j);
                            sv[u][j][0] = ((sc[0][0] + sc[0][2]) * half_lo(ds.x) + (sc[1][0] + sc[1][2]) * half_hi(ds.x)) * kTwo24;
                            sv[u][j][1] = ((sc[0][1] + sc[0][3]) * half_lo(ds.y) + (sc[1][1] + sc[1][3]) * half_hi(ds.y)) * kTwo24;
                        }
                    }
                }
                float tmax = -INFINITY;
                // only a pair's last tile can hold positions past its length, and masks are rare: every other tile
                // takes the short way (the same for all lanes of the warp)
                bool edge = p.mask != nullptr;
#pragma unroll
                for (int u = 0; u < U; ++u) edge |= !act[u] || p0[u] + 16 > c1;
                if (!edge) {
#pragma unroll
                    for (int u = 0; u < U; ++u)
#pragma unroll
                        for (int j = 0; j < 2; ++j) tmax = fmaxf(tmax, fmaxf(sv[u][j][0], sv[u][j][1]));
                } else {
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int pos = p0[u] + 8 * j + 2 * t;  // this lane's two positions: pos, pos + 1
                        if (p.mask != nullptr && pos < c1) {
                            // additive mask in natural units (the scores are in units of log2 e): the row of this lane's head
                            // (rows g and g + 8 of the A operand are the same head); the pointer is rebuilt here rather than
                            // kept in registers across the tile loop, which the q8_0 form cannot spare
                            const int      head = kvh * p.gqa + min(g, p.gqa - 1);
                            const __half * mrow = reinterpret_cast<const __half *>(p.mask + (size_t) (head % p.mask_ne2) * p.mask_nb_head +
                                                                                   (size_t) (stream % p.mask_ne3) * p.mask_nb_stream);
                            const float2 mv = make_float2(__half2float(mrow[pos]), pos + 1 < c1 ? __half2float(mrow[pos + 1]) : 0.0f);
                            sv[u][j][0] += mv.x * 1.4426950408889634f;
                            sv[u][j][1] += mv.y * 1.4426950408889634f;
                        }
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            sv[u][j][e] = pos + e < c1 ? sv[u][j][e] : -INFINITY;
                            tmax        = fmaxf(tmax, sv[u][j][e]);
                        }
                    }
                }
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m, tmax);
                const float alpha = m_new == -INFINITY ? 1.0f : ex2_approx(m - m_new);
                const float m_use = m_new == -INFINITY ? 0.0f : m_new;
                m                 = m_new;
                float pr[U][2][2];
                float psum_q8 = 0.0f;
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        pr[u][j][0] = ex2_approx(sv[u][j][0] - m_use);
                        pr[u][j][1] = ex2_approx(sv[u][j][1] - m_use);
                        psum_q8 += pr[u][j][0] + pr[u][j][1];
                    }
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {  // after the first tiles the running maxima rarely move
#pragma unroll
                    for (int n = 0; n < 8; ++n) {
                        o[n][0] *= alpha; o[n][1] *= alpha; o[n][2] *= alpha; o[n][3] *= alpha;
                    }
                    v_bias[0] *= alpha; v_bias[2] *= alpha;
                }
                if constexpr (!Q8) {
                    float psum = 0.0f;
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (!act[u]) continue;
                        const uint32_t vb = smem_base + st[u] * R::kStageBytes + R::kDataBytes;
                        uint32_t       pa[4];
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            float h0, l0, h1, l1;
                            split_hi_lo(pr[u][j][0], h0, l0);
                            split_hi_lo(pr[u][j][1], h1, l1);
                            pa[2 * j]     = pack_half2(h0, h1);
                            pa[2 * j + 1] = pack_half2(l0, l1);
                            psum += (h0 + l0) + (h1 + l1);
                        }
#pragma unroll
                        for (int n2 = 0; n2 < 4; ++n2) {
                            uint32_t b0, b1, b2, b3;
                            ldmatrix_x4_trans(vb + v_row * 128 + (((2 * n2 + v_chk) ^ (v_row & 7)) << 4), b0, b1, b2, b3);
                            mma_16816(o[2 * n2], pa, b0, b1);
                            mma_16816(o[2 * n2 + 1], pa, b2, b3);
                        }
                    }
                    l = l * alpha + psum;
                } else {
                    l = l * alpha + psum_q8;
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (!act[u]) continue;
                        const uint32_t kb = smem_base + st[u] * R::kStageBytes, vb = kb + R::kDataBytes;
                        // V scales are folded into the weights.  The two 32-column blocks of a row have different scales:
                        // rows 0-7 of the A operand carry the weights times the scale of block 0, rows 8-15 times the scale
                        // of block 1 (products in f16: twice 2^-11 relative, far inside the q8_0 tolerance), so one operand
                        // serves both chunk pairs; of each accumulator tile the half that belongs to its block is kept.
                        const uint32_t vsc = kb + 2 * R::kDataBytes + kKvTile * 4;
                        uint32_t       pa[4];
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint2    ds  = lds64(vsc + s_off + 32 * j);  // halves: (pos: b0, b1), (pos + 1: b0, b1)
                            const uint32_t ph  = pack_half2(pr[u][j][0], pr[u][j][1]);
                            const uint32_t sb0 = __byte_perm(ds.x, ds.y, 0x5410), sb1 = __byte_perm(ds.x, ds.y, 0x7632);
                            pa[2 * j]     = hmul2_bits(ph, sb0);
                            pa[2 * j + 1] = hmul2_bits(ph, sb1);
                        }
                        // what the +128 of the V bytes multiplies: the sums of these very operands, from one more MMA
                        // against a tile of ones (every column of its result is the row sum)
                        mma_16816(v_bias, pa, 0x3c003c00u, 0x3c003c00u);
                        // ldmatrix.trans on 16-bit units keeps byte pairs together: a register holds
                        // V[2t][2g], V[2t][2g+1], V[2t+1][2g], V[2t+1][2g+1] of one 16-column chunk, i.e. the B
                        // fragments of an "even columns" tile (bytes 0,2) and an "odd columns" tile (bytes 1,3).
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_ABL_NOV)
                        if (false)
#endif
#pragma unroll
                        for (int cp = 0; cp < 2; ++cp) {
                            uint32_t r0, r1, r2, r3;
                            ldmatrix_x4_trans(vb + (v_off ^ (cp << 5)), r0, r1, r2, r3);
                            mma_16816(o[4 * cp + 0], pa, u8_pair_to_half2(r0, 0x4240), u8_pair_to_half2(r1, 0x4240));
                            mma_16816(o[4 * cp + 1], pa, u8_pair_to_half2(r0, 0x4341), u8_pair_to_half2(r1, 0x4341));
                            mma_16816(o[4 * cp + 2], pa, u8_pair_to_half2(r2, 0x4240), u8_pair_to_half2(r3, 0x4240));
                            mma_16816(o[4 * cp + 3], pa, u8_pair_to_half2(r2, 0x4341), u8_pair_to_half2(r3, 0x4341));
                        }
                    }
                }
            }
            __syncwarp();
            // stages go back to the producer as soon as their tile is consumed, except the last one of the
            // pair's part: the warps are merged through it first
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (!have[u]) continue;
                if (i + u != seg - 1 && lane == 0) mbar_arrive(empty0 + 8 * st[u]);
                last_stage = st[u];
                if (++cstage == n_stages) { cstage = 0; cphase ^= 1; }
            }
        }

        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if constexpr (Q8) {
            // the accumulators hold sum(w * (v + 128)) * 2^-24: back to sum(w * v).  Block 0 (tiles 0-3) is in the rows
            // of the first half of the operand, block 1 (tiles 4-7) in those of the second; the other half of a tile
            // (the other block's scales on this block's bytes) is dropped.
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float b = -128.0f * v_bias[n < 4 ? 0 : 2];
                o[n][0] = fmaf(n < 4 ? o[n][0] : o[n][2], kTwo24, b);
                o[n][1] = fmaf(n < 4 ? o[n][1] : o[n][3], kTwo24, b);
                o[n][2] = o[n][3] = 0.0f;
            }
        }
        if (tid == 0 && it + seg >= n_tiles) DECODE_TRACE(4);

        if (*reinterpret_cast<volatile int *>(&abort_flag)) atomicOr(p.status, kStatusTimeout);  // raised here, once: the tile loop stays short
        // ---- merge the four warps through the stage of the last tile (all of them are done with it after the barrier)
        named_bar_sync(1, kConsumerWarps * 32);
        if (!ok || *reinterpret_cast<volatile int *>(&abort_flag)) return;
        float *   scratch    = reinterpret_cast<float *>(smem_gen + last_stage * R::kStageBytes);
        {
            float * mine = scratch + (warp * 8 + g) * kPartialStride;
            if (t == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                // output column of accumulator registers 0/2 and 1/3 of tile n
                //   f16 : tile n = columns 8n .. 8n+7, this lane holds 8n+2t and 8n+2t+1
                //   q8_0: tile n = chunk n/2 (16 columns), parity n%2: this lane holds 16(n/2)+4t+(n%2) and +2
                const int da = Q8 ? 16 * (n >> 1) + 4 * t + (n & 1) : 8 * n + 2 * t;
                const int db = Q8 ? da + 2 : da + 1;
                mine[2 + da] = o[n][0] + o[n][2];
                mine[2 + db] = o[n][1] + o[n][3];
            }
        }
        named_bar_sync(1, kConsumerWarps * 32);
        const bool whole = w.t == 0 && seg == w.tiles;  // the pair lies inside this run: no partials
        // a pair cut across runs: the run that holds its first tile uses the CTA's slot 1, every other run slot 0
        float *    slot  = p.partial + ((size_t) blockIdx.x * 2 + (w.t == 0 ? 1 : 0)) * p.gqa * kPartialStride;
        {
            const int hh = tid >> 4, d0 = (tid & 15) * 4;  // 8 heads x 16 threads x 4 values
            if (hh < p.gqa) {
                float M = -INFINITY;
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) M = fmaxf(M, scratch[(ww * 8 + hh) * kPartialStride]);
                float L = 0.0f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ww = 0; ww < kConsumerWarps; ++ww) {
                    const float * src = scratch + (ww * 8 + hh) * kPartialStride;
                    const float   fw  = src[0] == -INFINITY ? 0.0f : exp2f(src[0] - M);
                    L += src[1] * fw;
#pragma unroll
                    for (int d = 0; d < 4; ++d) acc[d] += src[2 + d0 + d] * fw;
                }
                if (whole) {
                    const int   head = kvh * p.gqa + hh;
                    const float inv  = L > 0.0f ? 1.0f / L : 0.0f;  // nothing visible -> zeros, as the reference
                    *reinterpret_cast<float4 *>(p.dst + ((size_t) stream * p.n_heads + head) * kHeadDim + d0) =
                        make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
                } else if (kClusterMode && p.cluster > 0) {
                    // into the first CTA of the cluster: slot `rank`, behind its ring
                    const uint32_t dstp = dsmem_addr(smem_base + n_stages * R::kStageBytes + (uint32_t) ((rank * kMaxGqa + hh) * kPartialStride) * 4, 0);
                    if ((tid & 15) == 0) dsmem_st2(dstp, M, L);
                    dsmem_st2(dstp + (2 + d0) * 4, acc[0], acc[1]);
                    dsmem_st2(dstp + (4 + d0) * 4, acc[2], acc[3]);
                } else {
                    float * dstp = slot + hh * kPartialStride;
                    if ((tid & 15) == 0) { dstp[0] = M; dstp[1] = L; }
                    *reinterpret_cast<float2 *>(dstp + 2 + d0)     = make_float2(acc[0], acc[1]);
                    *reinterpret_cast<float2 *>(dstp + 2 + d0 + 2) = make_float2(acc[2], acc[3]);
                }
            }
        }
        // the stage is free once every thread has read the scratch; the generic-proxy accesses above are ordered
        // before the bulk copy that refills it
        fence_proxy_async_smem();
        if (!whole && !(kClusterMode && p.cluster > 0) && tid == 0 && n_pending < 2) {  // a cut pair: its ticket is taken when the run ends
            const volatile int * cn = cut_note;
            const int f_pair = cn[1] + it - w.t;  // flat cut: the pair's first tile in the list
            int *     pd     = pending[n_pending];
            pd[0] = stream; pd[1] = kvh;
            pd[2] = cn[0] ? cn[3] : f_pair / cn[2];
            pd[3] = cn[0] ? cn[4] : (f_pair + w.tiles - 1) / cn[2];
            n_pending += 1;
        }
        named_bar_sync(1, kConsumerWarps * 32);
        if (lane == 0) mbar_arrive(empty0 + 8 * last_stage);

        it += seg;
        w.t += seg;
        if (w.t == w.tiles && it < n_tiles) walk_next_pair(p, w);
    }
    if (kClusterMode && p.cluster > 0 && parts > 1 && ok) {
        // Every thread's piece of the partial is on its way to the first CTA (the barrier that ends the merge has ordered
        // the stores before thread 0's arrival, which publishes them cluster-wide).  The first CTA folds when all parts
        // have arrived: no round trip to L2, no ticket.
        if (tid == 0) dsmem_arrive(dsmem_addr(smem_u32(&xbar), 0));
        if (rank == 0) {
            if (!mbar_wait_cluster_bounded(smem_u32(&xbar), 0)) {
                if (tid == 0) atomicOr(p.status, kStatusTimeout);
            } else {
                const int hh = tid >> 4, d0 = (tid & 15) * 4;  // 8 heads x 16 threads x 4 values
                if (hh < p.gqa) {
                    const float * slots = reinterpret_cast<const float *>(smem_gen + n_stages * R::kStageBytes);
                    float         M = -INFINITY, L = 0.0f, acc[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int r = 0; r < parts; ++r) {  // in list order, the running maximum raised part by part
                        const float * src = slots + (r * kMaxGqa + hh) * kPartialStride;
                        const float   mc  = src[0];
                        if (mc == -INFINITY) continue;
                        const float Mn = fmaxf(M, mc), fo = exp2f(M - Mn), fw = exp2f(mc - Mn);
                        M = Mn;
                        L = L * fo + src[1] * fw;
#pragma unroll
                        for (int d = 0; d < 4; ++d) acc[d] = acc[d] * fo + src[2 + d0 + d] * fw;
                    }
                    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
                    *reinterpret_cast<float4 *>(p.dst + ((size_t) w.stream * p.n_heads + (size_t) w.kvh * p.gqa + hh) * kHeadDim + d0) =
                        make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
                }
            }
        }
    }
    const int n_cut = ok && !(kClusterMode && p.cluster > 0) ? *reinterpret_cast<volatile int *>(&n_pending) : 0;  // written before the barrier that ends a merge
    if (n_cut > 0) {
        // Second pass without a second launch: every run that holds a part of a pair takes a ticket after publishing
        // its partials; the one that draws the last ticket folds them all and resets the counter.  The tickets of a
        // run's (at most two) cut pairs are taken together at its end, so a run that crosses from one pair into the
        // next pays the round trips to L2 once.  One release fence by one thread: the barrier that ends every merge
        // orders all threads' partial stores before it, and the fence is cumulative, so a ticket is taken only once
        // they are visible device-wide.  The tickets themselves are relaxed (both in flight together); the thread that
        // drew a last ticket fences once more (acquire), and the barrier below carries that order to the threads that
        // read the other CTAs' partials from L2.  Acquire-release fences, not the sequentially consistent
        // __threadfence(): nothing here needs a total order over fences, and the weaker one returns sooner.
        if (tid == 0) {
            fence_acq_rel_gpu();
            int * c0 = p.counters + pending[0][0] * p.n_kv_heads + pending[0][1];
            int * c1 = p.counters + pending[n_cut - 1][0] * p.n_kv_heads + pending[n_cut - 1][1];
            const int t0 = atomicAdd(c0, 1);
            const int t1 = n_cut > 1 ? atomicAdd(c1, 1) : -1;
            int flags = 0;
            if (t0 == pending[0][3] - pending[0][2]) { *c0 = 0; flags |= 1; }
            if (n_cut > 1 && t1 == pending[1][3] - pending[1][2]) { *c1 = 0; flags |= 2; }
            if (flags != 0) fence_acq_rel_gpu();
            fold_flag = flags;
        }
        named_bar_sync(1, kConsumerWarps * 32);
        const int flags = *reinterpret_cast<volatile int *>(&fold_flag);
        if (flags != 0) {
            const int hh = tid >> 4, d0 = (tid & 15) * 4;  // 8 heads x 16 threads x 4 values
            constexpr int kFoldWidth = Q8 ? 4 : 8;  // the q8_0 form has no registers to spare for eight
            if (hh < p.gqa) {
                // a CTA that drew the last ticket of both its cut pairs folds them side by side: the loads of both are
                // in flight together, instead of one fold waiting for its round trips to L2 after the other
                if (flags == 3) fold_pairs<2, kFoldWidth / 2>(p, pending, 0, hh, d0);
                else            fold_pairs<1, kFoldWidth>(p, pending, flags == 2 ? 1 : 0, hh, d0);
            }
        }
    }
    if (tid == 0) DECODE_TRACE(5);
}

}  // namespace

namespace vox {

// Grid size and shortest run of a decode launch.
//   - the grid is one wave: at most `wave` CTAs per SM (all that fit by default), every CTA a copy
//     pipeline that streams an equal share of the launch's tiles, so that the time of a launch does not
//     depend on how the rows are spread over the streams;
//   - a CTA pays a fixed cost at the end of each pair's part of its run (warp merge, partial write, ticket),
//     so a run holds at least 4 tiles (256 rows; measured on one stream: 8.0 -> 6.7 us per layer at 1024
//     rows with 4 x 256 instead of 2 x 512 rows per CTA, while 128 rows per CTA cost more than they save),
//     and at least 1/16 of the longest pair the bound allows, which keeps the partials the folding CTA reads
//     per pair at 17 or fewer;
//   - a launch with fewer tiles than that gets fewer CTAs.
// The cut itself happens on the device from the lengths of the moment; kv_bound only sizes the grid.
void decode_plan(const vox_engine * e, bool q8, int n_streams, int n_kv_heads, int kv_bound, int * grid, int * run_min) {
    const long long tiles_bound = std::max(1, (std::max(kv_bound, 1) + kKvTile - 1) / kKvTile);
    const long long pairs       = std::max(1LL, (long long) n_streams * n_kv_heads);
    const int       fit         = q8 ? Ring<true>::kCtasPerSm : Ring<false>::kCtasPerSm;
    int             wave        = fit;
    int             sms         = kDecodeMaxSms;
    if (e != nullptr) {
        const int tuned = e->decode_wave[q8 ? 1 : 0];
        if (tuned > 0) wave = std::min(tuned, fit);
        sms = std::min(sms, e->sm_count);
    }
    const long long rmin = std::max(4LL, (tiles_bound + 15) / 16);
    const long long want = (pairs * tiles_bound + rmin - 1) / rmin;
    *run_min = (int) rmin;
    *grid    = (int) std::max(1LL, std::min<long long>(want, (long long) sms * wave));
}

// Two partial slots per CTA of the largest grid either cache type would get (the caller of the size query
// does not say which type, nor which device: the bound assumes kDecodeMaxSms SMs, and launches never use more).
size_t decode_workspace_bytes(int n_streams, int n_heads, int n_kv_heads, int kv_bound) {
    if (n_streams <= 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return 0;
    int g_f16, g_q8, rmin;
    decode_plan(nullptr, false, n_streams, n_kv_heads, kv_bound, &g_f16, &rmin);
    decode_plan(nullptr, true, n_streams, n_kv_heads, kv_bound, &g_q8, &rmin);
    return (size_t) 2 * std::max(g_f16, g_q8) * (n_heads / n_kv_heads) * kPartialStride * sizeof(float);
}

// K/V described by tensor maps (f16: a cache layer, or caller tensors) or, for q8_0, by the start of the layer's tiles
// and the strides of a pair and a stream (a cache layer, or tiles built in the workspace); q/dst/lengths by pointers.
// `counters`: one zeroed int per (stream, kv head) of the launch, owned by whoever owns the K/V (a cache layer, or the
// engine).
int launch_decode(vox_engine * e, bool q8, const CUtensorMap & map_k, const CUtensorMap & map_v, const uint8_t * q8_tiles,
                  size_t q8_nb_head, size_t q8_nb_stream, int layer, int max_len, int n_streams, int n_heads, int n_kv_heads,
                  const int32_t * kv_len, int kv_len_const, int kv_bound, const float * q, size_t q_nb_head,
                  size_t q_nb_stream, float * dst, float scale, void * workspace, size_t workspace_bytes, int * counters,
                  cudaStream_t stream, const vox_kv_cache * append_to, const float * k_new, const float * v_new,
                  size_t new_nb_head, size_t new_nb_stream, bool early, const float * rope_table, const int32_t * order,
                  const vox_tensor * mask) {
    const uint32_t bit = q8 ? (1u << 9) : (1u << 8);
    if (!(e->attr_mask & bit)) {
        if (q8) VOX_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Ring<true>::kSmemBytes));
        else    VOX_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Ring<false>::kSmemBytes));
        e->attr_mask |= bit;
    }
    VOX_REQUIRE(n_streams > 0 && n_kv_heads > 0 && n_heads > 0 && n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= kMaxGqa,
                VOX_ATTN_INVALID_ARGUMENT, "decode: bad stream or head counts (%d streams, %d / %d heads)", n_streams, n_heads, n_kv_heads);
    VOX_REQUIRE((long long) n_streams * n_kv_heads * ((std::max(max_len, 1) + kKvTile - 1) / kKvTile) < (1LL << 30), VOX_ATTN_UNSUPPORTED,
                "decode: more than 2^30 tiles in one launch");
    VOX_REQUIRE(counters != nullptr, VOX_ATTN_INVALID_ARGUMENT, "decode: no ticket counters");
    DecodeParams p;
    p.q = reinterpret_cast<const uint8_t *>(q);
    p.q_nb_head = q_nb_head; p.q_nb_stream = q_nb_stream;
    p.kv_len = kv_len; p.kv_len_const = kv_len_const;
    p.dst = dst; p.n_streams = n_streams; p.n_kv_heads = n_kv_heads; p.n_heads = n_heads; p.gqa = n_heads / n_kv_heads;
    p.layer = layer; p.max_len = max_len;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = e->status_dev;
    p.counters = counters;
    p.early = early ? 1 : 0;
    {
        const int depth = q8 ? Ring<true>::kStages : Ring<false>::kStages;
        const int tuned = e->decode_early_tiles;
        // Two tiles: enough to start on as soon as Q is here.  A full ring from every CTA of the next launch is a burst
        // of bulk copies in which the last CTAs of this launch fold their partials, several times slower than in quiet
        // (measured, 32 streams x 2048 / 4096 rows: 11.6 / 16.7 us per launch with a full ring, 11.2 / 16.2 us with two
        // tiles, no difference on launches of 128 streams and more).
        p.early_tiles   = tuned >= 0 ? std::min(tuned, depth) : 2;
    }
    p.rope  = reinterpret_cast<const float2 *>(rope_table);
    p.order = order;
    p.q8_tiles = q8_tiles; p.q8_nb_head = q8_nb_head; p.q8_nb_stream = q8_nb_stream;
    VOX_REQUIRE(!q8 || q8_tiles != nullptr, VOX_ATTN_INVALID_ARGUMENT, "decode: no q8_0 tiles");
    p.k_new = p.v_new = nullptr;
    p.new_nb_head = p.new_nb_stream = 0;
    p.k_rows = p.v_rows = p.k_scales = p.v_scales = nullptr;
    p.nb_pos = p.nb_head = p.nb_stream = p.sb_pos = p.sb_head = p.sb_stream = 0;
    if (append_to != nullptr) {
        const vox_kv_cache * c = append_to;
        p.k_new = reinterpret_cast<const uint8_t *>(k_new);
        p.v_new = reinterpret_cast<const uint8_t *>(v_new);
        p.new_nb_head = new_nb_head; p.new_nb_stream = new_nb_stream;
        p.k_rows = c->k_data + (size_t) layer * c->nb_layer;
        p.v_rows = c->v_data + (size_t) layer * c->nb_layer;
        p.nb_pos = c->nb_pos; p.nb_head = c->nb_head; p.nb_stream = c->nb_stream;
        if (q8) {
            p.k_scales = c->k_scale + (size_t) layer * c->sb_layer;
            p.v_scales = c->v_scale + (size_t) layer * c->sb_layer;
            p.sb_pos = c->sb_pos; p.sb_head = c->sb_head; p.sb_stream = c->sb_stream;
        }
    }
    p.mask = nullptr;
    p.mask_nb_head = p.mask_nb_stream = 0;
    p.mask_ne2 = p.mask_ne3 = 1;
    if (mask != nullptr && mask->data != nullptr) {
        p.mask = static_cast<const uint8_t *>(mask->data);
        p.mask_nb_head = mask->nb[2]; p.mask_nb_stream = mask->nb[3];
        p.mask_ne2 = (int) mask->ne[2]; p.mask_ne3 = (int) mask->ne[3];
    }
    int grid = 1;
    decode_plan(e, q8, n_streams, n_kv_heads, kv_bound, &grid, &p.run_min);
    const size_t need = (size_t) 2 * grid * p.gqa * kPartialStride * sizeof(float);
    VOX_REQUIRE(workspace != nullptr && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 7) == 0,
                VOX_ATTN_WORKSPACE_TOO_SMALL, "decode needs %zu workspace bytes (8-byte aligned), got %zu", need, workspace_bytes);
    p.partial = static_cast<float *>(workspace);
    // Cluster mode for launches of few pairs: with a whole cluster of CTAs per pair inside one wave, the CTAs of a pair
    // exchange their partial results through distributed shared memory and no CTA pays the round trips of partials,
    // tickets and fold through L2.  A stream order is not supported there (the cluster's number is the pair's).
    // Only where a pair gets five CTAs or more: a pair cannot use more CTAs than its cluster has, so with small
    // clusters the long pairs of a ragged launch run far longer than an equal share (64 ragged streams, clusters of
    // three: 17.9 against 16.5 us per launch; 32 ragged streams, clusters of six: 11.4 against 12.7 us).
    const int depth  = q8 ? Ring<true>::kStages : Ring<false>::kStages;
    const int spare  = q8 ? 2 : 1;  // ring stages whose memory holds the partials instead: 18 KB / 16 KB
    const int slots  = std::min(kDecodeMaxSms, e->sm_count) * (q8 ? Ring<true>::kCtasPerSm : Ring<false>::kCtasPerSm);
    const int pairs  = n_streams * n_kv_heads;
    const int c_fit  = (q8 ? 2 * Ring<true>::kStageBytes : Ring<false>::kStageBytes) / (kMaxGqa * kPartialStride * 4);  // slots of partials that fit
    const int tiles_bound = std::max(1, (std::max(kv_bound, 1) + kKvTile - 1) / kKvTile);
    int       cluster = std::min(std::min(8, c_fit), slots / std::max(1, pairs));
    if (q8 || e->decode_cluster == 0 || order != nullptr || cluster < 5 || tiles_bound < 8 || (tiles_bound + cluster - 1) / cluster > kClusterMaxRun) cluster = 0;
    p.cluster  = cluster;
    p.n_stages = cluster > 0 ? depth - spare : depth;
    p.early_tiles = std::min(p.early_tiles, p.n_stages);
    if (cluster > 0) grid = pairs * cluster;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) grid); cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = q8 ? Ring<true>::kSmemBytes : Ring<false>::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (cluster > 0) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = (unsigned) cluster; attr[n_attr].val.clusterDim.y = 1; attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    if (q8) cudaLaunchKernelEx(&cfg, decode_kernel<true>, map_k, map_v, p);
    else    cudaLaunchKernelEx(&cfg, decode_kernel<false>, map_k, map_v, p);
    return check_launch(e, q8 ? "decode_kernel<q8_0>" : "decode_kernel<f16>");
}

// the operator's single-token call on a caller's own f16 tensors (vox_attn_forward): tickets from the engine's counters
int launch_decode_f16(vox_engine * e, const CUtensorMap & map_k, const CUtensorMap & map_v, int n_kv, int n_streams,
                      int n_heads, int n_kv_heads, const float * q, size_t q_nb_head, size_t q_nb_stream, float * dst,
                      float scale, const vox_tensor * mask, void * workspace, size_t workspace_bytes, cudaStream_t stream) {
    return launch_decode(e, false, map_k, map_v, nullptr, 0, 0, 0, n_kv, n_streams, n_heads, n_kv_heads, nullptr, n_kv, n_kv, q,
                         q_nb_head, q_nb_stream, dst, scale, workspace, workspace_bytes, e->counters_dev, stream, nullptr, nullptr,
                         nullptr, 0, 0, false, nullptr, nullptr, mask);
}

// ---- single-token calls over q8_0 K/V in ggml's block layout (the operator called on a caller's own quantised
// cache, third_party/ggml/src/ggml-common.h:221-224): the blocks are taken apart into the layout the q8_0 decode
// kernel reads (tiles of 64 rows: bytes and scales of K and V in one span, as the cache object keeps them), in the
// workspace, and that kernel runs on them.
// Nothing is re-quantised: the result is what the cache object gives for the same blocks.

struct RepackParams {
    const uint8_t * src[2];
    size_t          nb1[2], nb2[2], nb3[2];
    uint8_t *       tiles;  // [B][HK][n_pad / 64] tiles of kQ8TileBytes
    int             n_kv, n_pad, n_kvh, n_batch;
};
__global__ void __launch_bounds__(256) q8_0_blocks_to_tiles_kernel(const RepackParams p) {
    const long long n_blocks = 2LL * p.n_pad * p.n_kvh * p.n_batch;
    const bool      is_v     = blockIdx.y != 0;
    const uint8_t * src      = is_v ? p.src[1] : p.src[0];
    const size_t    nb1 = is_v ? p.nb1[1] : p.nb1[0], nb2 = is_v ? p.nb2[1] : p.nb2[0], nb3 = is_v ? p.nb3[1] : p.nb3[0];
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks; i += (long long) gridDim.x * blockDim.x) {
        const int       blk = (int) (i & 1);
        const long long row = i >> 1;
        const int       pos = (int) (row % p.n_pad);
        const long long pair = row / p.n_pad;  // (batch, kv head) flattened, kv head fastest
        const int       kvh = (int) (pair % p.n_kvh);
        const int       b   = (int) (pair / p.n_kvh);
        uint32_t        q[8] = {0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u};
        uint16_t        d    = 0;  // rows past n_kv (up to the next multiple of the tile) have a zero scale
        if (pos < p.n_kv) {
            const uint16_t * s = reinterpret_cast<const uint16_t *>(src + (size_t) pos * nb1 + (size_t) kvh * nb2 + (size_t) b * nb3 +
                                                                    (size_t) blk * 34);
            d = s[0];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = ((uint32_t) s[1 + 2 * j] | ((uint32_t) s[2 + 2 * j] << 16)) ^ 0x80808080u;  // q + 128, as the cache holds it
        }
        uint8_t * tile = p.tiles + (size_t) pair * (p.n_pad / kKvTile) * kQ8TileBytes + q8_tile_off(pos);
        uint8_t * bytes = tile + (is_v ? kQ8VBytesOff : 0);
        *reinterpret_cast<uint4 *>(bytes + q8_byte_off(pos, 32 * blk))      = make_uint4(q[0], q[1], q[2], q[3]);
        *reinterpret_cast<uint4 *>(bytes + q8_byte_off(pos, 32 * blk + 16)) = make_uint4(q[4], q[5], q[6], q[7]);
        *reinterpret_cast<uint16_t *>(tile + (is_v ? kQ8VScaleOff : kQ8KScaleOff) + q8_scale_off(pos, blk)) = d;
    }
}

// the mask of a single-token call as the decode kernel reads it: one contiguous f16 row per (head, batch) plane
bool decode_mask_ok(const vox_attn_args * a) {
    const vox_tensor & m = a->mask;
    if (m.data == nullptr) return true;
    return (reinterpret_cast<uintptr_t>(m.data) & 1) == 0 && m.nb[2] % 2 == 0 && m.nb[3] % 2 == 0 && m.ne[2] >= 1 && m.ne[3] >= 1;
}

static size_t q8_tiles_bytes(const vox_attn_args * a, int * n_pad_out) {
    const int n_pad = (int) ((a->k.ne[1] + kKvTile - 1) / kKvTile * kKvTile);
    if (n_pad_out) *n_pad_out = n_pad;
    return (size_t) (n_pad / kKvTile) * a->k.ne[2] * a->k.ne[3] * kQ8TileBytes;  // K and V bytes and scales, tile by tile
}

bool decode_q8_blocks_route_ok(const vox_attn_args * a) {
    const vox_tensor &q = a->q, &k = a->k, &v = a->v;
    if (q.ne[1] != 1 || !decode_mask_ok(a)) return false;
    if (k.type != VOX_TYPE_Q8_0 || v.type != VOX_TYPE_Q8_0) return false;
    if (q.ne[3] * k.ne[2] > kCounterSlots) return false;
    if (k.ne[1] < 1 || k.ne[1] != v.ne[1] || k.ne[2] != v.ne[2] || k.ne[3] != v.ne[3] || q.ne[2] / k.ne[2] > 8) return false;
    for (const vox_tensor * t : {&k, &v})
        if ((reinterpret_cast<uintptr_t>(t->data) & 1) != 0 || t->nb[1] % 2 || t->nb[2] % 2 || t->nb[3] % 2) return false;
    return true;
}

size_t decode_q8_blocks_workspace_bytes(const vox_attn_args * a) {
    if (!decode_q8_blocks_route_ok(a)) return 0;
    const size_t partials = decode_workspace_bytes((int) a->q.ne[3], (int) a->q.ne[2], (int) a->k.ne[2], (int) a->k.ne[1]);
    return ((partials + 255) & ~(size_t) 255) + q8_tiles_bytes(a, nullptr);
}

int launch_decode_q8_blocks(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t st) {
    int          n_pad = 0;
    const size_t tiles_bytes = q8_tiles_bytes(a, &n_pad);
    const int    B = (int) a->q.ne[3], HK = (int) a->k.ne[2], n_kv = (int) a->k.ne[1];
    const size_t partials = (decode_workspace_bytes(B, (int) a->q.ne[2], HK, n_kv) + 255) & ~(size_t) 255;
    VOX_REQUIRE(workspace != nullptr && workspace_bytes >= partials + tiles_bytes && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                VOX_ATTN_WORKSPACE_TOO_SMALL, "q8_0 decode needs %zu workspace bytes, got %zu", partials + tiles_bytes, workspace_bytes);
    uint8_t *    base = static_cast<uint8_t *>(workspace) + partials;
    RepackParams rp;
    const vox_tensor * ts[2] = {&a->k, &a->v};
    for (int i = 0; i < 2; ++i) {
        rp.src[i] = static_cast<const uint8_t *>(ts[i]->data);
        rp.nb1[i] = ts[i]->nb[1]; rp.nb2[i] = ts[i]->nb[2]; rp.nb3[i] = ts[i]->nb[3];
    }
    rp.tiles = base;
    rp.n_kv = n_kv; rp.n_pad = n_pad; rp.n_kvh = HK; rp.n_batch = B;
    const long long n_blocks = 2LL * n_pad * HK * B;
    const unsigned  gx = (unsigned) std::min<long long>((n_blocks + 255) / 256, 8LL * e->sm_count);
    q8_0_blocks_to_tiles_kernel<<<dim3(gx, 2), 256, 0, st>>>(rp);
    int rc = check_launch(e, "q8_0_blocks_to_tiles_kernel");
    if (rc != VOX_ATTN_OK) return rc;
    // the tiles as one cache layer of n_pad rows
    CUtensorMap  none;
    memset(&none, 0, sizeof(none));
    const size_t pair_bytes = (size_t) (n_pad / kKvTile) * kQ8TileBytes;
    return launch_decode(e, true, none, none, base, pair_bytes, pair_bytes * HK, 0, n_pad, B, (int) a->q.ne[2], HK, nullptr, n_kv, n_kv,
                         static_cast<const float *>(a->q.data), a->q.nb[2], a->q.nb[3], static_cast<float *>(a->dst.data), a->scale,
                         workspace, partials, e->counters_dev, st, nullptr, nullptr, nullptr, 0, 0, false, nullptr, nullptr,
                         a->mask.data ? &a->mask : nullptr);
}

}  // namespace vox

namespace {

// argument checks shared by vox_attn_decode and vox_attn_decode_static: everything that does not involve the workspace
int check_decode_args(const vox_engine * e, const vox_decode_args * a, const char * who) {
    VOX_REQUIRE(e && a && a->cache && a->q && a->dst, VOX_ATTN_INVALID_ARGUMENT, "%s: null argument", who);
    const vox_kv_cache * c = a->cache;
    VOX_REQUIRE(c->e == e, VOX_ATTN_INVALID_ARGUMENT, "cache belongs to another engine");
    VOX_REQUIRE(a->layer >= 0 && a->layer < c->cfg.n_layers, VOX_ATTN_INVALID_ARGUMENT, "layer %d out of range", a->layer);
    VOX_REQUIRE(a->n_streams > 0 && a->n_streams <= c->cfg.n_streams, VOX_ATTN_INVALID_ARGUMENT,
                "n_streams %d out of range (cache holds %d)", a->n_streams, c->cfg.n_streams);
    VOX_REQUIRE(a->n_heads > 0 && a->n_heads % c->cfg.n_kv_heads == 0, VOX_ATTN_INVALID_ARGUMENT,
                "n_heads %d is not a multiple of n_kv_heads %d", a->n_heads, c->cfg.n_kv_heads);
    VOX_REQUIRE(a->n_heads / c->cfg.n_kv_heads <= kMaxGqa, VOX_ATTN_UNSUPPORTED, "GQA ratio above 8 is not supported");
    VOX_REQUIRE(a->kv_len != nullptr, VOX_ATTN_INVALID_ARGUMENT, "kv_len is null");
    VOX_REQUIRE(a->kv_bound >= 0 && a->kv_bound <= c->cfg.max_len, VOX_ATTN_INVALID_ARGUMENT,
                "kv_bound %d exceeds the cache capacity %d", a->kv_bound, c->cfg.max_len);
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->q) & 7) == 0 && a->q_nb_head % 8 == 0 && a->q_nb_stream % 8 == 0,
                VOX_ATTN_INVALID_ARGUMENT, "q rows must be 8-byte aligned");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->dst) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT, "dst must be 16-byte aligned");
    if (a->k_new != nullptr || a->v_new != nullptr) {
        VOX_REQUIRE(a->k_new && a->v_new, VOX_ATTN_INVALID_ARGUMENT, "k_new and v_new must be given together");
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->k_new) & 7) == 0 && (reinterpret_cast<uintptr_t>(a->v_new) & 7) == 0 &&
                        a->new_nb_head % 8 == 0 && a->new_nb_stream % 8 == 0,
                    VOX_ATTN_INVALID_ARGUMENT, "k_new / v_new rows must be 8-byte aligned");
        VOX_REQUIRE(a->kv_bound >= 1, VOX_ATTN_INVALID_ARGUMENT, "kv_bound counts the arriving row: it cannot be 0 with k_new");
    }
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->rope_table) & 7) == 0, VOX_ATTN_INVALID_ARGUMENT, "rope_table must be 8-byte aligned");
    return VOX_ATTN_OK;
}

int decode_checked(vox_engine * e, const vox_decode_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    const vox_kv_cache * c       = a->cache;
    const bool           appends = a->k_new != nullptr;
    int * counters = c->counters + (size_t) a->layer * c->cfg.n_streams * c->cfg.n_kv_heads;
    const bool q8 = c->cfg.type == VOX_TYPE_Q8_0;
    return launch_decode(e, q8, c->map_k, c->map_v, q8 ? c->k_data + (size_t) a->layer * c->nb_layer : nullptr, c->nb_head, c->nb_stream,
                         a->layer, c->cfg.max_len,
                         a->n_streams, a->n_heads, c->cfg.n_kv_heads, a->kv_len, 0, a->kv_bound, a->q, a->q_nb_head, a->q_nb_stream,
                         a->dst, a->scale, workspace, workspace_bytes, counters, static_cast<cudaStream_t>(stream),
                         appends ? c : nullptr, a->k_new, a->v_new, a->new_nb_head, a->new_nb_stream,
                         (a->flags & VOX_DECODE_CACHE_STABLE) != 0, a->rope_table, a->stream_order, nullptr);
}

}  // namespace

#ifdef VOX_ATTN_DEVELOPER
// out: kTraceCtas x kTracePoints times in ns (0 entry, 1 work list cut, 2 consumers past the dependency wait, 3 first tile
// in shared memory, 4 last tile consumed, 5 consumers done, 6 first copy issued, 7 producer done)
extern "C" int vox_debug_decode_trace(unsigned long long * out) {
    return cudaMemcpyFromSymbol(out, g_decode_trace, sizeof(unsigned long long) * 2 * kTraceCtas * kTracePoints) == cudaSuccess ? 0 : 4;
}
#endif

extern "C" {

size_t vox_attn_decode_workspace_bytes(int n_streams, int n_heads, int n_kv_heads, int kv_bound) {
    return decode_workspace_bytes(n_streams, n_heads, n_kv_heads, kv_bound);
}

int vox_attn_decode(vox_engine * e, const vox_decode_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    const int rc = check_decode_args(e, a, "vox_attn_decode");
    if (rc != VOX_ATTN_OK) return rc;
    return decode_checked(e, a, workspace, workspace_bytes, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Decode without any allocation: split-KV partials in a built-in device array
// ---------------------------------------------------------------------------------------------
//
// Some hosts of this library may not allocate device memory at the point where they call
// attention: a real-time audio thread that must not enter the allocator, a host that has handed
// all device memory to its own arena up front, or a plugin that is only given input and output
// buffers by its framework.  For them the partial results of the split-KV pass live in the array
// below, which is part of the library image: every GPU that loads the library carries these
// bytes until the process exits, whether or not the entry point is ever called.
//
// In host code `g_decode_scratch` is only a handle for the runtime, not a device address, so the
// address is looked up with cudaGetSymbolAddress (once per device, with that device current) and
// that pointer is what the kernels receive.
//
// A decode launch writes two partial slots per CTA and its grid never exceeds one wave, so the need
// is bounded by the device: 2 x 4 CTAs x 148 SMs x 8 query heads per kv head x 264 bytes = 2.4 MiB.
constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

namespace {
constexpr int  kMaxDevices = 64;
unsigned char * g_scratch_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int vox_attn_decode_static(vox_engine * e, const vox_decode_args * a, void * stream) {
    // the same checks as vox_attn_decode, before anything is derived from the arguments
    const int rc = check_decode_args(e, a, "vox_attn_decode_static");
    if (rc != VOX_ATTN_OK) return rc;
    int current = -1;
    VOX_CUDA_TRY(cudaGetDevice(&current));
    VOX_REQUIRE(current == e->device && current >= 0 && current < kMaxDevices, VOX_ATTN_INVALID_ARGUMENT,
                "the engine's device %d must be the current device (current is %d)", e->device, current);
    const size_t need = decode_workspace_bytes(a->n_streams, a->n_heads, a->cache->cfg.n_kv_heads, a->kv_bound);
    VOX_REQUIRE(need <= kStaticScratchBytes, VOX_ATTN_WORKSPACE_TOO_SMALL,
                "this call needs %zu bytes of split-KV scratch but the built-in array holds %zu; "
                "use vox_attn_decode with a caller-provided workspace for this size",
                need, kStaticScratchBytes);
    if (g_scratch_ptr[current] == nullptr) {  // first call on this device: resolve the array's device address
        void * ptr = nullptr;
        VOX_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_decode_scratch));
        VOX_REQUIRE(ptr != nullptr, VOX_ATTN_CUDA_ERROR, "cudaGetSymbolAddress returned a null address");
        g_scratch_ptr[current] = static_cast<unsigned char *>(ptr);
    }
    // Nothing in the array has to start at zero: every partial a fold reads was written by a CTA
    // of the same call.  What the previous call left behind is simply overwritten.
    return decode_checked(e, a, g_scratch_ptr[current], kStaticScratchBytes, stream);
}
