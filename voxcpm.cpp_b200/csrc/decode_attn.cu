// Split-KV decode attention (one query token per stream) for sm_100a.
//
// Replaces, for the n_q == 1 call of MiniCPMModel::forward_step (src/minicpm.cpp:813-846 ->
// :708-710), what ggml's CPU backend does in ggml_compute_forward_flash_attn_ext_f16_one_chunk
// plus ggml_flash_attn_ext_reduce_partials (third_party/ggml/src/ggml-cpu/ops.cpp:8109-8345,
// 8637-8705) and what ggml-cuda does in flash_attn_ext_vec + flash_attn_combine_results
// (third_party/ggml/src/ggml-cuda/fattn-vec.cuh:19-507, fattn-common.cuh:728-779).
//
// Design (HBM-bound kernel; the cache is read exactly once):
//   grid  = (kv chunks, kv heads, streams); one CTA owns `chunk` consecutive cache rows of one
//           kv head of one stream and serves all GQA query heads that share it, so each K/V
//           byte is fetched once for the whole group;
//   copy  = a producer warp streams 64-row K and V tiles into a shared-memory ring (4 stages for f16, 6 for q8_0) with
//           bulk-tensor copies (cp.async.bulk.tensor, 128-byte swizzle) signalled on mbarriers;
//   math  = four consumer warps, 16 rows each.  Q (pre-scaled by scale*log2 e) is split as
//           hi + lo in f16 and the two parts occupy rows 0-7 and 8-15 of the m16n8k16 A operand,
//           so one MMA yields the hi and lo products and their sum carries ~22 bits of Q.  The
//           same trick carries the softmax weights P through the P.V MMA.  Accumulation is f32;
//   merge = warps are merged through shared memory; when the KV range was split across CTAs the
//           (max, sum, acc[64]) partials go to the workspace and the last CTA of the (stream, kv head)
//           to finish folds them (a ticket counter decides who is last).
// q8_0 K/V (int8 plane + scale plane) is dequantised in registers: int8 -> f16 is exact, the
// per-block scales are applied in f32 to the per-block score accumulators (K) and folded into
// the softmax weights (V), so Q is never quantised.
#include "kv_cache.cuh"

#include <algorithm>
#include <cstdlib>

using namespace vox;

namespace {

constexpr int kConsumerWarps = 4;
constexpr int kThreads       = (kConsumerWarps + 1) * 32;
constexpr int kPartialStride = 66;  // max, sum, acc[64]

struct DecodeParams {
    const uint8_t * q;
    size_t          q_nb_head, q_nb_stream;
    const int32_t * kv_len;
    int             kv_len_const;
    float *         partial;
    float *         dst;
    int             n_heads, gqa, chunk, n_chunks, layer, max_len;
    float           scale_log2;
    int *           status;
    int *           counters;  // non-null: the last CTA of a (stream, kv head) to finish folds the partials itself
    // Fused append (k_new non-null): kv_len[stream] counts the row that arrives with this call; the CTA
    // whose chunk holds position kv_len-1 converts it, stores it into the cache and uses it.
    const uint8_t * k_new;
    const uint8_t * v_new;
    size_t          new_nb_head, new_nb_stream;
    uint8_t *       k_rows;    // data planes of this layer
    uint8_t *       v_rows;
    uint8_t *       k_scales;  // scale planes of this layer (q8_0)
    uint8_t *       v_scales;
    size_t          nb_pos, nb_head, nb_stream, sb_pos, sb_head, sb_stream;
    // Non-zero: the lengths and the cache rows this launch reads were not written by the kernel just before
    // it on the stream (only Q and the arriving row were), so the first tiles are requested before the
    // programmatic-dependency wait, while that kernel is still draining.
    int             early;
    // Non-null: [stream][32] (cos, sin) pairs; Q and the arriving K row are rotated as they are read
    // (element i with element i + 32: the reference's ggml_rope_ext, GGML_ROPE_TYPE_NEOX).
    const float2 *  rope;
    // Non-null: a permutation of the streams; CTA z works on stream order[z] (longest first shortens a launch's tail)
    const int32_t * order;
};

__device__ __forceinline__ int stream_len(const DecodeParams & p, int stream) {
    int len = p.kv_len ? p.kv_len[stream] : p.kv_len_const;
    return max(0, min(len, p.max_len));
}

// Shared-memory ring: per stage one 64-row K tile and one 64-row V tile.
//   f16 : 2 x 8 KB (128-byte rows, 128-byte swizzle)                       -> 16 KB, 4 stages
//   q8_0: 2 x 4 KB int8 (64-byte rows, 64-byte swizzle) + 2 x 256 B scales -> 9 KB (1 KB aligned), 6 stages
template <bool Q8> struct Ring {
    static constexpr int kStages     = Q8 ? 6 : 4;
    // q8_0 tiles are half the bytes and its arithmetic chain is longer: one more CTA hides it.  Measured per 256-stream
    // launch (one tile per pass): 4 CTAs x 96 registers x 5 stages 45.6 us; 5 x 72 x 4: 48.1 us; 3 x 105 x 6: 48.2 us.
    // Stages are held while their tile is worked on, so depth pays: 4 CTAs x 6 stages (the most that fits) 43.8 -> 42.5 us.
    static constexpr int kCtasPerSm  = Q8 ? 4 : 3;
    static constexpr int kDataBytes  = Q8 ? kKvTile * 64 : kKvTile * 128;
    static constexpr int kStageBytes = Q8 ? 9 * 1024 : 2 * kDataBytes;
    static constexpr int kTxBytes    = Q8 ? 2 * kDataBytes + 2 * kKvTile * 4 : 2 * kDataBytes;
    static constexpr int kSmemBytes  = kStages * kStageBytes + 1024;
};

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float half_lo(uint32_t x) { return __half2float(__ushort_as_half((unsigned short) (x & 0xffffu))); }
__device__ __forceinline__ float half_hi(uint32_t x) { return __half2float(__ushort_as_half((unsigned short) (x >> 16))); }

// four signed bytes -> two half2 registers holding the exact values.  A byte b is biased to b+128,
// placed in the mantissa of 1024.0h (0x6400 | b+128 == 1024 + b + 128) and 1152 is subtracted.
// `sel_a` / `sel_b` pick which two bytes go to each register (PRMT selectors, 4 = the 0x64 byte).
__device__ __forceinline__ uint32_t s8_pair_to_half2(uint32_t biased, uint32_t selector) {
    const uint32_t h  = __byte_perm(biased, 0x64646464u, selector);
    const __half2  r  = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half((unsigned short) 0x6480)));
    return *reinterpret_cast<const uint32_t *>(&r);
}

// The row that arrives with this call, stored by the producer warp (lane l holds elements 2l, 2l+1 of K
// and of V; converted exactly as kv_append_kernel converts them) before it requests the tile that
// contains the row: the bulk copy then delivers the new row like any other.  The proxy fence orders
// these generic-proxy stores before the async-proxy read of the copy issued after the warp barrier.
template <bool Q8>
__device__ __forceinline__ void store_arriving_row(float2 kk, float2 vv, uint8_t * k_dst, uint8_t * v_dst, uint8_t * ks_dst,
                                                   uint8_t * vs_dst, int lane) {
    if constexpr (!Q8) {
        *reinterpret_cast<uint32_t *>(k_dst + lane * 4) = pack_half2(kk.x, kk.y);
        *reinterpret_cast<uint32_t *>(v_dst + lane * 4) = pack_half2(vv.x, vv.y);
    } else {
        char2 qk, qv;
        float dk, dv;
        q8_0_quantize_pair(kk.x, kk.y, qk, dk);
        q8_0_quantize_pair(vv.x, vv.y, qv, dv);
        *reinterpret_cast<char2 *>(k_dst + lane * 2) = qk;
        *reinterpret_cast<char2 *>(v_dst + lane * 2) = qv;
        if ((lane & 15) == 0) {
            *reinterpret_cast<__half *>(ks_dst + (lane >> 4) * 2) = __float2half_rn(dk);
            *reinterpret_cast<__half *>(vs_dst + (lane >> 4) * 2) = __float2half_rn(dv);
        }
    }
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncwarp();
}

template <bool Q8>
__global__ void __launch_bounds__(kThreads, Ring<Q8>::kCtasPerSm)
decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const __grid_constant__ CUtensorMap map_ks, const __grid_constant__ CUtensorMap map_vs, const DecodeParams p) {
    using R = Ring<Q8>;
    constexpr int kStages = R::kStages;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * kStages];
    __shared__ int      abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *      smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));

    // CTAs are handed out x first, z last, so the chunks of one (stream, kv head) start together and read neighbouring
    // memory (handing out all first chunks, then all second chunks, ... measured 9 % slower for f16: 54.1 against 49.7 us).
    // With `order` the streams are taken longest first, so that the last CTAs to start are short ones.
    const int chunk_id = blockIdx.x, kvh = blockIdx.y, stream = p.order ? p.order[blockIdx.z] : blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // set-up that reads nothing the previous kernel of the stream wrote: done while that kernel drains
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kStages]);
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumerWarps);
        }
        fence_mbar_init();
    }
    if (tid == kConsumerWarps * 32) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
        if constexpr (Q8) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_ks)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_vs)) : "memory");
        }
    }
    __syncthreads();
    // Dependency wait.  Every thread passes it before it triggers the launch of the next kernel, and the
    // CTAs of chunk 0 always pass it, so a kernel that starts early can rely on everything before its
    // predecessor being complete.
    if (!p.early) {
        pdl_wait();
        pdl_launch_dependents();
    }
    const int len = stream_len(p, stream);
    const int c0  = chunk_id * p.chunk;
    if (c0 >= len) {
        if (chunk_id == 0) {
            if (p.early) {
                pdl_wait();
                pdl_launch_dependents();
            }
            // a stream with no visible rows at all yields zeros
            if (warp < kConsumerWarps) {
                for (int i = tid; i < p.gqa * kHeadDim; i += kConsumerWarps * 32)
                    p.dst[((size_t) stream * p.n_heads + (size_t) kvh * p.gqa) * kHeadDim + i] = 0.0f;
            }
        }
        return;  // nothing visible in this chunk
    }
    const int c1      = min(c0 + p.chunk, len);
    const int n_tiles = (c1 - c0 + kKvTile - 1) / kKvTile;
    // fused append: this CTA holds the arriving row iff its chunk ends at the stream's length
    bool appends = false;
    if (p.k_new != nullptr && c1 == len) {
        appends = p.kv_len[stream] <= p.max_len;
        if (!appends && tid == 0) atomicOr(p.status, kStatusBadState);  // the stream has outgrown its rows: nothing is written
    }

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer
        int  issued  = 0;
        auto request = [&](int i) {  // lane 0: the copies of tile i; false when the CTA is giving up
            const int s = i % kStages;
            if (i >= kStages && !mbar_wait_bounded(empty0 + 8 * s, ((i / kStages) - 1) & 1)) {
                atomicOr(p.status, kStatusTimeout);
                atomicExch(&abort_flag, 1);
                return false;
            }
            if (*reinterpret_cast<volatile int *>(&abort_flag)) return false;
            const uint32_t sb  = smem_base + s * R::kStageBytes;
            const uint32_t bar = full0 + 8 * s;
            const int      pos = c0 + i * kKvTile;
            mbar_expect_tx(bar, R::kTxBytes);
            tma_load_5d(sb, &map_k, bar, 0, pos, kvh, stream, p.layer);
            tma_load_5d(sb + R::kDataBytes, &map_v, bar, 0, pos, kvh, stream, p.layer);
            if constexpr (Q8) {
                tma_load_5d(sb + 2 * R::kDataBytes, &map_ks, bar, 2 * pos, 0, kvh, stream, p.layer);
                tma_load_5d(sb + 2 * R::kDataBytes + kKvTile * 4, &map_vs, bar, 2 * pos, 0, kvh, stream, p.layer);
            }
            issued = i + 1;
            return true;
        };
        const int n_before = appends ? n_tiles - 1 : n_tiles;  // the arriving row lies in the last tile
        int       next     = 0;
        if (p.early) {  // fill the ring while the previous kernel drains
            if (lane == 0) {
                for (; next < min(n_before, kStages); ++next)
                    if (!request(next)) break;
            }
            pdl_wait();
            pdl_launch_dependents();
        }
        float2 kk = make_float2(0.f, 0.f), vv = kk;
        if (appends) {  // fetched now, stored just before the tile that holds the row is requested
            const size_t src = (size_t) stream * p.new_nb_stream + (size_t) kvh * p.new_nb_head + lane * 8;
            kk = *reinterpret_cast<const float2 *>(p.k_new + src);
            vv = *reinterpret_cast<const float2 *>(p.v_new + src);
            if (p.rope != nullptr) {
                // lane l holds elements 2l, 2l+1; their partners (32 further, or 32 back) sit in lane l ^ 16.
                // Separate multiplies and adds, in the operand order of the reference's rotate_pairs.
                const float2 * tb = p.rope + (size_t) stream * (kHeadDim / 2) + 2 * (lane & 15);
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
        }
        if (lane == 0) {
            for (int i = next; i < n_before; ++i)
                if (!request(i)) break;
        }
        if (appends) {
            __syncwarp();
            const size_t off  = (size_t) stream * p.nb_stream + (size_t) kvh * p.nb_head + (size_t) (len - 1) * p.nb_pos;
            const size_t soff = (size_t) stream * p.sb_stream + (size_t) kvh * p.sb_head + (size_t) (len - 1) * p.sb_pos;
            store_arriving_row<Q8>(kk, vv, p.k_rows + off, p.v_rows + off, p.k_scales + soff, p.v_scales + soff, lane);
            if (lane == 0 && issued == n_before) request(n_tiles - 1);
        }
        if (lane == 0 && *reinterpret_cast<volatile int *>(&abort_flag)) {
            // consumers gave up: let the copies already issued land before the CTA retires
            for (int i = max(0, issued - kStages); i < issued; ++i)
                mbar_wait_bounded(full0 + 8 * (i % kStages), (i / kStages) & 1);
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    if (p.early) {  // Q is written by the kernel before this one
        pdl_wait();
        pdl_launch_dependents();
    }

    // Q fragments of the four k-steps: rows 0-7 = hi part of the group's heads, rows 8-15 = lo part.
    // The 64 head dimensions may be fed to the MMAs in any order as long as K uses the same one:
    //   f16 : k-step c covers d = 16c .. 16c+15 in natural order (K fragments come from ldmatrix);
    //   q8_0: k-step s covers the 8 bytes per lane that one 64-bit shared load returns,
    //         d = 32*(s/2) + 8t + 4*(s%2) + {0,1,2,3}, so that k-steps 0,1 / 2,3 stay inside one
    //         32-value quantisation block and the block scale can be applied to their accumulator.
    uint32_t qa[4][4];
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
        }
    }

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    bool  ok = true;

    // per-lane ldmatrix row/chunk selectors (see the fragment layouts of mma.m16n8k16)
    const int k_row = 16 * warp + ((lane >> 4) << 3) + (lane & 7), k_chk = (lane >> 3) & 1;
    const int v_row = 16 * warp + (((lane >> 3) & 1) << 3) + (lane & 7), v_chk = lane >> 4;

    // Tiles per pass of a consumer warp.  q8_0 takes two (its 16 rows of each): the byte unpacking and the per-block
    // scales make its dependency chains long, and two independent tiles in one pass give the scheduler something to
    // overlap them with; max, rescale decision and row sum are then taken once per 32 rows.  Measured per 256-stream
    // launch: at 3 CTAs per SM (115 registers) 48.2 -> 45.4 us; at 4 CTAs per SM (96 registers, the configuration
    // used) 43.9 -> 43.8 us: with that register budget the compiler cannot keep both chains in flight.
    constexpr int U = Q8 ? 2 : 1;  // f16 with two tiles per pass measured 50.6 against 49.9 us: it holds two stages at a time
    for (int i = 0; i < n_tiles && ok; i += U) {
        int  st[U], p0[U];
        bool have[U], act[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            have[u] = i + u < n_tiles;
            st[u]   = (i + u) % kStages;
            p0[u]   = c0 + (i + u) * kKvTile + 16 * warp;
            act[u]  = have[u] && p0[u] < c1;
            if (have[u] && !mbar_wait_bounded(full0 + 8 * st[u], ((i + u) / kStages) & 1)) {
                atomicOr(p.status, kStatusTimeout);
                atomicExch(&abort_flag, 1);
                ok = false;
            }
        }
        if (!ok) break;
#ifdef VOX_DECODE_NOMATH  // experiment: the copy structure alone
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
                        const int row = 16 * warp + 8 * j + g;
                        float     sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};  // one accumulator per 32-value block
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            const uint2 raw = lds64(kb + row * 64 + (((2 * b + (t >> 1)) ^ ((row >> 1) & 3)) << 4) + ((t & 1) << 3));
                            const uint32_t x0 = raw.x ^ 0x80808080u, x1 = raw.y ^ 0x80808080u;
                            mma_16816(sc[b], qa[2 * b], s8_pair_to_half2(x0, 0x4140), s8_pair_to_half2(x0, 0x4342));
                            mma_16816(sc[b], qa[2 * b + 1], s8_pair_to_half2(x1, 0x4140), s8_pair_to_half2(x1, 0x4342));
                        }
                        // scales of positions 8j+2t and 8j+2t+1, both blocks: four consecutive halves
                        const uint2 ds = lds64(ksc + (16 * warp + 8 * j + 2 * t) * 4);
                        sv[u][j][0] = (sc[0][0] + sc[0][2]) * half_lo(ds.x) + (sc[1][0] + sc[1][2]) * half_hi(ds.x);
                        sv[u][j][1] = (sc[0][1] + sc[0][3]) * half_lo(ds.y) + (sc[1][1] + sc[1][3]) * half_hi(ds.y);
                    }
                }
            }
            float tmax = -INFINITY;
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int pos = p0[u] + 8 * j + 2 * t + e;
                        sv[u][j][e]   = pos < c1 ? sv[u][j][e] : -INFINITY;
                        tmax          = fmaxf(tmax, sv[u][j][e]);
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
                    // V scales are folded into the weights: one A operand per 32-wide block of output columns
                    const uint32_t vsc = kb + 2 * R::kDataBytes + kKvTile * 4;
                    uint32_t       pa[2][4];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint2 ds = lds64(vsc + (16 * warp + 8 * j + 2 * t) * 4);
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            // weights times V scale rounded to f16 once (2^-12 relative, far inside the q8_0
                            // tolerance): the lo rows of the A operand stay zero
                            pa[b][2 * j]     = pack_half2(pr[u][j][0] * (b ? half_hi(ds.x) : half_lo(ds.x)),
                                                          pr[u][j][1] * (b ? half_hi(ds.y) : half_lo(ds.y)));
                            pa[b][2 * j + 1] = 0u;
                        }
                    }
                    // ldmatrix.trans on 16-bit units keeps byte pairs together: a register holds
                    // V[2t][2g], V[2t][2g+1], V[2t+1][2g], V[2t+1][2g+1] of one 16-column chunk, i.e. the B
                    // fragments of an "even columns" tile (bytes 0,2) and an "odd columns" tile (bytes 1,3).
#pragma unroll
                    for (int cp = 0; cp < 2; ++cp) {
                        uint32_t r0, r1, r2, r3;
                        ldmatrix_x4_trans(vb + v_row * 64 + (((2 * cp + v_chk) ^ ((v_row >> 1) & 3)) << 4), r0, r1, r2, r3);
                        r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
                        mma_16816(o[4 * cp + 0], pa[cp], s8_pair_to_half2(r0, 0x4240), s8_pair_to_half2(r1, 0x4240));
                        mma_16816(o[4 * cp + 1], pa[cp], s8_pair_to_half2(r0, 0x4341), s8_pair_to_half2(r1, 0x4341));
                        mma_16816(o[4 * cp + 2], pa[cp], s8_pair_to_half2(r2, 0x4240), s8_pair_to_half2(r3, 0x4240));
                        mma_16816(o[4 * cp + 3], pa[cp], s8_pair_to_half2(r2, 0x4341), s8_pair_to_half2(r3, 0x4341));
                    }
                }
            }
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (have[u] && lane == 0) mbar_arrive(empty0 + 8 * st[u]);
    }

    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);

    // merge the four warps through shared memory (re-using the first stage once all tiles are consumed)
    named_bar_sync(1, kConsumerWarps * 32);
    if (!ok || *reinterpret_cast<volatile int *>(&abort_flag)) return;
    float * scratch = reinterpret_cast<float *>(smem_gen);
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
    {
        const int hh = tid >> 4, d0 = (tid & 15) * 4;  // 8 heads x 16 threads x 4 values
        if (hh < p.gqa) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, scratch[(w * 8 + hh) * kPartialStride]);
            float L = 0.0f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float * src = scratch + (w * 8 + hh) * kPartialStride;
                const float   f   = src[0] == -INFINITY ? 0.0f : exp2f(src[0] - M);
                L += src[1] * f;
#pragma unroll
                for (int d = 0; d < 4; ++d) acc[d] += src[2 + d0 + d] * f;
            }
            const int head = kvh * p.gqa + hh;
            if (p.n_chunks == 1) {
                const float inv = L > 0.0f ? 1.0f / L : 0.0f;  // nothing visible -> zeros, as the reference
                float4      r   = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
                *reinterpret_cast<float4 *>(p.dst + ((size_t) stream * p.n_heads + head) * kHeadDim + d0) = r;
            } else {
                float * dstp = p.partial + (((size_t) stream * p.n_heads + head) * p.n_chunks + chunk_id) * kPartialStride;
                if ((tid & 15) == 0) { dstp[0] = M; dstp[1] = L; }
#pragma unroll
                for (int d = 0; d < 4; ++d) dstp[2 + d0 + d] = acc[d];
            }
        }
    }
    if (p.n_chunks == 1 || p.counters == nullptr) return;

    // Second pass without a second launch: every CTA of this (stream, kv head) takes a ticket after
    // publishing its partials; the one that draws the last ticket folds them all and resets the counter.
    // One fence by one thread after the barrier: the barrier orders every thread's partial stores before
    // it, and the fence is cumulative, so the ticket is taken only once they are visible device-wide.
    named_bar_sync(1, kConsumerWarps * 32);
    const int n_valid = min(p.n_chunks, (len + p.chunk - 1) / p.chunk);
    if (tid == 0) {
        int * ctr = p.counters + stream * gridDim.y + kvh;
        __threadfence();
        const int ticket = atomicAdd(ctr, 1);
        const int last   = ticket == n_valid - 1;
        if (last) *ctr = 0;
        abort_flag = last ? 2 : 0;  // the shared flag doubles as the broadcast slot: 2 = this CTA merges
    }
    named_bar_sync(1, kConsumerWarps * 32);
    if (*reinterpret_cast<volatile int *>(&abort_flag) != 2) return;
    __threadfence();
    {
        const int hh = tid >> 4, d0 = (tid & 15) * 4;
        if (hh < p.gqa) {
            const int     head = kvh * p.gqa + hh;
            const float * src  = p.partial + ((size_t) stream * p.n_heads + head) * p.n_chunks * kPartialStride;
            float M = -INFINITY;
            for (int c = 0; c < n_valid; ++c) M = fmaxf(M, __ldcg(src + c * kPartialStride));
            float L = 0.0f, acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c = 0; c < n_valid; ++c) {
                const float * pc = src + c * kPartialStride;
                const float   mc = __ldcg(pc);
                const float   f  = mc == -INFINITY ? 0.0f : exp2f(mc - M);
                L += __ldcg(pc + 1) * f;
                const float2 lo = __ldcg(reinterpret_cast<const float2 *>(pc + 2 + d0));
                const float2 hi = __ldcg(reinterpret_cast<const float2 *>(pc + 4 + d0));
                acc[0] += lo.x * f; acc[1] += lo.y * f; acc[2] += hi.x * f; acc[3] += hi.y * f;
            }
            const float inv = L > 0.0f ? 1.0f / L : 0.0f;
            *reinterpret_cast<float4 *>(p.dst + ((size_t) stream * p.n_heads + head) * kHeadDim + d0) =
                make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
        }
    }
}

// Second pass of split-KV as a kernel of its own: used when a launch has more (stream, kv head)
// pairs than the engine has ticket counters.
__global__ void __launch_bounds__(64) decode_merge_kernel(const DecodeParams p) {
    const int head = blockIdx.x, stream = blockIdx.y, d = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int len     = stream_len(p, stream);
    const int n_valid = min(p.n_chunks, (len + p.chunk - 1) / p.chunk);
    const float * src = p.partial + ((size_t) stream * p.n_heads + head) * p.n_chunks * kPartialStride;
    float M = -INFINITY;
    for (int c = 0; c < n_valid; ++c) M = fmaxf(M, src[c * kPartialStride]);
    float L = 0.0f, acc = 0.0f;
    for (int c = 0; c < n_valid; ++c) {
        const float mc = src[c * kPartialStride];
        const float f  = mc == -INFINITY ? 0.0f : exp2f(mc - M);
        L += src[c * kPartialStride + 1] * f;
        acc += src[c * kPartialStride + 2 + d] * f;
    }
    p.dst[((size_t) stream * p.n_heads + head) * kHeadDim + d] = L > 0.0f ? acc / L : 0.0f;
}

}  // namespace

namespace vox {

// Rows per CTA and CTAs per (stream, kv head).  A CTA is a copy pipeline that needs a few tiles to fill
// and pays a fixed cost at its end (warp merge, partial write, ticket), so chunks are long:
//   - at most 1024 rows per CTA (measured on 256 ragged streams: 768..4096 rows are within 3 % of each
//     other, 256 rows cost 40 %): with many (stream, kv head) pairs that alone gives several waves of CTAs;
//   - with few pairs, more CTAs per pair until the launch has about 1.5 CTAs per SM for f16 and 3.5 for
//     q8_0 (its arithmetic chain is longer and four of its CTAs fit an SM), but never below 256 rows per
//     CTA nor above 8 CTAs per pair (16 when there are only a handful of pairs): every further CTA adds a
//     partial to write, fence and fold.  Measured per layer, one stream: 8.0 -> 6.7 us at 1024 rows with
//     4 x 256 instead of 2 x 512;
//   - a launch that would need between 1 and 1.5 waves is cut back to one wave if chunks stay within 2048
//     rows (32 streams at 8192 rows: 34 -> 30 us with 6 x 1408 instead of 8 x 1024; 512 CTAs do not fit
//     the 444 resident slots);
//   - every chunk of a launch gets the same number of rows (a short last chunk leaves its CTA idle while
//     the others still stream: 640+640+640+128 measured 5 % slower than 4 x 512 at 2048 rows).
void decode_plan(bool q8, int n_streams, int n_kv_heads, int kv_bound, int * chunk, int * n_chunks) {
    const char *    env    = getenv("VOX_DECODE_CHUNK");  // tuning aid: rows per CTA, overrides the plan
    const int       forced = env ? atoi(env) : 0;
    const long long kv     = std::max(kv_bound, 1);
    const long long pairs  = (long long) n_streams * n_kv_heads;
    const long long target = q8 ? 512 : 222;
    const long long slots  = 148LL * (q8 ? Ring<true>::kCtasPerSm : Ring<false>::kCtasPerSm);
    auto            cdiv   = [](long long a, long long b) { return (a + b - 1) / b; };
    const long long most   = std::min(cdiv(kv, 256), std::max(8LL, std::min(16LL, 32 / pairs)));
    long long       n      = std::max(cdiv(kv, 1024), std::min(cdiv(target, pairs), most));
    if (pairs * n > slots && 2 * pairs * n < 3 * slots && slots / pairs >= std::max(4LL, cdiv(kv, 2048))) n = slots / pairs;
    long long c = cdiv(cdiv(kv, n), kKvTile) * kKvTile;
    if (forced >= kKvTile) c = (forced / kKvTile) * kKvTile;
    *chunk    = (int) c;
    *n_chunks = (int) cdiv(kv, c);
}

// Workspace for either cache type (the caller of the size query does not say which): the larger split.
size_t decode_workspace_bytes(int n_streams, int n_heads, int n_kv_heads, int kv_bound) {
    int chunk, n_f16, n_q8;
    decode_plan(false, n_streams, n_kv_heads, kv_bound, &chunk, &n_f16);
    decode_plan(true, n_streams, n_kv_heads, kv_bound, &chunk, &n_q8);
    const int n = std::max(n_f16, n_q8);
    return n <= 1 ? 0 : (size_t) n_streams * n_heads * n * kPartialStride * sizeof(float);
}

// K/V described by tensor maps (a cache layer, or caller tensors); q/dst/lengths by pointers.
// map_ks / map_vs are the scale planes of a q8_0 cache (null for f16).
int launch_decode(vox_engine * e, bool q8, const CUtensorMap & map_k, const CUtensorMap & map_v, const CUtensorMap * map_ks,
                  const CUtensorMap * map_vs, int layer, int max_len, int n_streams, int n_heads, int n_kv_heads,
                  const int32_t * kv_len, int kv_len_const, int kv_bound, const float * q, size_t q_nb_head,
                  size_t q_nb_stream, float * dst, float scale, void * workspace, size_t workspace_bytes,
                  cudaStream_t stream, const vox_kv_cache * append_to = nullptr, const float * k_new = nullptr,
                  const float * v_new = nullptr, size_t new_nb_head = 0, size_t new_nb_stream = 0, bool early = false,
                  const float * rope_table = nullptr, const int32_t * order = nullptr) {
    const uint32_t bit = q8 ? (1u << 9) : (1u << 8);
    if (!(e->attr_mask & bit)) {
        if (q8) VOX_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Ring<true>::kSmemBytes));
        else    VOX_CUDA_TRY(cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Ring<false>::kSmemBytes));
        e->attr_mask |= bit;
    }
    DecodeParams p;
    p.q = reinterpret_cast<const uint8_t *>(q);
    p.q_nb_head = q_nb_head; p.q_nb_stream = q_nb_stream;
    p.kv_len = kv_len; p.kv_len_const = kv_len_const;
    p.dst = dst; p.n_heads = n_heads; p.gqa = n_heads / n_kv_heads; p.layer = layer; p.max_len = max_len;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = e->status_dev;
    p.early = early ? 1 : 0;
    p.rope  = reinterpret_cast<const float2 *>(rope_table);
    p.order = order;
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
    decode_plan(q8, n_streams, n_kv_heads, kv_bound, &p.chunk, &p.n_chunks);
    const size_t need = p.n_chunks <= 1 ? 0 : (size_t) n_streams * n_heads * p.n_chunks * kPartialStride * sizeof(float);
    VOX_REQUIRE(workspace_bytes >= need && (need == 0 || workspace != nullptr), VOX_ATTN_WORKSPACE_TOO_SMALL,
                "decode needs %zu workspace bytes, got %zu", need, workspace_bytes);
    p.partial = static_cast<float *>(workspace);
    // fused second pass needs one ticket counter per (stream, kv head); larger launches use the merge kernel
    p.counters = (long long) n_streams * n_kv_heads <= kCounterSlots ? e->counters_dev : nullptr;
    dim3 grid(p.n_chunks, n_kv_heads, n_streams);
    if (q8) launch_pdl(decode_kernel<true>, grid, dim3(kThreads), Ring<true>::kSmemBytes, stream, map_k, map_v, *map_ks, *map_vs, p);
    else    launch_pdl(decode_kernel<false>, grid, dim3(kThreads), Ring<false>::kSmemBytes, stream, map_k, map_v, map_k, map_v, p);
    int rc = check_launch(e, q8 ? "decode_kernel<q8_0>" : "decode_kernel<f16>");
    if (rc != VOX_ATTN_OK) return rc;
    if (p.n_chunks > 1 && p.counters == nullptr) {
        launch_pdl(decode_merge_kernel, dim3(n_heads, n_streams), dim3(64), 0, stream, p);
        rc = check_launch(e, "decode_merge_kernel");
    }
    return rc;
}

int launch_decode_f16(vox_engine * e, const CUtensorMap & map_k, const CUtensorMap & map_v, int layer, int max_len,
                      int n_streams, int n_heads, int n_kv_heads, const int32_t * kv_len, int kv_len_const, int kv_bound,
                      const float * q, size_t q_nb_head, size_t q_nb_stream, float * dst, float scale, void * workspace,
                      size_t workspace_bytes, cudaStream_t stream) {
    return launch_decode(e, false, map_k, map_v, nullptr, nullptr, layer, max_len, n_streams, n_heads, n_kv_heads, kv_len,
                         kv_len_const, kv_bound, q, q_nb_head, q_nb_stream, dst, scale, workspace, workspace_bytes, stream);
}

// ---- single-token calls over q8_0 K/V in ggml's block layout (the operator called on a caller's own quantised
// cache, third_party/ggml/src/ggml-common.h:221-224): the blocks are taken apart into the planes the q8_0 decode
// kernel reads (int8 rows of 64 bytes, two f16 scales per row), in the workspace, and that kernel runs on them.
// Nothing is re-quantised: the result is what the cache object gives for the same blocks.

struct RepackParams {
    const uint8_t * src[2];
    size_t          nb1[2], nb2[2], nb3[2];
    uint8_t *       rows[2];    // [B][HK][n_pad][64] int8
    uint8_t *       scales[2];  // [B][HK][n_pad][2] f16
    int             n_kv, n_pad, n_kvh, n_batch;
};
__global__ void __launch_bounds__(256) q8_0_blocks_to_planes_kernel(const RepackParams p) {
    const long long n_blocks = 2LL * p.n_pad * p.n_kvh * p.n_batch;
    const bool      is_v     = blockIdx.y != 0;
    const uint8_t * src      = is_v ? p.src[1] : p.src[0];
    uint8_t *       rows     = is_v ? p.rows[1] : p.rows[0];
    uint8_t *       scales   = is_v ? p.scales[1] : p.scales[0];
    const size_t    nb1 = is_v ? p.nb1[1] : p.nb1[0], nb2 = is_v ? p.nb2[1] : p.nb2[0], nb3 = is_v ? p.nb3[1] : p.nb3[0];
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks; i += (long long) gridDim.x * blockDim.x) {
        const int       blk = (int) (i & 1);
        const long long row = i >> 1;
        const int       pos = (int) (row % p.n_pad);
        const int       kvh = (int) ((row / p.n_pad) % p.n_kvh);
        const int       b   = (int) (row / ((long long) p.n_pad * p.n_kvh));
        uint32_t        q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint16_t        d    = 0;  // rows past n_kv (up to the next multiple of the tile) hold zeros
        if (pos < p.n_kv) {
            const uint16_t * s = reinterpret_cast<const uint16_t *>(src + (size_t) pos * nb1 + (size_t) kvh * nb2 + (size_t) b * nb3 +
                                                                    (size_t) blk * 34);
            d = s[0];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = (uint32_t) s[1 + 2 * j] | ((uint32_t) s[2 + 2 * j] << 16);
        }
        uint4 * o = reinterpret_cast<uint4 *>(rows + (size_t) row * 64 + (size_t) blk * 32);
        o[0] = make_uint4(q[0], q[1], q[2], q[3]);
        o[1] = make_uint4(q[4], q[5], q[6], q[7]);
        reinterpret_cast<uint16_t *>(scales)[row * 2 + blk] = d;
    }
}

static size_t q8_planes_bytes(const vox_attn_args * a, int * n_pad_out) {
    const int n_pad = (int) ((a->k.ne[1] + kKvTile - 1) / kKvTile * kKvTile);
    if (n_pad_out) *n_pad_out = n_pad;
    const size_t rows = (size_t) n_pad * a->k.ne[2] * a->k.ne[3];
    return 2 * (rows * 64 + rows * 4);  // K and V: int8 rows + scale pairs (both multiples of 256 bytes)
}

bool decode_q8_blocks_route_ok(const vox_attn_args * a) {
    const vox_tensor &q = a->q, &k = a->k, &v = a->v;
    if (q.ne[1] != 1 || a->mask.data != nullptr) return false;
    if (k.type != VOX_TYPE_Q8_0 || v.type != VOX_TYPE_Q8_0) return false;
    if (k.ne[1] < 1 || k.ne[1] != v.ne[1] || k.ne[2] != v.ne[2] || k.ne[3] != v.ne[3] || q.ne[2] / k.ne[2] > 8) return false;
    for (const vox_tensor * t : {&k, &v})
        if ((reinterpret_cast<uintptr_t>(t->data) & 1) != 0 || t->nb[1] % 2 || t->nb[2] % 2 || t->nb[3] % 2) return false;
    return true;
}

size_t decode_q8_blocks_workspace_bytes(const vox_attn_args * a) {
    if (!decode_q8_blocks_route_ok(a)) return 0;
    const size_t partials = decode_workspace_bytes((int) a->q.ne[3], (int) a->q.ne[2], (int) a->k.ne[2], (int) a->k.ne[1]);
    return ((partials + 255) & ~(size_t) 255) + q8_planes_bytes(a, nullptr);
}

int launch_decode_q8_blocks(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t st) {
    int          n_pad = 0;
    const size_t planes = q8_planes_bytes(a, &n_pad);
    const int    B = (int) a->q.ne[3], HK = (int) a->k.ne[2], n_kv = (int) a->k.ne[1];
    const size_t partials = (decode_workspace_bytes(B, (int) a->q.ne[2], HK, n_kv) + 255) & ~(size_t) 255;
    VOX_REQUIRE(workspace != nullptr && workspace_bytes >= partials + planes && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                VOX_ATTN_WORKSPACE_TOO_SMALL, "q8_0 decode needs %zu workspace bytes, got %zu", partials + planes, workspace_bytes);
    uint8_t *    base = static_cast<uint8_t *>(workspace) + partials;
    const size_t rows = (size_t) n_pad * HK * B;
    RepackParams rp;
    const vox_tensor * ts[2] = {&a->k, &a->v};
    for (int i = 0; i < 2; ++i) {
        rp.src[i] = static_cast<const uint8_t *>(ts[i]->data);
        rp.nb1[i] = ts[i]->nb[1]; rp.nb2[i] = ts[i]->nb[2]; rp.nb3[i] = ts[i]->nb[3];
        rp.rows[i]   = base + i * rows * 64;
        rp.scales[i] = base + 2 * rows * 64 + i * rows * 4;
    }
    rp.n_kv = n_kv; rp.n_pad = n_pad; rp.n_kvh = HK; rp.n_batch = B;
    const long long n_blocks = 2LL * (long long) rows;
    const unsigned  gx = (unsigned) std::min<long long>((n_blocks + 255) / 256, 8LL * e->sm_count);
    q8_0_blocks_to_planes_kernel<<<dim3(gx, 2), 256, 0, st>>>(rp);
    int rc = check_launch(e, "q8_0_blocks_to_planes_kernel");
    if (rc != VOX_ATTN_OK) return rc;
    // the planes described as one cache layer of n_pad rows (the same descriptors vox_kv_create builds)
    CUtensorMap    mk, mv, mks, mvs;
    const uint64_t dims[5]     = {64, (uint64_t) n_pad, (uint64_t) HK, (uint64_t) B, 1};
    const uint64_t strides[4]  = {64, (uint64_t) 64 * n_pad, (uint64_t) 64 * n_pad * HK, (uint64_t) 64 * n_pad * HK * B};
    const uint32_t box[5]      = {64, kKvTile, 1, 1, 1};
    const uint64_t sdims[5]    = {(uint64_t) n_pad * 2, 1, (uint64_t) HK, (uint64_t) B, 1};
    const uint64_t sstrides[4] = {(uint64_t) 4 * n_pad, (uint64_t) 4 * n_pad, (uint64_t) 4 * n_pad * HK, (uint64_t) 4 * n_pad * HK * B};
    const uint32_t sbox[5]     = {2 * kKvTile, 1, 1, 1, 1};
    CUtensorMap * ms[2] = {&mk, &mv};
    CUtensorMap * ss[2] = {&mks, &mvs};
    for (int i = 0; i < 2; ++i) {
        rc = make_tensor_map(e, ms[i], rp.rows[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc == VOX_ATTN_OK)
            rc = make_tensor_map(e, ss[i], rp.scales[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, sdims, sstrides, sbox, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != VOX_ATTN_OK) return rc;
    }
    return launch_decode(e, true, mk, mv, &mks, &mvs, 0, n_pad, B, (int) a->q.ne[2], HK, nullptr, n_kv, n_kv,
                         static_cast<const float *>(a->q.data), a->q.nb[2], a->q.nb[3], static_cast<float *>(a->dst.data), a->scale,
                         workspace, partials, st);
}

}  // namespace vox

extern "C" {

size_t vox_attn_decode_workspace_bytes(int n_streams, int n_heads, int n_kv_heads, int kv_bound) {
    if (n_streams <= 0 || n_heads <= 0 || n_kv_heads <= 0) return 0;
    return decode_workspace_bytes(n_streams, n_heads, n_kv_heads, kv_bound);
}

int vox_attn_decode(vox_engine * e, const vox_decode_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    VOX_REQUIRE(e && a && a->cache && a->q && a->dst, VOX_ATTN_INVALID_ARGUMENT, "vox_attn_decode: null argument");
    const vox_kv_cache * c = a->cache;
    VOX_REQUIRE(c->e == e, VOX_ATTN_INVALID_ARGUMENT, "cache belongs to another engine");
    VOX_REQUIRE(a->layer >= 0 && a->layer < c->cfg.n_layers, VOX_ATTN_INVALID_ARGUMENT, "layer %d out of range", a->layer);
    VOX_REQUIRE(a->n_streams > 0 && a->n_streams <= c->cfg.n_streams, VOX_ATTN_INVALID_ARGUMENT,
                "n_streams %d out of range (cache holds %d)", a->n_streams, c->cfg.n_streams);
    VOX_REQUIRE(a->n_heads > 0 && a->n_heads % c->cfg.n_kv_heads == 0, VOX_ATTN_INVALID_ARGUMENT,
                "n_heads %d is not a multiple of n_kv_heads %d", a->n_heads, c->cfg.n_kv_heads);
    VOX_REQUIRE(a->n_heads / c->cfg.n_kv_heads <= 8, VOX_ATTN_UNSUPPORTED, "GQA ratio above 8 is not supported");
    VOX_REQUIRE(a->kv_len != nullptr, VOX_ATTN_INVALID_ARGUMENT, "kv_len is null");
    VOX_REQUIRE(a->kv_bound >= 0 && a->kv_bound <= c->cfg.max_len, VOX_ATTN_INVALID_ARGUMENT,
                "kv_bound %d exceeds the cache capacity %d", a->kv_bound, c->cfg.max_len);
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->q) & 7) == 0 && a->q_nb_head % 8 == 0 && a->q_nb_stream % 8 == 0,
                VOX_ATTN_INVALID_ARGUMENT, "q rows must be 8-byte aligned");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->dst) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT, "dst must be 16-byte aligned");
    const bool appends = a->k_new != nullptr || a->v_new != nullptr;
    if (appends) {
        VOX_REQUIRE(a->k_new && a->v_new, VOX_ATTN_INVALID_ARGUMENT, "k_new and v_new must be given together");
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->k_new) & 7) == 0 && (reinterpret_cast<uintptr_t>(a->v_new) & 7) == 0 &&
                        a->new_nb_head % 8 == 0 && a->new_nb_stream % 8 == 0,
                    VOX_ATTN_INVALID_ARGUMENT, "k_new / v_new rows must be 8-byte aligned");
        VOX_REQUIRE(a->kv_bound >= 1, VOX_ATTN_INVALID_ARGUMENT, "kv_bound counts the arriving row: it cannot be 0 with k_new");
    }
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->rope_table) & 7) == 0, VOX_ATTN_INVALID_ARGUMENT, "rope_table must be 8-byte aligned");
    return launch_decode(e, c->cfg.type == VOX_TYPE_Q8_0, c->map_k, c->map_v, &c->map_ks, &c->map_vs, a->layer, c->cfg.max_len, a->n_streams, a->n_heads, c->cfg.n_kv_heads,
                         a->kv_len, 0, a->kv_bound, a->q, a->q_nb_head, a->q_nb_stream, a->dst, a->scale, workspace,
                         workspace_bytes, static_cast<cudaStream_t>(stream), appends ? c : nullptr, a->k_new, a->v_new,
                         a->new_nb_head, a->new_nb_stream, (a->flags & VOX_DECODE_CACHE_STABLE) != 0, a->rope_table, a->stream_order);
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
constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB = 63 550 partials: e.g. 256 streams x 16 heads x 8192 rows (8 chunks each)
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

namespace {
constexpr int  kMaxDevices = 64;
unsigned char * g_scratch_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int vox_attn_decode_static(vox_engine * e, const vox_decode_args * a, void * stream) {
    VOX_REQUIRE(e && a && a->cache, VOX_ATTN_INVALID_ARGUMENT, "vox_attn_decode_static: null argument");
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
    // Nothing in the array has to start at zero: every partial a merge reads was written by the
    // decode kernel of the same call.  What the previous call left behind is simply overwritten.
    return vox_attn_decode(e, a, g_scratch_ptr[current], kStaticScratchBytes, stream);
}
