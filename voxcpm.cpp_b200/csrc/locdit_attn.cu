// LocDiT CFG attention: every layer, both CFG branches and every head of one CFM timestep in a
// single persistent launch.
//
// Replaces the eight ggml_flash_attn_ext nodes per network evaluation that
// LocDiTModel::forward_cfg_pair_projected emits (src/locdit.cpp:401-464): there the cond and
// uncond branches are packed along the sequence axis (2 x 9 = 18 tokens) and separated by a
// block-diagonal f16 mask (src/locdit.cpp:63-130).  Here the branches are a batch axis, which is
// the same arithmetic without the masked half of the score matrix.  ggml-cuda would run
// flash_attn_ext_f16<64,64,32,1> plus two F32->F16 converts per node
// (third_party/ggml/src/ggml-cuda/fattn.cu:280-458, fattn-common.cuh:830-890).
//
// A CTA owns one (stream, layer, branch, kv head) group per trip of a persistent loop.  The query
// rows of the heads that share the kv head are contiguous in memory, so the group is ONE small
// matrix problem: S = Q[gqa*seq, 64] K^T[64, seq], a softmax over <= 16 keys per row, and
// O = P[gqa*seq, seq] V[seq, 64].  Each warp takes 16 of those rows and runs both products on the
// tensor cores (mma.m16n8k16, f16 operands, f32 accumulate).  To stay at f32 accuracy with f16
// operands every operand is split as hi + lo and three products are issued (hi*hi, hi*lo, lo*hi);
// the dropped lo*lo term is below 2^-22 relative.  Operands of the next group are fetched with
// cp.async into a second buffer while the current group is computed, so with many streams the
// kernel streams Q/K/V from HBM, and with one stream it is a single short launch per timestep.
// (Three and four buffers per CTA, i.e. two or three groups on their way, were measured: 80 and 118 us
// per 256-stream launch against 71 us with two, because fewer CTAs then fit an SM.  One buffer per CTA,
// only the warps that have rows and six CTAs per SM, meant for launches of few groups: 13.9 against 14.3
// us at 32 streams, 84 against 71 us at 256: not kept.  Unpadded, swizzled staging rows, with which four
// CTAs fit an SM instead of three: 72 against 71 us.  The kernel is not short of copies in flight.)
#include "common.cuh"

#include <algorithm>

using namespace vox;

namespace {

constexpr int kMaxSeq  = 16;
constexpr int kRowPad  = 72;   // floats per staged f32 row (288 B): 64-bit fragment reads are conflict-free
constexpr int kHalfPad = 72;   // halves per row of the f16 K/V tiles (144 B): ldmatrix rows fall in distinct banks
constexpr int kMaxWarp = 8;    // 16-row tiles per group: gqa * seq <= 128

struct LocditParams {
    const float *q, *k, *v;
    float *      dst;
    int          n_groups;  // streams * layers * 2 branches * kv heads
    int          n_heads, n_kv_heads, gqa, seq;
    float        scale_log2;
};

__device__ __forceinline__ void cp_async16(float * smem_dst, const float * gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// (x, y) -> packed f16 pair of the rounded values and packed f16 pair of the remainders
__device__ __forceinline__ void split_pair(float x, float y, uint32_t & hi, uint32_t & lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2  b = __half22float2(h);
    const __half2 r = __floats2half2_rn(x - b.x, y - b.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&r);
}

__global__ void __launch_bounds__(kMaxWarp * 32) locdit_attn_kernel(const LocditParams p) {
    extern __shared__ __align__(16) float smem_f[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int seq = p.seq, n_rows = p.gqa * seq;
    // two stages of f32 [K tile][V tile][Q rows of the group], then the f16 hi/lo tiles of K and V
    const int stage_floats = (2 * seq + n_rows) * kRowPad;
    __half *  kv16         = reinterpret_cast<__half *>(smem_f + 2 * stage_floats);  // [Khi][Klo][Vhi][Vlo], 16 x kHalfPad each
    const int q_vecs = n_rows * 16, kv_vecs = seq * 16;  // float4 per tile
    pdl_wait();
    pdl_launch_dependents();

    auto issue_loads = [&](int grp, int buf) {
        float *   st   = smem_f + buf * stage_floats;
        const int kvh  = grp % p.n_kv_heads;
        const int slot = grp / p.n_kv_heads;  // (stream, layer, branch) flattened, branch fastest
        const float * kg = p.k + ((size_t) slot * p.n_kv_heads + kvh) * seq * kHeadDim;
        const float * vg = p.v + ((size_t) slot * p.n_kv_heads + kvh) * seq * kHeadDim;
        const float * qg = p.q + ((size_t) slot * p.n_heads + kvh * p.gqa) * seq * kHeadDim;  // gqa heads x seq rows, contiguous
        for (int i = tid; i < kv_vecs; i += kMaxWarp * 32) {
            const int r = i >> 4, c = i & 15;
            cp_async16(st + r * kRowPad + c * 4, kg + i * 4);
            cp_async16(st + (seq + r) * kRowPad + c * 4, vg + i * 4);
        }
        for (int i = tid; i < q_vecs; i += kMaxWarp * 32) {
            const int r = i >> 4, c = i & 15;
            cp_async16(st + (2 * seq + r) * kRowPad + c * 4, qg + i * 4);
        }
    };

    int grp = blockIdx.x, buf = 0;
    if (grp < p.n_groups) issue_loads(grp, buf);
    cp_async_commit();
    for (; grp < p.n_groups; grp += gridDim.x, buf ^= 1) {
        cp_async_wait_all();
        __syncthreads();  // this group's operands are visible; everyone is done with the other buffer and the f16 tiles
        if (grp + (int) gridDim.x < p.n_groups) issue_loads(grp + gridDim.x, buf ^ 1);
        cp_async_commit();

        const float * st = smem_f + buf * stage_floats;
        // K and V -> f16 hi/lo tiles of 16 rows (rows past seq are zero), once per group for all warps
        for (int i = tid; i < 2 * 16 * 32; i += kMaxWarp * 32) {
            const int which = i >> 9, row = (i >> 5) & 15, dp = i & 31;
            float2 x = make_float2(0.0f, 0.0f);
            if (row < seq) x = *reinterpret_cast<const float2 *>(st + (which * seq + row) * kRowPad + 2 * dp);
            uint32_t hi, lo;
            split_pair(x.x, x.y, hi, lo);
            __half * tile = kv16 + which * 2 * 16 * kHalfPad + row * kHalfPad + 2 * dp;
            *reinterpret_cast<uint32_t *>(tile)                 = hi;
            *reinterpret_cast<uint32_t *>(tile + 16 * kHalfPad) = lo;
        }
        __syncthreads();

        const int row0 = 16 * warp;
        if (row0 >= n_rows) continue;
        const int     kvh  = grp % p.n_kv_heads;
        const int     slot = grp / p.n_kv_heads;
        const float * qs   = st + 2 * seq * kRowPad;
        const int     ra = row0 + g, rb = row0 + g + 8;  // the two rows this lane holds in every fragment

        // ---- S = Q K^T, three products per (key tile, k-step)
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const uint32_t k_hi = smem_u32(kv16), k_lo = k_hi + 16 * kHalfPad * 2;
        const int      lm_row = ((lane >> 4) << 3) + (lane & 7), lm_chk = (lane >> 3) & 1;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t ahi[4], alo[4];
            {
                const float2 z  = make_float2(0.0f, 0.0f);
                const float2 xa = ra < n_rows ? *reinterpret_cast<const float2 *>(qs + ra * kRowPad + 16 * c + 2 * t) : z;
                const float2 ya = ra < n_rows ? *reinterpret_cast<const float2 *>(qs + ra * kRowPad + 16 * c + 8 + 2 * t) : z;
                const float2 xb = rb < n_rows ? *reinterpret_cast<const float2 *>(qs + rb * kRowPad + 16 * c + 2 * t) : z;
                const float2 yb = rb < n_rows ? *reinterpret_cast<const float2 *>(qs + rb * kRowPad + 16 * c + 8 + 2 * t) : z;
                split_pair(xa.x, xa.y, ahi[0], alo[0]);
                split_pair(xb.x, xb.y, ahi[1], alo[1]);
                split_pair(ya.x, ya.y, ahi[2], alo[2]);
                split_pair(yb.x, yb.y, ahi[3], alo[3]);
            }
            uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
            const uint32_t off = (lm_row * kHalfPad + (2 * c + lm_chk) * 8) * 2;
            ldmatrix_x4(k_hi + off, h0, h1, h2, h3);
            ldmatrix_x4(k_lo + off, l0, l1, l2, l3);
            mma_16816(sc[0], ahi, h0, h1);
            mma_16816(sc[1], ahi, h2, h3);
            mma_16816(sc[0], ahi, l0, l1);
            mma_16816(sc[1], ahi, l2, l3);
            mma_16816(sc[0], alo, h0, h1);
            mma_16816(sc[1], alo, h2, h3);
        }

        // ---- softmax over the keys of each row (registers 0,1 = row ra, 2,3 = row rb; tile j holds keys 8j+2t, 8j+2t+1)
        float pa[2][2], pb[2][2];
        float ma = -INFINITY, mb = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool vis = 8 * j + 2 * t + e < seq;
                pa[j][e] = vis ? sc[j][e] * p.scale_log2 : -INFINITY;
                pb[j][e] = vis ? sc[j][2 + e] * p.scale_log2 : -INFINITY;
                ma = fmaxf(ma, pa[j][e]);
                mb = fmaxf(mb, pb[j][e]);
            }
        ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 1));
        mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
        ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 2));
        mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
        float sa = 0.0f, sb = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                pa[j][e] = ex2_approx(pa[j][e] - ma);  // key 0 is always visible: the maxima are finite
                pb[j][e] = ex2_approx(pb[j][e] - mb);
                sa += pa[j][e];
                sb += pb[j][e];
            }
        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
        sb += __shfl_xor_sync(0xffffffffu, sb, 1);
        sa += __shfl_xor_sync(0xffffffffu, sa, 2);
        sb += __shfl_xor_sync(0xffffffffu, sb, 2);
        const float ia = 1.0f / sa, ib = 1.0f / sb;
        // the two key tiles of S are exactly the A fragment of one k-step of P V
        uint32_t phi[4], plo[4];
        split_pair(pa[0][0] * ia, pa[0][1] * ia, phi[0], plo[0]);
        split_pair(pb[0][0] * ib, pb[0][1] * ib, phi[1], plo[1]);
        split_pair(pa[1][0] * ia, pa[1][1] * ia, phi[2], plo[2]);
        split_pair(pb[1][0] * ib, pb[1][1] * ib, phi[3], plo[3]);

        // ---- O = P V and store: output tile n holds columns 8n+2t, 8n+2t+1 of rows ra, rb
        const uint32_t v_hi = k_hi + 2 * 16 * kHalfPad * 2, v_lo = v_hi + 16 * kHalfPad * 2;
        const int      vt_row = (((lane >> 3) & 1) << 3) + (lane & 7), vt_chk = lane >> 4;
        const int      ha = ra / seq, hb = rb / seq;
        float * oa = p.dst + (((size_t) slot * seq + (ra - ha * seq)) * p.n_heads + kvh * p.gqa + ha) * kHeadDim + 2 * t;
        float * ob = p.dst + (((size_t) slot * seq + (rb - hb * seq)) * p.n_heads + kvh * p.gqa + hb) * kHeadDim + 2 * t;
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
            float o0[4] = {0.f, 0.f, 0.f, 0.f}, o1[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
            const uint32_t off = (vt_row * kHalfPad + (2 * n2 + vt_chk) * 8) * 2;
            ldmatrix_x4_trans(v_hi + off, h0, h1, h2, h3);
            ldmatrix_x4_trans(v_lo + off, l0, l1, l2, l3);
            mma_16816(o0, phi, h0, h1);
            mma_16816(o1, phi, h2, h3);
            mma_16816(o0, phi, l0, l1);
            mma_16816(o1, phi, l2, l3);
            mma_16816(o0, plo, h0, h1);
            mma_16816(o1, plo, h2, h3);
            if (ra < n_rows) {
                *reinterpret_cast<float2 *>(oa + 16 * n2)     = make_float2(o0[0], o0[1]);
                *reinterpret_cast<float2 *>(oa + 16 * n2 + 8) = make_float2(o1[0], o1[1]);
            }
            if (rb < n_rows) {
                *reinterpret_cast<float2 *>(ob + 16 * n2)     = make_float2(o0[2], o0[3]);
                *reinterpret_cast<float2 *>(ob + 16 * n2 + 8) = make_float2(o1[2], o1[3]);
            }
        }
    }
    cp_async_wait_all();
}

}  // namespace

extern "C" int vox_attn_locdit_step(vox_engine * e, const vox_locdit_args * a, void * stream) {
    VOX_REQUIRE(e && a && a->q && a->k && a->v && a->dst, VOX_ATTN_INVALID_ARGUMENT, "vox_attn_locdit_step: null argument");
    VOX_REQUIRE(a->head_dim == kHeadDim, VOX_ATTN_UNSUPPORTED, "head_dim %d not supported (64 only)", a->head_dim);
    VOX_REQUIRE(a->seq >= 1 && a->seq <= kMaxSeq, VOX_ATTN_UNSUPPORTED, "seq %d not supported (1..%d)", a->seq, kMaxSeq);
    VOX_REQUIRE(a->n_streams > 0 && a->n_layers > 0 && a->n_heads > 0 && a->n_kv_heads > 0, VOX_ATTN_INVALID_ARGUMENT,
                "extents must be positive");
    VOX_REQUIRE(a->n_heads % a->n_kv_heads == 0, VOX_ATTN_INVALID_ARGUMENT, "n_heads %d is not a multiple of n_kv_heads %d",
                a->n_heads, a->n_kv_heads);
    VOX_REQUIRE(a->n_heads / a->n_kv_heads <= 8, VOX_ATTN_UNSUPPORTED, "GQA ratio above 8 is not supported");
    for (const void * ptr : {(const void *) a->q, (const void *) a->k, (const void *) a->v, (const void *) a->dst})
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT, "buffers must be 16-byte aligned");
    const long long groups = (long long) a->n_streams * a->n_layers * 2 * a->n_kv_heads;
    VOX_REQUIRE(groups < (1LL << 30), VOX_ATTN_INVALID_ARGUMENT, "too many attention groups");
    LocditParams p;
    p.q = a->q; p.k = a->k; p.v = a->v; p.dst = a->dst;
    p.n_groups = (int) groups; p.n_heads = a->n_heads; p.n_kv_heads = a->n_kv_heads;
    p.gqa = a->n_heads / a->n_kv_heads; p.seq = a->seq; p.scale_log2 = a->scale * 1.4426950408889634f;
    const int    n_rows = p.gqa * a->seq;
    const size_t smem   = sizeof(float) * 2 * (size_t) (2 * a->seq + n_rows) * kRowPad + sizeof(__half) * 4 * 16 * kHalfPad;
    if (!(e->attr_mask & 1u)) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(locdit_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
        e->attr_mask |= 1u;
    }
    const int per_sm = (int) std::max<size_t>(1, std::min<size_t>(6, (220 * 1024) / (smem + 1024)));
    const int blocks = (int) std::min<long long>(groups, (long long) e->sm_count * per_sm);
    launch_pdl(locdit_attn_kernel, dim3(blocks), dim3(kMaxWarp * 32), smem, static_cast<cudaStream_t>(stream), p);
    return check_launch(e, "locdit_attn_kernel");
}
