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
// The problems are tiny (seq <= 16, head_dim 64) and f32 end to end: a CTA owns one
// (stream, layer, branch, kv head) group, stages K, V and the group's Q rows in shared memory, and
// each of its warps serves one query head of the group.  The grid is persistent: min(#groups,
// resident CTAs) blocks walk the group list, so one launch covers any number of streams, and the
// operands of the next group are fetched with cp.async into a second buffer while the current
// group is computed.
#include "common.cuh"

#include <algorithm>

using namespace vox;

namespace {

constexpr int kMaxSeq  = 16;
constexpr int kRowPad  = 68;  // floats per staged row: 16-byte aligned, conflict-free for float4 reads
constexpr int kPPad    = 20;  // floats per row of a warp's probability matrix (16 columns + pad, 16-byte aligned)
constexpr int kMaxWarp = 8;   // query heads per kv head (GQA ratio)

struct LocditParams {
    const float *q, *k, *v;
    float *      dst;
    int          n_groups;  // streams * layers * 2 branches * kv heads
    int          n_heads, n_kv_heads, gqa, seq;
    float        scale;
};

__device__ __forceinline__ void cp_async16(float * smem_dst, const float * gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// SEQ > 0: sequence length known at compile time (loops unrolled, V columns kept in registers);
// SEQ == 0: any length up to kMaxSeq.
template <int SEQ>
__global__ void __launch_bounds__(kMaxWarp * 32) locdit_attn_kernel(const LocditParams p) {
    extern __shared__ __align__(16) float smem_f[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = SEQ > 0 ? SEQ : p.seq;
    // two stages of [K tile][V tile][one Q tile per warp], rows padded to kRowPad floats, then one
    // probability matrix per warp
    const int stage_floats = (2 + kMaxWarp) * seq * kRowPad;
    float *   pw           = smem_f + 2 * stage_floats + warp * seq * kPPad;
    const int vec_per_tile = seq * 16;  // float4 per [seq][64] tile

    auto issue_loads = [&](int grp, int buf) {
        float *   st   = smem_f + buf * stage_floats;
        const int kvh  = grp % p.n_kv_heads;
        const int slot = grp / p.n_kv_heads;  // (stream, layer, branch) flattened, branch fastest
        const float * kg = p.k + ((size_t) slot * p.n_kv_heads + kvh) * seq * kHeadDim;
        const float * vg = p.v + ((size_t) slot * p.n_kv_heads + kvh) * seq * kHeadDim;
        for (int i = tid; i < vec_per_tile; i += kMaxWarp * 32) {
            const int r = i >> 4, c = i & 15;
            cp_async16(st + r * kRowPad + c * 4, kg + i * 4);
            cp_async16(st + seq * kRowPad + r * kRowPad + c * 4, vg + i * 4);
        }
        if (warp < p.gqa) {
            const float * qg = p.q + ((size_t) slot * p.n_heads + kvh * p.gqa + warp) * seq * kHeadDim;
            float *       qw = st + (2 + warp) * seq * kRowPad;
            for (int i = lane; i < vec_per_tile; i += 32) {
                const int r = i >> 4, c = i & 15;
                cp_async16(qw + r * kRowPad + c * 4, qg + i * 4);
            }
        }
    };

    int grp = blockIdx.x, buf = 0;
    if (grp < p.n_groups) issue_loads(grp, buf);
    cp_async_commit();
    for (; grp < p.n_groups; grp += gridDim.x, buf ^= 1) {
        cp_async_wait_all();
        __syncthreads();  // this group's operands are visible; everyone is done with the other buffer
        if (grp + (int) gridDim.x < p.n_groups) issue_loads(grp + gridDim.x, buf ^ 1);
        cp_async_commit();
        if (warp >= p.gqa) continue;

        const float * st   = smem_f + buf * stage_floats;
        const float * ks   = st;
        const float * vs   = st + seq * kRowPad;
        const float * qw   = st + (2 + warp) * seq * kRowPad;
        const int     kvh  = grp % p.n_kv_heads;
        const int     slot = grp / p.n_kv_heads;
        const int     head = kvh * p.gqa + warp;

        // scores: (row, key) pairs dealt round-robin to lanes, each a 64-long f32 dot product
        for (int pi = lane; pi < seq * seq; pi += 32) {
            const int r = pi / seq, c = pi - r * seq;
            const float4 * qr = reinterpret_cast<const float4 *>(qw + r * kRowPad);
            const float4 * kr = reinterpret_cast<const float4 *>(ks + c * kRowPad);
            float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (int d = 0; d < 16; d += 2) {
                const float4 a = qr[d], b = kr[d], a2 = qr[d + 1], b2 = kr[d + 1];
                s0 += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
                s1 += a2.x * b2.x + a2.y * b2.y + a2.z * b2.z + a2.w * b2.w;
            }
            pw[r * kPPad + c] = (s0 + s1) * p.scale;
        }
        __syncwarp();
        if (lane < seq) {
            float * row = pw + lane * kPPad;
            float   mx  = -INFINITY;
#pragma unroll
            for (int c = 0; c < (SEQ > 0 ? SEQ : kMaxSeq); ++c)
                if (c < seq) mx = fmaxf(mx, row[c]);
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < (SEQ > 0 ? SEQ : kMaxSeq); ++c)
                if (c < seq) {
                    const float e = __expf(row[c] - mx);
                    row[c] = e;
                    sum += e;
                }
            const float inv = 1.0f / sum;
#pragma unroll
            for (int c = 0; c < (SEQ > 0 ? SEQ : kMaxSeq); ++c)
                if (c < seq) row[c] *= inv;
        }
        __syncwarp();
        // out[r][d] = sum_c P[r][c] V[c][d]; lane owns d = lane and lane + 32, with its two V columns in registers
        float v0[SEQ > 0 ? SEQ : kMaxSeq], v1[SEQ > 0 ? SEQ : kMaxSeq];
#pragma unroll
        for (int c = 0; c < (SEQ > 0 ? SEQ : kMaxSeq); ++c) {
            v0[c] = c < seq ? vs[c * kRowPad + lane] : 0.0f;
            v1[c] = c < seq ? vs[c * kRowPad + lane + 32] : 0.0f;
        }
        float * og = p.dst + ((size_t) slot * seq * p.n_heads + head) * kHeadDim;
        for (int r = 0; r < seq; ++r) {
            const float4 * prow = reinterpret_cast<const float4 *>(pw + r * kPPad);
            float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
            for (int c4 = 0; c4 < ((SEQ > 0 ? SEQ : kMaxSeq) + 3) / 4; ++c4) {
                const float4 w = prow[c4];  // columns past seq hold stale values; their V registers are zero
                const float  ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = c4 * 4 + j;
                    if (c < (SEQ > 0 ? SEQ : kMaxSeq) && c < seq) {
                        o0 += ww[j] * v0[c];
                        o1 += ww[j] * v1[c];
                    }
                }
            }
            float * orow = og + (size_t) r * p.n_heads * kHeadDim;  // result layout [D, H, seq, ...]
            orow[lane]      = o0;
            orow[lane + 32] = o1;
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
    VOX_REQUIRE(a->n_heads / a->n_kv_heads <= kMaxWarp, VOX_ATTN_UNSUPPORTED, "GQA ratio above %d is not supported", kMaxWarp);
    for (const void * ptr : {(const void *) a->q, (const void *) a->k, (const void *) a->v, (const void *) a->dst})
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT, "buffers must be 16-byte aligned");
    const long long groups = (long long) a->n_streams * a->n_layers * 2 * a->n_kv_heads;
    VOX_REQUIRE(groups < (1LL << 30), VOX_ATTN_INVALID_ARGUMENT, "too many attention groups");
    LocditParams p;
    p.q = a->q; p.k = a->k; p.v = a->v; p.dst = a->dst;
    p.n_groups = (int) groups; p.n_heads = a->n_heads; p.n_kv_heads = a->n_kv_heads;
    p.gqa = a->n_heads / a->n_kv_heads; p.seq = a->seq; p.scale = a->scale;
    const size_t smem = sizeof(float) * (2 * (size_t) (2 + kMaxWarp) * a->seq * kRowPad + (size_t) kMaxWarp * a->seq * kPPad);
    auto kernel = a->seq == 9 ? locdit_attn_kernel<9> : a->seq == 5 ? locdit_attn_kernel<5> : locdit_attn_kernel<0>;
    if (!(e->attr_mask & (1u << (a->seq == 9 ? 0 : a->seq == 5 ? 1 : 2)))) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
        e->attr_mask |= 1u << (a->seq == 9 ? 0 : a->seq == 5 ? 1 : 2);
    }
    const int per_sm   = (int) std::max<size_t>(1, std::min<size_t>(8, (220 * 1024) / (smem + 1024)));
    const int blocks   = (int) std::min<long long>(groups, (long long) e->sm_count * per_sm);
    kernel<<<blocks, kMaxWarp * 32, smem, static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch(e, "locdit_attn_kernel");
}
