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
// (stream, layer, branch, kv head) group, stages K and V once in shared memory, and each of its
// warps serves one query head of the group.  The grid is persistent: min(#groups, resident CTAs)
// blocks walk the group list, so one launch covers any number of streams.
#include "common.cuh"

#include <algorithm>

using namespace vox;

namespace {

constexpr int kMaxSeq  = 16;
constexpr int kRowPad  = 68;  // floats per staged row: 16-byte aligned, conflict-free for float4 reads
constexpr int kMaxWarp = 8;   // query heads per kv head (GQA ratio)

struct LocditParams {
    const float *q, *k, *v;
    float *      dst;
    int          n_groups;  // streams * layers * 2 branches * kv heads
    int          n_heads, n_kv_heads, gqa, seq;
    float        scale;
};

__global__ void __launch_bounds__(kMaxWarp * 32) locdit_attn_kernel(const LocditParams p) {
    extern __shared__ __align__(16) float smem_f[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = p.seq;
    // [K tile][V tile][one Q tile per warp][one score matrix per warp], rows padded to kRowPad floats
    float * ks = smem_f;
    float * vs = ks + seq * kRowPad;
    float * qw = vs + seq * kRowPad + warp * seq * kRowPad;
    float * pw = smem_f + (2 + kMaxWarp) * seq * kRowPad + warp * seq * (kMaxSeq + 1);
    const int vec_per_tile = seq * 16;  // float4 per [seq][64] tile

    for (int grp = blockIdx.x; grp < p.n_groups; grp += gridDim.x) {
        const int kvh  = grp % p.n_kv_heads;
        const int slot = grp / p.n_kv_heads;  // (stream, layer, branch) flattened, branch fastest
        const float4 * kg = reinterpret_cast<const float4 *>(p.k + ((size_t) slot * p.n_kv_heads + kvh) * seq * kHeadDim);
        const float4 * vg = reinterpret_cast<const float4 *>(p.v + ((size_t) slot * p.n_kv_heads + kvh) * seq * kHeadDim);
        for (int i = tid; i < vec_per_tile; i += blockDim.x) {
            const int r = i >> 4, c = i & 15;
            *reinterpret_cast<float4 *>(&ks[r * kRowPad + c * 4]) = kg[i];
            *reinterpret_cast<float4 *>(&vs[r * kRowPad + c * 4]) = vg[i];
        }
        if (warp < p.gqa) {
            const int head = kvh * p.gqa + warp;
            const float4 * qg = reinterpret_cast<const float4 *>(p.q + ((size_t) slot * p.n_heads + head) * seq * kHeadDim);
            for (int i = lane; i < vec_per_tile; i += 32) {
                const int r = i >> 4, c = i & 15;
                *reinterpret_cast<float4 *>(&qw[r * kRowPad + c * 4]) = qg[i];
            }
        }
        __syncthreads();

        if (warp < p.gqa) {
            const int head = kvh * p.gqa + warp;
            // scores: (row, key) pairs dealt round-robin to lanes, each a 64-long f32 dot product
            for (int pi = lane; pi < seq * seq; pi += 32) {
                const int r = pi / seq, c = pi - r * seq;
                const float4 * qr = reinterpret_cast<const float4 *>(&qw[r * kRowPad]);
                const float4 * kr = reinterpret_cast<const float4 *>(&ks[c * kRowPad]);
                float s = 0.0f;
#pragma unroll
                for (int d = 0; d < 16; ++d) {
                    const float4 a = qr[d], b = kr[d];
                    s += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
                }
                pw[r * (kMaxSeq + 1) + c] = s * p.scale;
            }
            __syncwarp();
            if (lane < seq) {
                float mx = -INFINITY;
                for (int c = 0; c < seq; ++c) mx = fmaxf(mx, pw[lane * (kMaxSeq + 1) + c]);
                float sum = 0.0f;
                for (int c = 0; c < seq; ++c) {
                    const float e = __expf(pw[lane * (kMaxSeq + 1) + c] - mx);
                    pw[lane * (kMaxSeq + 1) + c] = e;
                    sum += e;
                }
                const float inv = 1.0f / sum;
                for (int c = 0; c < seq; ++c) pw[lane * (kMaxSeq + 1) + c] *= inv;
            }
            __syncwarp();
            // out[r][d] = sum_c P[r][c] V[c][d]; lane owns d = lane and lane + 32
            float * og = p.dst + ((size_t) slot * seq * p.n_heads + head) * kHeadDim;
            for (int r = 0; r < seq; ++r) {
                float o0 = 0.0f, o1 = 0.0f;
                for (int c = 0; c < seq; ++c) {
                    const float w = pw[r * (kMaxSeq + 1) + c];
                    o0 += w * vs[c * kRowPad + lane];
                    o1 += w * vs[c * kRowPad + lane + 32];
                }
                float * orow = og + (size_t) r * p.n_heads * kHeadDim;  // result layout [D, H, seq, ...]
                orow[lane]      = o0;
                orow[lane + 32] = o1;
            }
        }
        __syncthreads();
    }
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
    VOX_REQUIRE(groups < (1LL << 31), VOX_ATTN_INVALID_ARGUMENT, "too many attention groups");
    LocditParams p;
    p.q = a->q; p.k = a->k; p.v = a->v; p.dst = a->dst;
    p.n_groups = (int) groups; p.n_heads = a->n_heads; p.n_kv_heads = a->n_kv_heads;
    p.gqa = a->n_heads / a->n_kv_heads; p.seq = a->seq; p.scale = a->scale;
    const size_t smem = sizeof(float) * ((size_t) (2 + kMaxWarp) * a->seq * kRowPad + (size_t) kMaxWarp * a->seq * (kMaxSeq + 1));
    static bool attr_done = false;
    if (!attr_done) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(locdit_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        attr_done = true;
    }
    const int resident = e->sm_count * (int) std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / (smem + 1024)));
    const int blocks   = (int) std::min<long long>(groups, resident);
    locdit_attn_kernel<<<blocks, kMaxWarp * 32, smem, static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch(e, "locdit_attn_kernel");
}
