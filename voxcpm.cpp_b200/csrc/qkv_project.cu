// Batched Q/K/V projection of a decode step, with the rotary embedding and the cache store in its epilogue.
//
// Replaces, for the single-token step of every stream of a group, the three graph nodes in front of attention in
// MiniCPMModel::attention_forward (src/minicpm.cpp:644-701): ggml_mul_mat(qkv_proj, hidden) (or the separate q/k/v
// projections stacked), apply_rope on q and k (:582-600, ggml_rope_ext NEOX), and the ggml_cpy of the new K/V rows into the
// cache views (:684-685).  The reference runs them once per stream, so the projection weights (2.6 MB of f16 for
// 1024 -> 1280) are read once per stream and step; here ONE launch serves all streams of a group, the weights are read
// once, and Q leaves in the layout the decode launch reads while K and V go straight into the cache rows (or, for a
// host that keeps the two apart, into f32 rows for the decode launch's own store).
//
// Arithmetic as the reference's CPU backend does it for f16 weights (ggml_compute_forward_mul_mat with vec_dot_type
// F16, third_party/ggml/src/ggml-cpu/ggml-cpu.c:217; ggml_vec_dot_f16, ggml-cpu/vec.cpp:264): the activations are
// rounded to f16, products are exact, accumulation is f32.
//
// Kernel: D[tokens, features] = X[tokens, K] . W[features, K]^T on tcgen05.  A CTA owns 128 tokens x one head
// (64 features): both operands are K-major (a token's hidden vector, a feature's weight row), fetched by bulk-tensor
// copies in 64-wide K blocks (128-byte rows, 128-byte swizzle) into a four-stage ring; one thread issues
// tcgen05.mma (kind::f16, M = 128, N = 64, four k-steps per block), the accumulator (64 columns of TMEM) is read
// by four warps, one thread per token: that thread holds the token's whole head, so the rotary pairs (i, i + 32) and
// the q8_0 block maxima are all inside one thread.
// What bounds it: a CTA fills its shared memory at about 45 KB/us and a whole K range is 384 KB per CTA (two thirds of
// it the activations, which every head's CTA of a token tile fetches again from the L2), so the 40 CTAs of a
// 256-stream launch take about 10 us on 40 of the 148 SMs.  Tried: a ring of eight stages (no change: the ring is not
// what it waits for); the K range split over four CTAs with their partial sums folded by the last to finish through
// the workspace (160 CTAs: 21 us, the fold and a second wave cost more than the split saves).
#include "kv_cache.cuh"
#include "tcgen05.cuh"

#include <algorithm>

using namespace vox;

namespace {

constexpr int kTokTile  = 128;                      // tokens per CTA (TMEM lanes)
constexpr int kKBlock   = 64;                       // K elements per stage: 128-byte rows
constexpr int kRing     = 4;
constexpr int kABytes   = kTokTile * 128;           // [128 tokens][64 k] f16
constexpr int kBBytes   = kHeadDim * 128;           // [64 features][64 k] f16
constexpr int kStageQkv = kABytes + kBBytes;
constexpr int kSmemQkv  = kRing * kStageQkv + 1024;
constexpr int kThreadsQkv = 256;                    // producer, issuer, two idle warps, four epilogue warps
constexpr int kStageRow   = kHeadDim + 4;           // floats per row of the epilogue's staging tile (padded against bank conflicts)
static_assert(kRing * kStageQkv >= kTokTile * kStageRow * 4, "the idle ring holds the staging tile");

struct QkvParams {
    int             n_streams, k_dim, n_heads, n_kv_heads;
    const float2 *  rope;       // [stream][32] (cos, sin) or null
    float *         q;          // [stream][H][64]
    float *         k_new;      // [stream][HK][64] or null
    float *         v_new;
    // cache rows (k_new == null): this layer's K / V rows (q8_0: bytes and scales of its first tile) and their strides
    uint8_t *       k_rows;
    uint8_t *       v_rows;
    uint8_t *       k_scales;
    uint8_t *       v_scales;
    size_t          nb_pos, nb_head, nb_stream, sb_pos, sb_head, sb_stream;
    const int32_t * positions;  // [stream]: the row each stream's K/V go to (+ pos_offset)
    int             pos_offset, max_len, cache_type;
    int *           status;
};

__global__ void __launch_bounds__(256) f32_to_f16_rows_kernel(const uint8_t * x, size_t nb_stream, int k_dim, int n_streams, __half * out) {
    pdl_wait();
    pdl_launch_dependents();
    const long long n = (long long) n_streams * (k_dim / 4);
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long) gridDim.x * blockDim.x) {
        const int    s = (int) (i / (k_dim / 4)), c = (int) (i % (k_dim / 4));
        const float4 v = *reinterpret_cast<const float4 *>(x + (size_t) s * nb_stream + (size_t) c * 16);
        const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        *reinterpret_cast<uint2 *>(out + (size_t) s * k_dim + 4 * c) =
            make_uint2(*reinterpret_cast<const uint32_t *>(&a), *reinterpret_cast<const uint32_t *>(&b));
    }
}

// one cache row (64 values held by one thread) in the cache's type
__device__ __forceinline__ void store_cache_row(const QkvParams & p, uint8_t * rows, uint8_t * scales, int stream, int kvh, int pos,
                                                const float (&x)[64]) {
    uint8_t * pair = rows + (size_t) stream * p.nb_stream + (size_t) kvh * p.nb_head;
    if (p.cache_type == VOX_TYPE_F16) {
        uint8_t * dst = pair + (size_t) pos * p.nb_pos;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4 *>(dst + 16 * c) = make_uint4(pack_half2(x[8 * c], x[8 * c + 1]), pack_half2(x[8 * c + 2], x[8 * c + 3]),
                                                                   pack_half2(x[8 * c + 4], x[8 * c + 5]), pack_half2(x[8 * c + 6], x[8 * c + 7]));
    } else {
        // quantize_row_q8_0_ref (third_party/ggml/src/ggml-quants.c:199-222) on each 32-value block; bytes stored as q + 128,
        // in the row's place inside its tile of the cache (16-byte pieces, swizzled: q8_byte_off)
        uint8_t * dst  = pair + q8_tile_off(pos);
        uint8_t * sdst = scales + (size_t) stream * p.sb_stream + (size_t) kvh * p.sb_head + q8_tile_off(pos) + q8_scale_off(pos, 0);
        __half    d2[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[32 * b + i]));
            const float d  = amax / 127.0f;
            const float id = d != 0.0f ? 1.0f / d : 0.0f;
            d2[b] = __float2half_rn(d);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t wds[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t word = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int qv = (int) roundf(x[32 * b + 16 * c + 4 * j + e] * id) + 128;
                        word |= (uint32_t) (qv & 0xff) << (8 * e);
                    }
                    wds[j] = word;
                }
                *reinterpret_cast<uint4 *>(dst + q8_byte_off(pos, 32 * b + 16 * c)) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
            }
        }
        *reinterpret_cast<__half2 *>(sdst) = __halves2half2(d2[0], d2[1]);
    }
}

__global__ void __launch_bounds__(kThreadsQkv, 2)
qkv_project_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const QkvParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * kRing + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int      abort_flag;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int      tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int      head = blockIdx.x;            // 0 .. H-1: Q heads, then HK K heads, then HK V heads
    const int      tok0 = blockIdx.y * kTokTile;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = full0 + 8 * kRing, done = empty0 + 8 * kRing;
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kRing; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(done, 1);
        fence_mbar_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), 64);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();  // the f16 copy of the activations comes from the kernel before
    pdl_launch_dependents();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&tmem_base_slot);
    const int      n_kb = p.k_dim / kKBlock;
    auto give_up = [&]() {
        atomicOr(p.status, kStatusTimeout);
        atomicExch(&abort_flag, 1);
    };
    auto aborted = [&]() { return *reinterpret_cast<volatile int *>(&abort_flag) != 0; };

    if (warp == 0) {
        if (lane == 0) {  // producer: X rows of this token tile and W rows of this head, one K block per stage
            for (int kb = 0; kb < n_kb && !aborted(); ++kb) {
                const int st = kb % kRing;
                if (kb >= kRing && !mbar_wait_bounded(empty0 + 8 * st, ((kb / kRing) - 1) & 1)) { give_up(); break; }
                const uint32_t sa = smem_base + st * kStageQkv;
                mbar_expect_tx(full0 + 8 * st, kStageQkv);
                tma_load_5d(sa, &map_x, full0 + 8 * st, kb * kKBlock, tok0, 0, 0, 0);
                tma_load_5d(sa + kABytes, &map_w, full0 + 8 * st, kb * kKBlock, head * kHeadDim, 0, 0, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // issuer
            constexpr uint32_t idesc = idesc_f16(kHeadDim, false);
            const uint64_t     dA = smem_desc_sw128(smem_base), dB = smem_desc_sw128(smem_base + kABytes);
            bool ok = true;
            for (int kb = 0; kb < n_kb && !aborted(); ++kb) {
                const int st = kb % kRing;
                if (!mbar_wait_bounded(full0 + 8 * st, (kb / kRing) & 1)) { give_up(); ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < kKBlock / 16; ++k)
                    tc_mma_f16(tmem, dA + (uint64_t) st * (kStageQkv >> 4) + k * 2, dB + (uint64_t) st * (kStageQkv >> 4) + k * 2, idesc,
                               (kb | k) != 0);
                tc_commit(empty0 + 8 * st);  // the stage may be refilled once these have retired
            }
            if (ok) tc_commit(done);
        }
    } else if (warp >= 4) {
        // epilogue: one thread per token
        const int row = tid - 128, token = tok0 + row;
        const bool arrived = mbar_wait_bounded(done, 0);
        if (!arrived) give_up();
        if (arrived) {
            tc_fence_after();
            uint32_t r[64];
            tmem_ld64_sync(tmem + ((uint32_t) (32 * (warp & 3)) << 16), r);
            if (token < p.n_streams) {
                float x[64];
#pragma unroll
                for (int i = 0; i < 64; ++i) x[i] = __uint_as_float(r[i]);
                const bool is_q = head < p.n_heads, is_k = !is_q && head < p.n_heads + p.n_kv_heads;
                if (p.rope != nullptr && (is_q || is_k)) {
                    // element i with element i + 32, separate multiplies and adds in the operand order of the reference's
                    // rotate_pairs (third_party/ggml/src/ggml-cpu/ops.cpp, ggml_rope_ext with GGML_ROPE_TYPE_NEOX)
                    const float2 * tb = p.rope + (size_t) token * 32;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float2 cs = tb[i];
                        const float  x0 = x[i], x1 = x[i + 32];
                        x[i]      = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
                        x[i + 32] = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
                    }
                }
                if (!is_q && p.k_new == nullptr) {
                    const int kvh = is_k ? head - p.n_heads : head - p.n_heads - p.n_kv_heads;
                    const int pos = p.positions[token] + p.pos_offset;
                    if (pos < 0 || pos >= p.max_len) atomicOr(p.status, kStatusBadState);  // never write outside the stream's rows
                    else store_cache_row(p, is_k ? p.k_rows : p.v_rows, is_k ? p.k_scales : p.v_scales, token, kvh, pos, x);
                } else {
                    // f32 rows leave through shared memory (the ring is idle by now), so that neighbouring threads write
                    // neighbouring 16-byte pieces of a token's row instead of each thread its own row, 4 KB from the next
                    float4 * stage = reinterpret_cast<float4 *>(smem_raw + (smem_base - smem_u32(smem_raw))) + (size_t) row * (kStageRow / 4);
#pragma unroll
                    for (int i = 0; i < 16; ++i) stage[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
                }
            }
        }
        {
            const bool f32_rows = head < p.n_heads || p.k_new != nullptr;  // the same for every thread of the CTA
            if (f32_rows) {
                named_bar_sync(1, 128);  // every epilogue thread gets here, whatever became of its wait
                if (aborted()) goto epilogue_done;
                const bool is_q = head < p.n_heads, is_k = !is_q && head < p.n_heads + p.n_kv_heads;
                float *    base = is_q ? p.q + (size_t) head * kHeadDim
                                       : (is_k ? p.k_new + (size_t) (head - p.n_heads) * kHeadDim : p.v_new + (size_t) (head - p.n_heads - p.n_kv_heads) * kHeadDim);
                const size_t tok_stride = (size_t) (is_q ? p.n_heads : p.n_kv_heads) * kHeadDim;
                for (int pc = row; pc < kTokTile * 16; pc += 128) {
                    const int rr = pc >> 4, q4 = pc & 15;
                    if (tok0 + rr >= p.n_streams) break;
                    const float4 v = reinterpret_cast<const float4 *>(smem_raw + (smem_base - smem_u32(smem_raw)))[(size_t) rr * (kStageRow / 4) + q4];
                    reinterpret_cast<float4 *>(base + (size_t) (tok0 + rr) * tok_stride)[q4] = v;
                }
            }
        }
    }
epilogue_done:
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 64);
    }
}

}  // namespace

extern "C" {

size_t vox_qkv_workspace_bytes(int n_streams, int hidden) {
    if (n_streams <= 0 || hidden <= 0) return 0;
    return ((size_t) n_streams * hidden * sizeof(__half) + 255) & ~(size_t) 255;
}

int vox_qkv_project(vox_engine * e, const vox_qkv_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    VOX_REQUIRE(e && a && a->x && a->w_qkv && a->q, VOX_ATTN_INVALID_ARGUMENT, "vox_qkv_project: null argument");
    VOX_REQUIRE(a->head_dim == kHeadDim, VOX_ATTN_UNSUPPORTED, "head_dim %d not supported (64 only)", a->head_dim);
    VOX_REQUIRE(a->w_type == VOX_TYPE_F16, VOX_ATTN_UNSUPPORTED, "projection weights of type %d are not supported (f16 only)", a->w_type);
    VOX_REQUIRE(a->n_streams > 0 && a->n_heads > 0 && a->n_kv_heads > 0, VOX_ATTN_INVALID_ARGUMENT, "bad stream or head counts");
    VOX_REQUIRE(a->hidden > 0 && a->hidden % kKBlock == 0, VOX_ATTN_UNSUPPORTED, "hidden size %d is not a multiple of 64", a->hidden);
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->x) & 15) == 0 && a->x_nb_stream % 16 == 0 && a->x_nb_stream >= (size_t) a->hidden * 4,
                VOX_ATTN_INVALID_ARGUMENT, "x columns must be 16-byte aligned and at least hidden floats apart");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->w_qkv) & 15) == 0 && a->w_nb_row % 16 == 0 && a->w_nb_row >= (size_t) a->hidden * 2,
                VOX_ATTN_INVALID_ARGUMENT, "weight rows must be 16-byte aligned and at least hidden halves apart");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->q) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT, "q must be 16-byte aligned");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->rope_table) & 7) == 0, VOX_ATTN_INVALID_ARGUMENT, "rope_table must be 8-byte aligned");
    const bool to_cache = a->cache != nullptr;
    if (to_cache) {
        const vox_kv_cache * c = a->cache;
        VOX_REQUIRE(c->e == e, VOX_ATTN_INVALID_ARGUMENT, "cache belongs to another engine");
        VOX_REQUIRE(a->layer >= 0 && a->layer < c->cfg.n_layers, VOX_ATTN_INVALID_ARGUMENT, "layer %d out of range", a->layer);
        VOX_REQUIRE(a->n_streams <= c->cfg.n_streams && a->n_kv_heads == c->cfg.n_kv_heads, VOX_ATTN_INVALID_ARGUMENT,
                    "streams or kv heads do not fit the cache");
        VOX_REQUIRE(a->positions != nullptr, VOX_ATTN_INVALID_ARGUMENT, "positions is null");
        VOX_REQUIRE(a->k_new == nullptr && a->v_new == nullptr, VOX_ATTN_INVALID_ARGUMENT, "give a cache or k_new / v_new, not both");
    } else {
        VOX_REQUIRE(a->k_new && a->v_new, VOX_ATTN_INVALID_ARGUMENT, "k_new and v_new (or a cache) are needed");
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->k_new) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->v_new) & 15) == 0,
                    VOX_ATTN_INVALID_ARGUMENT, "k_new / v_new must be 16-byte aligned");
    }
    const size_t need = vox_qkv_workspace_bytes(a->n_streams, a->hidden);
    VOX_REQUIRE(workspace != nullptr && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                VOX_ATTN_WORKSPACE_TOO_SMALL, "the projection needs %zu workspace bytes (16-byte aligned), got %zu", need, workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!(e->attr_mask & (1u << 14))) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(qkv_project_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemQkv));
        e->attr_mask |= 1u << 14;
    }
    // activations rounded to f16 once, [stream][hidden] (where a fused norm would write them in the first place)
    __half *       x16 = static_cast<__half *>(workspace);
    const long long quads = (long long) a->n_streams * (a->hidden / 4);
    launch_pdl(f32_to_f16_rows_kernel, dim3((unsigned) std::min<long long>((quads + 255) / 256, 4LL * e->sm_count)), dim3(256), 0, st,
               reinterpret_cast<const uint8_t *>(a->x), a->x_nb_stream, a->hidden, a->n_streams, x16);
    int rc = check_launch(e, "f32_to_f16_rows_kernel");
    if (rc != VOX_ATTN_OK) return rc;

    const int n_out = (a->n_heads + 2 * a->n_kv_heads) * kHeadDim;
    CUtensorMap    mx, mw;
    const uint64_t xd[5] = {(uint64_t) a->hidden, (uint64_t) a->n_streams, 1, 1, 1};
    const uint64_t xs[4] = {(uint64_t) a->hidden * 2, (uint64_t) a->hidden * 2 * a->n_streams, (uint64_t) a->hidden * 2 * a->n_streams,
                            (uint64_t) a->hidden * 2 * a->n_streams};
    const uint32_t xb[5] = {kKBlock, kTokTile, 1, 1, 1};
    rc = make_tensor_map(e, &mx, x16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != VOX_ATTN_OK) return rc;
    const uint64_t wd[5] = {(uint64_t) a->hidden, (uint64_t) n_out, 1, 1, 1};
    const uint64_t ws[4] = {(uint64_t) a->w_nb_row, (uint64_t) a->w_nb_row * n_out, (uint64_t) a->w_nb_row * n_out, (uint64_t) a->w_nb_row * n_out};
    const uint32_t wb[5] = {kKBlock, kHeadDim, 1, 1, 1};
    rc = make_tensor_map(e, &mw, const_cast<void *>(a->w_qkv), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != VOX_ATTN_OK) return rc;

    QkvParams p;
    p.n_streams = a->n_streams; p.k_dim = a->hidden; p.n_heads = a->n_heads; p.n_kv_heads = a->n_kv_heads;
    p.rope = reinterpret_cast<const float2 *>(a->rope_table);
    p.q = a->q; p.k_new = a->k_new; p.v_new = a->v_new;
    p.k_rows = p.v_rows = p.k_scales = p.v_scales = nullptr;
    p.nb_pos = p.nb_head = p.nb_stream = p.sb_pos = p.sb_head = p.sb_stream = 0;
    p.positions = a->positions; p.pos_offset = a->pos_offset; p.max_len = 0; p.cache_type = VOX_TYPE_F16;
    p.status = e->status_dev;
    if (to_cache) {
        const vox_kv_cache * c = a->cache;
        p.k_rows = c->k_data + (size_t) a->layer * c->nb_layer;
        p.v_rows = c->v_data + (size_t) a->layer * c->nb_layer;
        p.nb_pos = c->nb_pos; p.nb_head = c->nb_head; p.nb_stream = c->nb_stream;
        p.max_len = c->cfg.max_len; p.cache_type = c->cfg.type;
        if (c->cfg.type == VOX_TYPE_Q8_0) {
            p.k_scales = c->k_scale + (size_t) a->layer * c->sb_layer;
            p.v_scales = c->v_scale + (size_t) a->layer * c->sb_layer;
            p.sb_pos = c->sb_pos; p.sb_head = c->sb_head; p.sb_stream = c->sb_stream;
        }
    }
    const dim3 grid((unsigned) (a->n_heads + 2 * a->n_kv_heads), (unsigned) ((a->n_streams + kTokTile - 1) / kTokTile));
    launch_pdl(qkv_project_kernel, grid, dim3(kThreadsQkv), kSmemQkv, st, mx, mw, p);
    return check_launch(e, "qkv_project_kernel");
}

}  // extern "C"
