// Batched linear layers of a decode step: the output projection of attention and the SwiGLU MLP, for all streams of
// a group at once.
//
// Replaces, for the single-token step of every stream, ggml_mul_mat(o_proj, attn) (src/minicpm.cpp:715) with the
// residual add of layer_forward (:765-768), and mlp_forward (:718-747): ggml_mul_mat(gate_up_proj, hidden),
// ggml_swiglu_split(gate, up), ggml_mul_mat(down_proj, fused), with the residual add (:773-776); optionally the RMS
// norm in front (rms_norm, :572-580) as part of the conversion of the activations.  The reference runs these once per
// stream, so every weight matrix (30 MB of f16 per layer of the 1024 / 4096 model) is read once per stream and step;
// here one launch per matrix serves all streams and the weights are read once.
//
// Arithmetic as the reference's CPU backend does it for f16 weights (ggml_compute_forward_mul_mat with vec_dot_type
// F16, third_party/ggml/src/ggml-cpu/ggml-cpu.c:217; ggml_vec_dot_f16, ggml-cpu/vec.cpp:264): activations rounded to
// f16, exact products, f32 accumulation; silu(g) * u as ggml_swiglu_split computes it (g / (1 + exp(-g)) * u in f32);
// the RMS norm as ggml_compute_forward_rms_norm_f32 (ggml-cpu/ops.cpp:3725-3755) followed by ggml_mul with the weight.
//
// Kernel: D[tokens, features] = X[tokens, K] . W[features, K]^T on tcgen05, a CTA on 128 tokens x 64 accumulator
// columns (64 features; for SwiGLU 32 gate features and the 32 up features that go with them), operands K-major by
// bulk-tensor copies in 64-wide K blocks into a four-stage ring, one thread issuing tcgen05.mma (kind::f16, M = 128,
// N = 64).  With 256 tokens there are few such tiles (32 for a 1024 x 1024 matrix) and a CTA fills its shared memory at
// no more than about 45 KB/us, so the K range is split over a thread-block cluster of up to eight CTAs: each
// accumulates its share of K in tensor memory, then the CTAs exchange accumulators through distributed shared memory,
// each ending up with all partial sums of its own eighth of the columns (CTA r gets columns 4r .. 4r+3 and
// 32+4r .. 32+4r+3, so that a gate feature and its up feature meet in one thread), adds them in rank order (the result
// does not depend on timing) and finishes those columns: scale and residual, or silu(gate) * up.
#include "tcgen05.cuh"

#include <algorithm>

using namespace vox;

namespace {

constexpr int kLinTok    = 128;                 // tokens per CTA (TMEM lanes)
constexpr int kLinCols   = 64;                  // accumulator columns per CTA
constexpr int kLinKBlock = 64;                  // K elements per stage: 128-byte rows
constexpr int kLinRing   = 4;
constexpr int kLinABytes = kLinTok * 128;       // [128 tokens][64 k] f16
constexpr int kLinBBytes = kLinCols * 128;      // [64 rows][64 k] f16
constexpr int kLinStage  = kLinABytes + kLinBBytes;
constexpr int kLinSmem   = kLinRing * kLinStage + 1024;
constexpr int kLinThreads = 256;                // producer, issuer, two idle warps, four epilogue warps
constexpr int kLinMaxSplit = 8;
static_assert(kLinRing * kLinStage >= kLinTok * kLinCols * 4, "the ring must hold the accumulators the cluster exchanges");

struct LinearParams {
    int           n_tokens, k_dim, n_out;  // n_out: output features (SwiGLU: of the product gate * up)
    int           mode;                    // vox_linear_mode
    float         scale;
    const float * residual;
    size_t        res_nb_token;
    float *       out;
    size_t        out_nb_token;
    int *         status;
};

// Activations -> f16 rows [token][K], with the RMS norm of the row in front when a weight is given: one block per
// token.  y = x * (1 / sqrt(mean(x^2) + eps)), then y * w, each rounded to f32 as the reference's two nodes round them.
__global__ void __launch_bounds__(256) linear_prepare_kernel(const uint8_t * x, size_t nb_token, int k_dim, const float * norm_w, float eps,
                                                             __half * out) {
    __shared__ float part[8];
    pdl_wait();
    pdl_launch_dependents();
    const int     token = blockIdx.x, tid = threadIdx.x;
    const float * row = reinterpret_cast<const float *>(x + (size_t) token * nb_token);
    float         scale = 1.0f;
    if (norm_w != nullptr) {
        float s = 0.0f;
        for (int i = tid; i < k_dim; i += 256) s += row[i] * row[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if ((tid & 31) == 0) part[tid >> 5] = s;
        __syncthreads();
        float total = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) total += part[i];
        scale = 1.0f / sqrtf(total / (float) k_dim + eps);
    }
    for (int i = tid; i < k_dim; i += 256) {
        float v = row[i];
        if (norm_w != nullptr) v = __fmul_rn(__fmul_rn(v, scale), norm_w[i]);
        out[(size_t) token * k_dim + i] = __float2half_rn(v);
    }
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of `addr` of this CTA's shared memory in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// grid: x = column tiles, y = token tiles, z = S CTAs along K (one cluster)
template <int S>
__global__ void __launch_bounds__(kLinThreads, 2)
linear_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const LinearParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * kLinRing + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int      abort_flag;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *      smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const int      tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int      tile = blockIdx.x, tok0 = blockIdx.y * kLinTok;
    const int      rank = S > 1 ? (int) cluster_rank() : 0;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = full0 + 8 * kLinRing, done = empty0 + 8 * kLinRing;
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kLinRing; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(done, 1);
        fence_mbar_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), kLinCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();  // the f16 copy of the activations comes from the kernel before
    pdl_launch_dependents();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&tmem_base_slot);
    const int      n_kb = p.k_dim / kLinKBlock / S, kb0 = rank * n_kb;  // this CTA's share of the K blocks
    auto give_up = [&]() {
        atomicOr(p.status, kStatusTimeout);
        atomicExch(&abort_flag, 1);
    };
    auto aborted = [&]() { return *reinterpret_cast<volatile int *>(&abort_flag) != 0; };
    // weight rows behind the accumulator columns: 0-31 and 32-63 are two runs of 32 rows (SwiGLU: gate rows, up rows)
    const int row_a = p.mode == VOX_LINEAR_SWIGLU ? tile * 32 : tile * kLinCols;
    const int row_b = p.mode == VOX_LINEAR_SWIGLU ? p.n_out + tile * 32 : tile * kLinCols + 32;

    if (warp == 0) {
        if (lane == 0) {  // producer
            for (int i = 0; i < n_kb && !aborted(); ++i) {
                const int st = i % kLinRing;
                if (i >= kLinRing && !mbar_wait_bounded(empty0 + 8 * st, ((i / kLinRing) - 1) & 1)) { give_up(); break; }
                const uint32_t sa = smem_base + st * kLinStage;
                const int      kx = (kb0 + i) * kLinKBlock;
                mbar_expect_tx(full0 + 8 * st, kLinStage);
                tma_load_5d(sa, &map_x, full0 + 8 * st, kx, tok0, 0, 0, 0);
                tma_load_5d(sa + kLinABytes, &map_w, full0 + 8 * st, kx, row_a, 0, 0, 0);
                tma_load_5d(sa + kLinABytes + kLinBBytes / 2, &map_w, full0 + 8 * st, kx, row_b, 0, 0, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // issuer
            constexpr uint32_t idesc = idesc_f16(kLinCols, false);
            const uint64_t     dA = smem_desc_sw128(smem_base), dB = smem_desc_sw128(smem_base + kLinABytes);
            bool ok = true;
            for (int i = 0; i < n_kb && !aborted(); ++i) {
                const int st = i % kLinRing;
                if (!mbar_wait_bounded(full0 + 8 * st, (i / kLinRing) & 1)) { give_up(); ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < kLinKBlock / 16; ++k)
                    tc_mma_f16(tmem, dA + (uint64_t) st * (kLinStage >> 4) + k * 2, dB + (uint64_t) st * (kLinStage >> 4) + k * 2, idesc,
                               (i | k) != 0);
                tc_commit(empty0 + 8 * st);  // the stage may be refilled once these have retired
            }
            if (ok) tc_commit(done);
        }
    }

    // ---- epilogue: one thread per token holds the 64 accumulator columns of its row
    const bool epi = warp >= 4;
    const int  row = tid - 128, token = tok0 + row;
    uint32_t   r[kLinCols];
    bool       have = false;
    if (epi) {
        if (mbar_wait_bounded(done, 0)) {
            tc_fence_after();
            tmem_ld64_sync(tmem + ((uint32_t) (32 * (warp & 3)) << 16), r);
            have = true;
        } else {
            give_up();
        }
    }
    // columns this CTA finishes: h of the first 32 and the h that go with them of the second 32
    constexpr int h = 32 / S;
    float         a[h], b[h];  // sums of columns rank * h + i and 32 + rank * h + i
    if constexpr (S == 1) {
        if (epi && have) {
#pragma unroll
            for (int i = 0; i < 32; ++i) { a[i] = __uint_as_float(r[i]); b[i] = __uint_as_float(r[32 + i]); }
        }
    } else {
        // Every CTA of the cluster is past its MMAs once its epilogue threads are here: the rings are idle and take the
        // accumulators, [source rank][token][2h columns] f32 (32 KB whatever the split).
        __syncwarp();
        cluster_sync_all();
        if (epi && have) {
            const uint32_t mine = smem_base + ((uint32_t) (rank * kLinTok + row) * 2 * h) * 4;
#pragma unroll
            for (int d = 0; d < S; ++d) {
                const uint32_t dst = map_to_rank(mine, (uint32_t) d);
#pragma unroll
                for (int j = 0; j < h; j += 4) {
                    st_cluster_f4(dst + 4 * j, __uint_as_float(r[d * h + j]), __uint_as_float(r[d * h + j + 1]),
                                  __uint_as_float(r[d * h + j + 2]), __uint_as_float(r[d * h + j + 3]));
                    st_cluster_f4(dst + 4 * (h + j), __uint_as_float(r[32 + d * h + j]), __uint_as_float(r[32 + d * h + j + 1]),
                                  __uint_as_float(r[32 + d * h + j + 2]), __uint_as_float(r[32 + d * h + j + 3]));
                }
            }
        }
        __syncwarp();
        cluster_sync_all();
        if (epi) {
#pragma unroll
            for (int i = 0; i < h; ++i) a[i] = b[i] = 0.0f;
#pragma unroll
            for (int s = 0; s < S; ++s) {  // in rank order: the sum does not depend on which CTA was first
                const float4 * src = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(smem_gen) + (size_t) (s * kLinTok + row) * 2 * h);
#pragma unroll
                for (int j = 0; j < h / 4; ++j) {
                    const float4 va = src[j], vb = src[h / 4 + j];
                    a[4 * j] += va.x; a[4 * j + 1] += va.y; a[4 * j + 2] += va.z; a[4 * j + 3] += va.w;
                    b[4 * j] += vb.x; b[4 * j + 1] += vb.y; b[4 * j + 2] += vb.z; b[4 * j + 3] += vb.w;
                }
            }
        }
    }
    if (epi && have && token < p.n_tokens && !aborted()) {
        float *       out = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(p.out) + (size_t) token * p.out_nb_token);
        const float * res = p.residual ? reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(p.residual) + (size_t) token * p.res_nb_token) : nullptr;
        if (p.mode == VOX_LINEAR_SWIGLU) {
            const int c0 = tile * 32 + rank * h;
#pragma unroll
            for (int i = 0; i < h; ++i) {
                const float g = a[i];
                out[c0 + i]   = g / (1.0f + expf(-g)) * b[i];  // ggml_swiglu_split: silu(gate) * up
            }
        } else {
            const int c0 = tile * kLinCols + rank * h;
#pragma unroll
            for (int i = 0; i < h; ++i) {
                float va = a[i], vb = b[i];
                if (p.mode == VOX_LINEAR_RESIDUAL) {  // hidden = residual + scale * product (ggml_scale, then ggml_add)
                    va = __fadd_rn(res[c0 + i], __fmul_rn(va, p.scale));
                    vb = __fadd_rn(res[c0 + 32 + i], __fmul_rn(vb, p.scale));
                }
                out[c0 + i]      = va;
                out[c0 + 32 + i] = vb;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kLinCols);
    }
}

// CTAs along K: as many as keep every CTA at two K blocks or more, without going far past two CTAs per SM in all
int pick_split(int k_dim, int tiles, int sms) {
    int s = 1;
    while (s < kLinMaxSplit && (k_dim / kLinKBlock) % (2 * s) == 0 && k_dim / kLinKBlock / (2 * s) >= 2 && tiles * 2 * s <= 2 * sms + sms / 2) s *= 2;
    return s;
}

}  // namespace

extern "C" {

size_t vox_linear_workspace_bytes(int n_tokens, int k_dim) {
    if (n_tokens <= 0 || k_dim <= 0) return 0;
    return ((size_t) n_tokens * k_dim * sizeof(__half) + 255) & ~(size_t) 255;
}

int vox_linear(vox_engine * e, const vox_linear_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    VOX_REQUIRE(e && a && a->x && a->w && a->out, VOX_ATTN_INVALID_ARGUMENT, "vox_linear: null argument");
    VOX_REQUIRE(a->mode == VOX_LINEAR_PLAIN || a->mode == VOX_LINEAR_RESIDUAL || a->mode == VOX_LINEAR_SWIGLU, VOX_ATTN_INVALID_ARGUMENT,
                "vox_linear: unknown mode %d", a->mode);
    VOX_REQUIRE(a->w_type == VOX_TYPE_F16, VOX_ATTN_UNSUPPORTED, "weights of type %d are not supported (f16 only)", a->w_type);
    VOX_REQUIRE(a->n_tokens > 0, VOX_ATTN_INVALID_ARGUMENT, "n_tokens must be positive");
    VOX_REQUIRE(a->k_dim > 0 && a->k_dim % kLinKBlock == 0, VOX_ATTN_UNSUPPORTED, "input size %d is not a multiple of 64", a->k_dim);
    const int tile_out = a->mode == VOX_LINEAR_SWIGLU ? 32 : kLinCols;
    VOX_REQUIRE(a->n_out > 0 && a->n_out % tile_out == 0, VOX_ATTN_UNSUPPORTED, "output size %d is not a multiple of %d", a->n_out, tile_out);
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->x) & 3) == 0 && a->x_nb_token % 4 == 0 && a->x_nb_token >= (size_t) a->k_dim * 4,
                VOX_ATTN_INVALID_ARGUMENT, "x rows must be 4-byte aligned and at least k_dim floats apart");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->w) & 15) == 0 && a->w_nb_row % 16 == 0 && a->w_nb_row >= (size_t) a->k_dim * 2,
                VOX_ATTN_INVALID_ARGUMENT, "weight rows must be 16-byte aligned and at least k_dim halves apart");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->out) & 3) == 0 && a->out_nb_token % 4 == 0 && a->out_nb_token >= (size_t) a->n_out * 4,
                VOX_ATTN_INVALID_ARGUMENT, "out rows must be 4-byte aligned and at least n_out floats apart");
    if (a->mode == VOX_LINEAR_RESIDUAL)
        VOX_REQUIRE(a->residual != nullptr && a->res_nb_token % 4 == 0 && a->res_nb_token >= (size_t) a->n_out * 4, VOX_ATTN_INVALID_ARGUMENT,
                    "the residual mode needs residual rows at least n_out floats apart");
    const size_t need = vox_linear_workspace_bytes(a->n_tokens, a->k_dim);
    VOX_REQUIRE(workspace != nullptr && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                VOX_ATTN_WORKSPACE_TOO_SMALL, "vox_linear needs %zu workspace bytes (16-byte aligned), got %zu", need, workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!(e->attr_mask & (1u << 15))) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        e->attr_mask |= 1u << 15;
    }
    __half * x16 = static_cast<__half *>(workspace);
    launch_pdl(linear_prepare_kernel, dim3((unsigned) a->n_tokens), dim3(256), 0, st, reinterpret_cast<const uint8_t *>(a->x), a->x_nb_token,
               a->k_dim, a->norm_weight, a->norm_eps, x16);
    int rc = check_launch(e, "linear_prepare_kernel");
    if (rc != VOX_ATTN_OK) return rc;

    const int      w_rows = a->mode == VOX_LINEAR_SWIGLU ? 2 * a->n_out : a->n_out;
    CUtensorMap    mx, mw;
    const uint64_t xd[5] = {(uint64_t) a->k_dim, (uint64_t) a->n_tokens, 1, 1, 1};
    const uint64_t xs[4] = {(uint64_t) a->k_dim * 2, (uint64_t) a->k_dim * 2 * a->n_tokens, (uint64_t) a->k_dim * 2 * a->n_tokens,
                            (uint64_t) a->k_dim * 2 * a->n_tokens};
    const uint32_t xb[5] = {kLinKBlock, kLinTok, 1, 1, 1};
    rc = make_tensor_map(e, &mx, x16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != VOX_ATTN_OK) return rc;
    const uint64_t wd[5] = {(uint64_t) a->k_dim, (uint64_t) w_rows, 1, 1, 1};
    const uint64_t ws[4] = {(uint64_t) a->w_nb_row, (uint64_t) a->w_nb_row * w_rows, (uint64_t) a->w_nb_row * w_rows, (uint64_t) a->w_nb_row * w_rows};
    const uint32_t wb[5] = {kLinKBlock, 32, 1, 1, 1};
    rc = make_tensor_map(e, &mw, const_cast<void *>(a->w), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != VOX_ATTN_OK) return rc;

    LinearParams p;
    p.n_tokens = a->n_tokens; p.k_dim = a->k_dim; p.n_out = a->n_out; p.mode = a->mode;
    p.scale = a->mode == VOX_LINEAR_RESIDUAL ? a->scale : 1.0f;
    p.residual = a->residual; p.res_nb_token = a->res_nb_token;
    p.out = a->out; p.out_nb_token = a->out_nb_token;
    p.status = e->status_dev;
    const int col_tiles = a->n_out / tile_out, tok_tiles = (a->n_tokens + kLinTok - 1) / kLinTok;
    const int split = pick_split(a->k_dim, col_tiles * tok_tiles, e->sm_count);

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) col_tiles, (unsigned) tok_tiles, (unsigned) split);
    cfg.blockDim = dim3(kLinThreads);
    cfg.dynamicSmemBytes = kLinSmem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (split > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1; attr[n_attr].val.clusterDim.y = 1; attr[n_attr].val.clusterDim.z = (unsigned) split;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    switch (split) {
        case 1: cudaLaunchKernelEx(&cfg, linear_kernel<1>, mx, mw, p); break;
        case 2: cudaLaunchKernelEx(&cfg, linear_kernel<2>, mx, mw, p); break;
        case 4: cudaLaunchKernelEx(&cfg, linear_kernel<4>, mx, mw, p); break;
        default: cudaLaunchKernelEx(&cfg, linear_kernel<8>, mx, mw, p); break;
    }
    return check_launch(e, "linear_kernel");
}

}  // extern "C"
