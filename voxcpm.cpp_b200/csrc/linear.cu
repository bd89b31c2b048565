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
static_assert(kLinRing * kLinStage >= 3 * kLinTok * kLinCols * 4 && kLinRing * kLinStage >= kLinTok * (kLinCols + 4) * 4,
              "the idle ring holds what a CTA sends, what it receives and what it writes out");

// Developer build (-DVOX_ATTN_DEVELOPER): the time (globaltimer, ns) at which thread 128 of a CTA passes a few points.
#ifdef VOX_ATTN_DEVELOPER
constexpr int kLinTraceCtas = 1024, kLinTracePoints = 8;
__device__ unsigned long long g_linear_trace[kLinTraceCtas][kLinTracePoints];
__device__ __forceinline__ unsigned long long lin_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define LIN_TRACE(point)                                                                                                      \
    do {                                                                                                                      \
        const int cta__ = (int) (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));                             \
        if (threadIdx.x == 128 && cta__ < kLinTraceCtas) g_linear_trace[cta__][point] = lin_ns();                            \
    } while (0)
#else
#define LIN_TRACE(point)
#endif

struct LinearParams {
    int           n_tokens, k_dim, n_out;  // n_out: output features (SwiGLU: of the product gate * up)
    int           mode;                    // vox_linear_mode
    float         scale;
    const float * residual;
    size_t        res_nb_token;
    uint8_t *     out;
    size_t        out_nb_token;
    int           out_f16;
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
    const bool    vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;  // k_dim is a multiple of 64
    float         scale = 1.0f;
    if (norm_w != nullptr) {
        float s = 0.0f;
        if (vec) {
            for (int i = tid; i < k_dim / 4; i += 256) {
                const float4 v = reinterpret_cast<const float4 *>(row)[i];
                s += v.x * v.x; s += v.y * v.y; s += v.z * v.z; s += v.w * v.w;
            }
        } else {
            for (int i = tid; i < k_dim; i += 256) s += row[i] * row[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if ((tid & 31) == 0) part[tid >> 5] = s;
        __syncthreads();
        float total = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) total += part[i];
        scale = 1.0f / sqrtf(total / (float) k_dim + eps);
    }
    __half * orow = out + (size_t) token * k_dim;
    if (vec) {
        for (int i = tid; i < k_dim / 4; i += 256) {
            float4 v = reinterpret_cast<const float4 *>(row)[i];
            if (norm_w != nullptr) {
                const float4 w = reinterpret_cast<const float4 *>(norm_w)[i];
                v.x = __fmul_rn(__fmul_rn(v.x, scale), w.x); v.y = __fmul_rn(__fmul_rn(v.y, scale), w.y);
                v.z = __fmul_rn(__fmul_rn(v.z, scale), w.z); v.w = __fmul_rn(__fmul_rn(v.w, scale), w.w);
            }
            *reinterpret_cast<uint2 *>(orow + 4 * i) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
        }
    } else {
        for (int i = tid; i < k_dim; i += 256) {
            float v = row[i];
            if (norm_w != nullptr) v = __fmul_rn(__fmul_rn(v, scale), norm_w[i]);
            orow[i] = __float2half_rn(v);
        }
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
    __shared__ uint64_t bars[2 * kLinRing + 2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int      abort_flag;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *      smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const int      tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int      tile = blockIdx.x, tok0 = blockIdx.y * kLinTok;
    const int      rank = S > 1 ? (int) cluster_rank() : 0;
    LIN_TRACE(0);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = full0 + 8 * kLinRing, done = empty0 + 8 * kLinRing, xbar = done + 8;
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kLinRing; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(done, 1);
        mbar_init(xbar, 1);
        fence_mbar_init();
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), kLinCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    LIN_TRACE(1);
    // The next kernel of the stream may be scheduled from here on; it still waits, in its own dependency wait, for this
    // grid to complete, and every thread of this grid passes its own wait before it touches what the kernel before wrote.
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
            // The weights do not come from the kernel before: the first ring of them is asked for ahead of the dependency
            // wait, so their way from HBM is covered by that kernel's last microseconds.
            const int n_early = min(n_kb, kLinRing);
            for (int i = 0; i < n_early; ++i) {
                const uint32_t sa = smem_base + i * kLinStage;
                const int      kx = (kb0 + i) * kLinKBlock;
                mbar_expect_tx(full0 + 8 * i, kLinStage);
                tma_load_5d(sa + kLinABytes, &map_w, full0 + 8 * i, kx, row_a, 0, 0, 0);
                tma_load_5d(sa + kLinABytes + kLinBBytes / 2, &map_w, full0 + 8 * i, kx, row_b, 0, 0, 0);
            }
            pdl_wait();  // the f16 copy of the activations comes from the kernel before
            for (int i = 0; i < n_kb && !aborted(); ++i) {
                const int st = i % kLinRing;
                if (i >= kLinRing && !mbar_wait_bounded(empty0 + 8 * st, ((i / kLinRing) - 1) & 1)) { give_up(); break; }
                const uint32_t sa = smem_base + st * kLinStage;
                const int      kx = (kb0 + i) * kLinKBlock;
                if (i >= n_early) {
                    mbar_expect_tx(full0 + 8 * st, kLinStage);
                    tma_load_5d(sa + kLinABytes, &map_w, full0 + 8 * st, kx, row_a, 0, 0, 0);
                    tma_load_5d(sa + kLinABytes + kLinBBytes / 2, &map_w, full0 + 8 * st, kx, row_b, 0, 0, 0);
                }
                tma_load_5d(sa, &map_x, full0 + 8 * st, kx, tok0, 0, 0, 0);
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
    if (!(warp == 0 && lane == 0)) pdl_wait();  // the residual may come from the kernel before as well
    LIN_TRACE(2);
    const bool epi = warp >= 4;
    const int  row = tid - 128, token = tok0 + row;
    uint32_t   r[kLinCols];
    bool       have = false;
    if (epi) {
        if (mbar_wait_bounded(done, 0)) {
            tc_fence_after();
            LIN_TRACE(3);
            tmem_ld64_sync(tmem + ((uint32_t) (32 * (warp & 3)) << 16), r);
            have = true;
        } else {
            give_up();
        }
    }
    // columns this CTA finishes: h of the first 32 and the h that go with them of the second 32
    constexpr int      h = 32 / S;
    constexpr uint32_t kSendOff = 0, kRecvOff = 32 * 1024, kOutOff = S == 1 ? 0 : 64 * 1024;  // areas of the (idle) ring
    constexpr int      kOutStride = 2 * h + 4;  // floats per staged row: four more than it holds, against bank conflicts
    float              a[h], b[h];  // sums of columns rank * h + i and 32 + rank * h + i
    if constexpr (S == 1) {
        if (epi && have) {
#pragma unroll
            for (int i = 0; i < 32; ++i) { a[i] = __uint_as_float(r[i]); b[i] = __uint_as_float(r[32 + i]); }
        }
    } else {
        // The CTAs of the cluster exchange accumulators: every CTA lays its 64 columns out by destination
        // ([destination rank][token][2h columns] f32, 4 KB per destination at S = 8) and sends each destination its part
        // with one bulk copy through distributed shared memory, which counts the bytes on the receiver's barrier.
        // (Storing the pieces one by one with st.shared::cluster took 5 us per launch.)
        // Every CTA of the cluster is past its MMAs once its epilogue threads have passed the cluster barrier: the rings
        // are idle from there on and take the copies.
        if (tid == 128) mbar_expect_tx(xbar, kLinTok * kLinCols * 4);  // what the S senders (this CTA among them) will deliver
        __syncwarp();
        cluster_sync_all();
        LIN_TRACE(4);
        if (epi && have) {
#pragma unroll
            for (int d = 0; d < S; ++d) {
                float4 * dst = reinterpret_cast<float4 *>(smem_gen + kSendOff) + ((size_t) (d * kLinTok + row) * 2 * h) / 4;
#pragma unroll
                for (int j = 0; j < h / 4; ++j) {
                    dst[j] = make_float4(__uint_as_float(r[d * h + 4 * j]), __uint_as_float(r[d * h + 4 * j + 1]),
                                         __uint_as_float(r[d * h + 4 * j + 2]), __uint_as_float(r[d * h + 4 * j + 3]));
                    dst[h / 4 + j] = make_float4(__uint_as_float(r[32 + d * h + 4 * j]), __uint_as_float(r[32 + d * h + 4 * j + 1]),
                                                 __uint_as_float(r[32 + d * h + 4 * j + 2]), __uint_as_float(r[32 + d * h + 4 * j + 3]));
                }
            }
        }
        if (epi) {
            fence_proxy_async_smem();  // the rows above are read by the bulk copies
            named_bar_sync(1, 128);
            if (tid == 128 && !aborted()) {
                constexpr uint32_t part = kLinTok * 2 * h * 4;  // bytes per destination
#pragma unroll
                for (int d = 0; d < S; ++d)
                    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     map_to_rank(smem_base + kRecvOff + (uint32_t) rank * part, (uint32_t) d)),
                                 "r"(smem_base + kSendOff + (uint32_t) d * part), "r"(part), "r"(map_to_rank(xbar, (uint32_t) d))
                                 : "memory");
            }
            const bool arrived = mbar_wait_bounded(xbar, 0);
            LIN_TRACE(5);
            if (!arrived) give_up();
#pragma unroll
            for (int i = 0; i < h; ++i) a[i] = b[i] = 0.0f;
            if (arrived) {
#pragma unroll
                for (int s2 = 0; s2 < S; ++s2) {  // in rank order: the sum does not depend on which CTA was first
                    const float4 * src = reinterpret_cast<const float4 *>(smem_gen + kRecvOff) + ((size_t) (s2 * kLinTok + row) * 2 * h) / 4;
#pragma unroll
                    for (int j = 0; j < h / 4; ++j) {
                        const float4 va = src[j], vb = src[h / 4 + j];
                        a[4 * j] += va.x; a[4 * j + 1] += va.y; a[4 * j + 2] += va.z; a[4 * j + 3] += va.w;
                        b[4 * j] += vb.x; b[4 * j + 1] += vb.y; b[4 * j + 2] += vb.z; b[4 * j + 3] += vb.w;
                    }
                }
            }
        }
    }
    // The results leave through shared memory, so that neighbouring threads write neighbouring pieces of a token's row
    // (a thread storing its own row float by float, rows 4 to 32 KB apart, took 15 us for 8 MB of output).
    if (epi) {
        const bool swiglu = p.mode == VOX_LINEAR_SWIGLU;
        float *    stage  = reinterpret_cast<float *>(smem_gen + kOutOff) + (size_t) row * kOutStride;
        if (swiglu) {
#pragma unroll
            for (int i = 0; i < h; ++i) stage[i] = a[i] / (1.0f + expf(-a[i])) * b[i];  // ggml_swiglu_split: silu(gate) * up
        } else {
#pragma unroll
            for (int i = 0; i < h; ++i) { stage[i] = a[i]; stage[h + i] = b[i]; }
        }
        named_bar_sync(1, 128);
        if (have && !aborted()) {
            const int per_row = swiglu ? h / 4 : 2 * h / 4;  // 16-byte pieces of a row that this CTA writes
            const int c0      = swiglu ? tile * 32 + rank * h : tile * kLinCols + rank * h;
            for (int pc = row; pc < kLinTok * per_row; pc += 128) {
                const int rr = pc / per_row, q = pc - rr * per_row;
                if (tok0 + rr >= p.n_tokens) break;  // rows only grow along the loop
                const int col = c0 + (q < h / 4 ? 4 * q : 32 + 4 * (q - h / 4));
                float4    v   = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(smem_gen + kOutOff) + (size_t) rr * kOutStride + 4 * q);
                uint8_t * orow = p.out + (size_t) (tok0 + rr) * p.out_nb_token;
                if (p.mode == VOX_LINEAR_RESIDUAL) {  // hidden = residual + scale * product (ggml_scale, then ggml_add)
                    const float * res = reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(p.residual) + (size_t) (tok0 + rr) * p.res_nb_token) + col;
                    v.x = __fadd_rn(res[0], __fmul_rn(v.x, p.scale));
                    v.y = __fadd_rn(res[1], __fmul_rn(v.y, p.scale));
                    v.z = __fadd_rn(res[2], __fmul_rn(v.z, p.scale));
                    v.w = __fadd_rn(res[3], __fmul_rn(v.w, p.scale));
                }
                if (p.out_f16) {
                    *reinterpret_cast<uint2 *>(orow + (size_t) col * 2) = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
                } else {
                    float * o = reinterpret_cast<float *>(orow) + col;
                    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
                }
            }
        }
    }
    if constexpr (S > 1) {
        // no CTA leaves while a copy it sent, or one sent to it, may still be on its way
        __syncwarp();
        cluster_sync_all();
    }
    LIN_TRACE(6);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, kLinCols);
    }
    LIN_TRACE(7);
}

// CTAs along K.  A matrix with few tiles (o_proj, down_proj: 32 tiles for 256 tokens) is split as far as every CTA keeps
// four K blocks or more and the grid stays within two CTAs per SM: a CTA's fixed costs (set-up, the exchange and the
// barriers of the cluster) are about 6 us (measured on 256 tokens x 1024 -> 1024: 13.3 / 10.6 / 12.4 us per launch pair
// with 2 / 4 / 8 CTAs along K; x 4096 -> 1024: 21.0 / 15.4 / 13.8 us).  A matrix with a tile for every other SM or more
// (gate_up: 128 and more) is not split: its CTAs fill the GPU as they are, and clusters only add their costs (32
// tokens, 1024 -> 2 x 4096: 16.6 / 20.1 / 25.5 us with 1 / 2 / 4 CTAs along K).
int pick_split(int k_dim, int tiles, int sms) {
    if (tiles * 2 > sms) return 1;
    int s = 1;
    while (s < kLinMaxSplit && (k_dim / kLinKBlock) % (2 * s) == 0 && k_dim / kLinKBlock / (2 * s) >= 4 && tiles * 2 * s <= 2 * sms) s *= 2;
    return s;
}

}  // namespace

#ifdef VOX_ATTN_DEVELOPER
// out: kLinTraceCtas x kLinTracePoints times in ns of the last launch (0 entry, 1 set-up done, 2 past the dependency wait,
// 3 accumulator complete, 4 / 5 past the first / second cluster barrier, 6 results stored, 7 tensor memory released)
extern "C" int vox_debug_linear_trace(unsigned long long * out) {
    return cudaMemcpyFromSymbol(out, g_linear_trace, sizeof(unsigned long long) * kLinTraceCtas * kLinTracePoints) == cudaSuccess ? 0 : 4;
}
#endif

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
    const bool x16 = a->x_type == VOX_TYPE_F16, out16 = a->out_type == VOX_TYPE_F16;
    VOX_REQUIRE((a->x_type == VOX_TYPE_F32 || x16) && (a->out_type == VOX_TYPE_F32 || out16), VOX_ATTN_UNSUPPORTED,
                "x and out are f32 or f16 (types %d, %d)", a->x_type, a->out_type);
    if (x16) {
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->x) & 15) == 0 && a->x_nb_token % 16 == 0 && a->x_nb_token >= (size_t) a->k_dim * 2,
                    VOX_ATTN_INVALID_ARGUMENT, "f16 x rows must be 16-byte aligned and at least k_dim halves apart");
        VOX_REQUIRE(a->norm_weight == nullptr, VOX_ATTN_UNSUPPORTED, "the norm needs f32 x");
    } else {
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->x) & 3) == 0 && a->x_nb_token % 4 == 0 && a->x_nb_token >= (size_t) a->k_dim * 4,
                    VOX_ATTN_INVALID_ARGUMENT, "x rows must be 4-byte aligned and at least k_dim floats apart");
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->norm_weight) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT, "norm_weight must be 16-byte aligned");
    }
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->w) & 15) == 0 && a->w_nb_row % 16 == 0 && a->w_nb_row >= (size_t) a->k_dim * 2,
                VOX_ATTN_INVALID_ARGUMENT, "weight rows must be 16-byte aligned and at least k_dim halves apart");
    const size_t out_elem = out16 ? 2 : 4;
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->out) & (out16 ? 7 : 3)) == 0 && a->out_nb_token % (out16 ? 8 : 4) == 0 &&
                    a->out_nb_token >= (size_t) a->n_out * out_elem,
                VOX_ATTN_INVALID_ARGUMENT, "out rows must be aligned (4 bytes for f32, 8 for f16) and at least n_out values apart");
    if (a->mode == VOX_LINEAR_RESIDUAL) {
        VOX_REQUIRE(!out16, VOX_ATTN_UNSUPPORTED, "the residual mode writes f32");
        VOX_REQUIRE(a->residual != nullptr && a->res_nb_token % 4 == 0 && a->res_nb_token >= (size_t) a->n_out * 4, VOX_ATTN_INVALID_ARGUMENT,
                    "the residual mode needs residual rows at least n_out floats apart");
    }
    const size_t need = x16 ? 0 : vox_linear_workspace_bytes(a->n_tokens, a->k_dim);
    VOX_REQUIRE(x16 || (workspace != nullptr && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0),
                VOX_ATTN_WORKSPACE_TOO_SMALL, "vox_linear needs %zu workspace bytes (16-byte aligned), got %zu", need, workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!(e->attr_mask & (1u << 15))) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        VOX_CUDA_TRY(cudaFuncSetAttribute(linear_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLinSmem));
        e->attr_mask |= 1u << 15;
    }
    int rc = VOX_ATTN_OK;
    const void * xh = a->x;                      // f16 rows the product reads
    uint64_t     xh_stride = a->x_nb_token;
    if (!x16) {
        xh = workspace;
        xh_stride = (uint64_t) a->k_dim * 2;
        launch_pdl(linear_prepare_kernel, dim3((unsigned) a->n_tokens), dim3(256), 0, st, reinterpret_cast<const uint8_t *>(a->x), a->x_nb_token,
                   a->k_dim, a->norm_weight, a->norm_eps, static_cast<__half *>(workspace));
        rc = check_launch(e, "linear_prepare_kernel");
        if (rc != VOX_ATTN_OK) return rc;
    }

    const int      w_rows = a->mode == VOX_LINEAR_SWIGLU ? 2 * a->n_out : a->n_out;
    CUtensorMap    mx, mw;
    const uint64_t xd[5] = {(uint64_t) a->k_dim, (uint64_t) a->n_tokens, 1, 1, 1};
    const uint64_t xs[4] = {xh_stride, xh_stride * a->n_tokens, xh_stride * a->n_tokens, xh_stride * a->n_tokens};
    const uint32_t xb[5] = {kLinKBlock, kLinTok, 1, 1, 1};
    rc = make_tensor_map(e, &mx, const_cast<void *>(xh), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B);
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
    p.out = static_cast<uint8_t *>(a->out); p.out_nb_token = a->out_nb_token; p.out_f16 = out16 ? 1 : 0;
    p.status = e->status_dev;
    const int col_tiles = a->n_out / tile_out, tok_tiles = (a->n_tokens + kLinTok - 1) / kLinTok;
    int split = pick_split(a->k_dim, col_tiles * tok_tiles, e->sm_count);
    if (e->linear_split > 0 && (a->k_dim / kLinKBlock) % e->linear_split == 0 &&
        (e->linear_split == 1 || e->linear_split == 2 || e->linear_split == 4 || e->linear_split == 8))
        split = e->linear_split;

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
