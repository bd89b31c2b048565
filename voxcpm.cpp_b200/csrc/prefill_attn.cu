// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), K/V fed by TMA.
//
// Replaces the n_q == n_kv call that MiniCPMModel::forward makes with the f16 mask from
// create_causal_mask (src/minicpm.cpp:602-620, 779-802 -> :708-710); the mask is implied by a
// causal offset instead of being materialised and re-read (512 KB per 512-token graph there).
// On the CPU this is ggml's tiled path (third_party/ggml/src/ggml-cpu/ops.cpp:8347-8633); ggml-cuda
// would run the mma.sync kernel flash_attn_ext_f16 (fattn-mma-f16.cuh:1459-1628).
//
// One CTA = 128 query rows of one head.  Six warps:
//   warps 0-3  softmax: thread r owns query row r = TMEM lane r.  Per 128-key tile it reads the
//              scores S from TMEM (tcgen05.ld), takes the row maximum, writes P = 2^(c*(S - max)) as
//              f16 into shared memory in the 128-byte-swizzled K-major layout the tensor core reads,
//              then adds the tile's P.V (read back from TMEM) into its f32 output row in registers
//              with the usual running-max rescale.
//   warp 4     producer: one lane issues cp.async.bulk.tensor copies of 128-row K and V tiles into a
//              two-stage ring.
//   warp 5     MMA issuer: one lane issues tcgen05.mma (kind::f16, M=128): S = Q.K^T (N=128, 4 k-steps)
//              into TMEM columns 0-127 and O_tile = P.V (N=64, 8 k-steps, V read MN-major straight from
//              the row-major tile) into columns 128-191; completion is signalled with tcgen05.commit.
// Q arrives as f32 and is rounded to f16 once per CTA (exact when it already holds f16 values);
// scale*log2(e) is applied to S in f32.  Accumulation is f32 everywhere.
// Every wait is bounded; on expiry the status word is set and all roles fall through to the common
// exit, where the TMEM columns are released.
#include "common.cuh"

#include <algorithm>

using namespace vox;

namespace vox {
int launch_generic(vox_engine * e, const vox_attn_args * a, int causal_offset, cudaStream_t stream);
}

namespace {

constexpr int kTile      = 128;            // query rows per CTA and keys per tile
constexpr int kTileBytes = kTile * 128;    // one [128][64] f16 tile
constexpr int kKvStages  = 2;
constexpr int kThreadsPf = 6 * 32;
constexpr int kTmemCols  = 256;            // S: columns 0-127, O tile: 128-191
constexpr int kSmemPf    = kTileBytes * (1 + 2 * kKvStages + 2) + 1024;  // Q, K/V ring, P (two 64-key halves)

struct PrefillParams {
    const uint8_t * q;
    size_t          q_nb1, q_nb2, q_nb3;
    float *         dst;
    int             n_q, n_kv, n_heads, gqa, causal_offset;
    float           scale_log2;
    int *           status;
};

// ---- tcgen05 wrappers ---------------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 consecutive f32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor (64-bit) of a 128-byte-swizzled tile whose 8-row groups are 1024
// bytes apart: start address, leading/stride byte offsets (>> 4), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr & 0x3FFFFu) >> 4);        // bits [0,14)
    d |= (uint64_t) 1 << 16;                         // leading byte offset (unused with one swizzle atom per row group)
    d |= (uint64_t) (1024 >> 4) << 32;               // stride byte offset: next group of 8 rows
    d |= (uint64_t) 1 << 46;                         // descriptor version (sm_100)
    d |= (uint64_t) 2 << 61;                         // SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f16: f32 accumulate, f16 A and B, M = 128.
constexpr uint32_t idesc_f16(int n, bool b_mn_major) {
    return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (kTile >> 4) << 24);
}

__global__ void __launch_bounds__(kThreadsPf, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * kKvStages + 6];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int      abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *      smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sQ = smem_base, sKV = smem_base + kTileBytes, sP = sKV + 2 * kKvStages * kTileBytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // heavier (later) query tiles first so that the causal triangle drains evenly
    const int n_qtiles = (p.n_q + kTile - 1) / kTile;
    const int qtile = n_qtiles - 1 - blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
    const int kvh   = head / p.gqa;
    const int q0    = qtile * kTile;
    const int last_row = min(q0 + kTile, p.n_q) - 1;
    const int n_tiles  = min((p.n_kv + kTile - 1) / kTile, (last_row + p.causal_offset) / kTile + 1);

    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kKvStages]);
    const uint32_t bQ = smem_u32(&bars[2 * kKvStages]), bSready = bQ + 8, bSfree = bQ + 16, bPready = bQ + 24, bPVdone = bQ + 32,
                   bOfree = bQ + 40;
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(bQ, 128);
        mbar_init(bSready, 1);
        mbar_init(bSfree, 128);
        mbar_init(bPready, 128);
        mbar_init(bPVdone, 1);
        mbar_init(bOfree, 128);
        fence_mbar_init();
    }
    if (warp == 5) tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&tmem_base_slot);

    auto give_up = [&]() {
        atomicOr(p.status, kStatusTimeout);
        atomicExch(&abort_flag, 1);
    };
    auto aborted = [&]() { return *reinterpret_cast<volatile int *>(&abort_flag) != 0; };

    if (warp == 4) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            for (int j = 0; j < n_tiles && !aborted(); ++j) {
                const int s = j % kKvStages;
                if (j >= kKvStages && !mbar_wait_bounded(empty0 + 8 * s, ((j / kKvStages) - 1) & 1)) { give_up(); break; }
                const uint32_t dst = sKV + s * 2 * kTileBytes;
                mbar_expect_tx(full0 + 8 * s, 2 * kTileBytes);
                tma_load_5d(dst, &map_k, full0 + 8 * s, 0, j * kTile, kvh, batch, 0);
                tma_load_5d(dst + kTileBytes, &map_v, full0 + 8 * s, 0, j * kTile, kvh, batch, 0);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_f16(kTile, false), idesc_pv = idesc_f16(kHeadDim, true);
            bool ok = mbar_wait_bounded(bQ, 0);
            if (!ok) give_up();
            for (int j = 0; j < n_tiles && ok && !aborted(); ++j) {
                const int      s  = j % kKvStages;
                const uint32_t sK = sKV + s * 2 * kTileBytes, sV = sK + kTileBytes;
                if (!mbar_wait_bounded(full0 + 8 * s, (j / kKvStages) & 1)) { give_up(); break; }
                if (j > 0 && !mbar_wait_bounded(bSfree, (j - 1) & 1)) { give_up(); break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 4; ++k)  // S = Q K^T: four k-steps of 16 along head_dim, 32 bytes each inside the swizzle atom
                    tc_mma_f16(tmem, smem_desc_sw128(sQ + 32 * k), smem_desc_sw128(sK + 32 * k), idesc_qk, k > 0);
                tc_commit(bSready);
                if (!mbar_wait_bounded(bPready, j & 1)) { give_up(); break; }
                if (j > 0 && !mbar_wait_bounded(bOfree, (j - 1) & 1)) { give_up(); break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 8; ++k)  // O_tile = P V: eight k-steps of 16 keys; P half-tiles of 64 keys, V rows 16 at a time
                    tc_mma_f16(tmem + kTile, smem_desc_sw128(sP + (k >> 2) * kTileBytes + 32 * (k & 3)),
                               smem_desc_sw128(sV + 2048 * k), idesc_pv, k > 0);
                tc_commit(bPVdone);
                tc_commit(empty0 + 8 * s);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps: thread = query row
        const int  row   = tid;  // 0..127 == TMEM lane
        const int  qpos  = q0 + row;
        const bool live  = qpos < p.n_q;
        {
            // Q row -> f16, written as eight 16-byte chunks at their swizzled places
            uint8_t * dstrow = smem_gen + row * 128;
            const float * src = reinterpret_cast<const float *>(p.q + (size_t) qpos * p.q_nb1 + (size_t) head * p.q_nb2 +
                                                                (size_t) batch * p.q_nb3);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint4 w = make_uint4(0, 0, 0, 0);
                if (live) {
                    const float2 a = *reinterpret_cast<const float2 *>(src + 8 * c), b = *reinterpret_cast<const float2 *>(src + 8 * c + 2);
                    const float2 cc = *reinterpret_cast<const float2 *>(src + 8 * c + 4), d = *reinterpret_cast<const float2 *>(src + 8 * c + 6);
                    w = make_uint4(pack_half2(a.x, a.y), pack_half2(b.x, b.y), pack_half2(cc.x, cc.y), pack_half2(d.x, d.y));
                }
                *reinterpret_cast<uint4 *>(dstrow + ((c ^ (row & 7)) << 4)) = w;
            }
            fence_proxy_async_smem();
            mbar_arrive(bQ);
        }
        const uint32_t t_row = tmem + ((uint32_t) (warp * 32) << 16);  // this warp's lane quarter
        const int      limit = min(qpos + p.causal_offset, p.n_kv - 1);  // last key this row may see
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        bool  ok = true;
        for (int j = 0; j < n_tiles && ok && !aborted(); ++j) {
            if (!mbar_wait_bounded(bSready, j & 1)) { give_up(); break; }
            tc_fence_after();
            const int  k0     = j * kTile;
            const bool masked = k0 + kTile - 1 > min(q0 + p.causal_offset, p.n_kv - 1);  // CTA-uniform: any row of the tile may be cut
            float v[32];
            // pass 1: row maximum of this tile
            float tmax = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                tmem_ld32(t_row + 32 * c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float x = (masked && k0 + 32 * c + i > limit) ? -INFINITY : v[i];
                    tmax = fmaxf(tmax, x);
                }
            }
            const float m_new = fmaxf(m, tmax * p.scale_log2);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float alpha = m == -INFINITY ? 0.0f : exp2f(m - m_use);
            m = m_new;
            // pass 2: P = 2^(c*S - max), f16, into the two 64-key halves of the P tile
            float psum = 0.0f;
            uint8_t * prow = smem_gen + (sP - smem_base) + row * 128;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                tmem_ld32(t_row + 32 * c, v);
                uint32_t h[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float x0 = (masked && k0 + 32 * c + i > limit) ? 0.0f : exp2f(fmaf(v[i], p.scale_log2, -m_use));
                    const float x1 = (masked && k0 + 32 * c + i + 1 > limit) ? 0.0f : exp2f(fmaf(v[i + 1], p.scale_log2, -m_use));
                    const __half2 hh = __floats2half2_rn(x0, x1);
                    h[i >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                    const float2 back = __half22float2(hh);
                    psum += back.x + back.y;  // the sum of the weights the tensor core will actually use
                }
                uint8_t * half_tile = prow + (c >> 1) * kTileBytes;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int chunk = (c & 1) * 4 + u;
                    *reinterpret_cast<uint4 *>(half_tile + ((chunk ^ (row & 7)) << 4)) = make_uint4(h[4 * u], h[4 * u + 1], h[4 * u + 2], h[4 * u + 3]);
                }
            }
            tc_fence_before();
            mbar_arrive(bSfree);  // S may be overwritten by the next tile's Q.K^T
            fence_proxy_async_smem();
            mbar_arrive(bPready);  // P is visible to the tensor core
            l = l * alpha + psum;
            if (!mbar_wait_bounded(bPVdone, j & 1)) { give_up(); break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                tmem_ld32(t_row + kTile + 32 * c, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[32 * c + i] = fmaf(acc[32 * c + i], alpha, v[i]);
            }
            tc_fence_before();
            mbar_arrive(bOfree);
        }
        if (live && !aborted()) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            float4 * out = reinterpret_cast<float4 *>(p.dst + (((size_t) batch * p.n_q + qpos) * p.n_heads + head) * kHeadDim);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                out[i] = make_float4(acc[4 * i] * inv, acc[4 * i + 1] * inv, acc[4 * i + 2] * inv, acc[4 * i + 3] * inv);
        }
    }

    // common exit: tensor-core work has been waited for by the softmax warps; release TMEM
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

bool tc_route_ok(const vox_attn_args * a) {
    const vox_tensor &k = a->k, &v = a->v;
    if (k.type != VOX_TYPE_F16 || v.type != VOX_TYPE_F16) return false;
    if (k.ne[2] != v.ne[2] || k.ne[3] != v.ne[3]) return false;
    if (a->q.ne[1] < 1 || k.ne[1] < 1) return false;
    for (const vox_tensor * t : {&k, &v}) {
        if ((reinterpret_cast<uintptr_t>(t->data) & 15) != 0) return false;
        if (t->nb[1] % 16 || t->nb[2] % 16 || t->nb[3] % 16) return false;
    }
    return true;
}

}  // namespace

extern "C" {

size_t vox_attn_prefill_workspace_bytes(const vox_attn_args * a) {
    (void) a;
    return 0;
}

int vox_attn_prefill(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    (void) workspace;
    (void) workspace_bytes;
    VOX_REQUIRE(e && a, VOX_ATTN_INVALID_ARGUMENT, "vox_attn_prefill: null argument");
    VOX_REQUIRE(a->mask.data == nullptr, VOX_ATTN_INVALID_ARGUMENT,
                "vox_attn_prefill implies the causal mask; pass mask.data == NULL (use vox_attn_forward for explicit masks)");
    VOX_REQUIRE(vox_attn_supported(a), VOX_ATTN_INVALID_ARGUMENT, "%s", vox_attn_last_error_string());
    VOX_REQUIRE(a->q.data && a->k.data && a->v.data && a->dst.data, VOX_ATTN_INVALID_ARGUMENT, "null data pointer");
    VOX_REQUIRE(a->k.ne[1] >= a->q.ne[1], VOX_ATTN_INVALID_ARGUMENT, "n_kv %lld < n_q %lld", (long long) a->k.ne[1],
                (long long) a->q.ne[1]);
    const int    offset = (int) (a->k.ne[1] - a->q.ne[1]);
    cudaStream_t st     = static_cast<cudaStream_t>(stream);
    if (!tc_route_ok(a)) return launch_generic(e, a, offset, st);  // f32 / q8_0 K/V or unaligned strides

    CUtensorMap    mk, mv;
    const uint64_t dims[5] = {64, (uint64_t) a->k.ne[1], (uint64_t) a->k.ne[2], (uint64_t) a->k.ne[3], 1};
    const uint32_t box[5]  = {64, kTile, 1, 1, 1};
    const vox_tensor * ts[2] = {&a->k, &a->v};
    CUtensorMap *      ms[2] = {&mk, &mv};
    for (int i = 0; i < 2; ++i) {
        const uint64_t strides[4] = {ts[i]->nb[1], ts[i]->nb[2], ts[i]->nb[3],
                                     std::max<uint64_t>(ts[i]->nb[3] * (uint64_t) ts[i]->ne[3], 16)};
        int rc = make_tensor_map(e, ms[i], ts[i]->data, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != VOX_ATTN_OK) return rc;
    }
    if (!(e->attr_mask & (1u << 12))) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPf));
        e->attr_mask |= 1u << 12;
    }
    PrefillParams p;
    p.q = static_cast<const uint8_t *>(a->q.data);
    p.q_nb1 = a->q.nb[1]; p.q_nb2 = a->q.nb[2]; p.q_nb3 = a->q.nb[3];
    p.dst = static_cast<float *>(a->dst.data);
    p.n_q = (int) a->q.ne[1]; p.n_kv = (int) a->k.ne[1]; p.n_heads = (int) a->q.ne[2];
    p.gqa = (int) (a->q.ne[2] / a->k.ne[2]); p.causal_offset = offset;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.status = e->status_dev;
    dim3 grid((p.n_q + kTile - 1) / kTile, p.n_heads, (unsigned) a->q.ne[3]);
    prefill_tc_kernel<<<grid, kThreadsPf, kSmemPf, st>>>(mk, mv, p);
    return check_launch(e, "prefill_tc_kernel");
}

}  // extern "C"
