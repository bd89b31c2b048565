// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), K/V fed by TMA.
//
// Replaces the n_q == n_kv call that MiniCPMModel::forward makes with the f16 mask from
// create_causal_mask (src/minicpm.cpp:602-620, 779-802 -> :708-710); the mask is implied by a
// causal offset instead of being materialised and re-read (512 KB per 512-token graph there).
// On the CPU this is ggml's tiled path (third_party/ggml/src/ggml-cpu/ops.cpp:8347-8633); ggml-cuda
// would run the mma.sync kernel flash_attn_ext_f16 (fattn-mma-f16.cuh:1459-1628).
//
// A work item = 128 query rows of one head of one sequence.  CTAs are persistent (two per SM) and walk
// a heaviest-first item list in snake order; barriers, TMEM and the tile of ones are set up once, and the
// next item's Q rows are fetched while the current item's last P.V retires and its output is written.
// Ten warps:
//   warps 0-7  softmax: two threads per query row (row r = TMEM lane r).  Warps 0-3 own score columns
//              0-63 and output columns 0-31, warps 4-7 the other halves.  Per 128-key tile a thread
//              reads its scores from TMEM (tcgen05.ld), the pair agrees on the row maximum through shared
//              memory, each writes P = 2^(c*S - max) as f16 into shared memory in the 128-byte-swizzled
//              K-major layout the tensor core reads.  The output row and the row sums accumulate in TMEM
//              over all tiles (no per-tile read-back); they are rescaled in place only when the running
//              maximum jumps by more than 2^8, and read once at the end.
//   warp 8     producer: one lane issues cp.async.bulk.tensor copies of 128-row K tiles (one buffer,
//              refilled as soon as Q.K^T has retired, i.e. while the softmax of that tile runs) and V tiles
//              (two-stage ring).
//   warp 9     MMA issuer: one lane issues tcgen05.mma (kind::f16, M=128): S = Q.K^T (N=128, 4 k-steps)
//              into TMEM columns 0-127, O_tile = P.V (N=64, 8 k-steps, V read MN-major straight from the
//              row-major tile) into columns 128-191, and P.1 (N=16, a tile of ones) into columns 192-207,
//              which yields the row sums of exactly the rounded weights the tensor core used.
//              Completion is signalled with tcgen05.commit.
// Q arrives as f32 and is rounded to f16 once per CTA (exact when it already holds f16 values);
// scale*log2(e) is applied to S in f32.  Accumulation is f32 everywhere.  100 KB of shared memory and
// 256 TMEM columns per CTA: two CTAs share an SM, one computing softmax while the other waits on copies.
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
constexpr int kVStages   = 2;              // V tiles are prefetched two ahead; K has one buffer, refilled when Q.K^T retires
constexpr int kSoftmaxThreads = 256;
constexpr int kThreadsPf = kSoftmaxThreads + 64;
constexpr int kTmemCols  = 256;            // S: columns 0-127, O tile: 128-191, row sums: 192-207
constexpr int kOnesBytes = 4096;           // a [16][128] f16 tile of ones (any layout: every element is 1)
constexpr int kSmemPf    = kTileBytes * (1 + 1 + kVStages + 2) + kOnesBytes + 1024;  // Q, K, V ring, P (two 64-key halves), ones

struct PrefillParams {
    const uint8_t * q;
    size_t          q_nb1, q_nb2, q_nb3;
    float *         dst;
    int             n_q, n_kv, n_heads, gqa, causal_offset;
    int             n_batch, n_qtiles, n_items;
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
// 64 consecutive columns: two loads in flight, one wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
    uint32_t r[64];
#pragma unroll
    for (int h = 0; h < 2; ++h)
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[32 * h + 0]), "=r"(r[32 * h + 1]), "=r"(r[32 * h + 2]), "=r"(r[32 * h + 3]), "=r"(r[32 * h + 4]), "=r"(r[32 * h + 5]),
              "=r"(r[32 * h + 6]), "=r"(r[32 * h + 7]), "=r"(r[32 * h + 8]), "=r"(r[32 * h + 9]), "=r"(r[32 * h + 10]), "=r"(r[32 * h + 11]),
              "=r"(r[32 * h + 12]), "=r"(r[32 * h + 13]), "=r"(r[32 * h + 14]), "=r"(r[32 * h + 15]), "=r"(r[32 * h + 16]), "=r"(r[32 * h + 17]),
              "=r"(r[32 * h + 18]), "=r"(r[32 * h + 19]), "=r"(r[32 * h + 20]), "=r"(r[32 * h + 21]), "=r"(r[32 * h + 22]), "=r"(r[32 * h + 23]),
              "=r"(r[32 * h + 24]), "=r"(r[32 * h + 25]), "=r"(r[32 * h + 26]), "=r"(r[32 * h + 27]), "=r"(r[32 * h + 28]), "=r"(r[32 * h + 29]),
              "=r"(r[32 * h + 30]), "=r"(r[32 * h + 31])
            : "r"(taddr + 32 * h)
            : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, float x) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(__float_as_uint(x)) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    return __uint_as_float(r);
}

// 2^x on the special-function unit (one MUFU instruction; arguments here are <= 0)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
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

// Rare path of the softmax warps, kept out of line so that its 32 registers do not weigh on the tile loop:
// multiply this thread's 32 output columns (and, for the first column half, the row sum) in TMEM by f.
__device__ __noinline__ void rescale_accumulators(uint32_t t_row, int half, float f) {
    tc_fence_after();
    float o[32];
    tmem_ld32(t_row + kTile + 32 * half, o);
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] *= f;
    tmem_st32(t_row + kTile + 32 * half, o);
    if (half == 0) tmem_st1(t_row + kTile + kHeadDim, tmem_ld1(t_row + kTile + kHeadDim) * f);
    tc_fence_before();
}

// One unit of work: 128 query rows (tile `qtile`) of one head of one sequence.  Items are numbered
// heaviest first (late query tiles see more keys); CTA c of G takes items c, 2G-1-c, 2G+c, ... so that
// a heavy first item is followed by a light one.
struct WorkItem {
    int qtile, head, batch, n_tiles, q0;
};
__device__ __forceinline__ bool work_item(const PrefillParams & p, int round, WorkItem & w) {
    const int G = gridDim.x, c = blockIdx.x;
    const int idx = round * G + ((round & 1) ? G - 1 - c : c);
    if (idx >= p.n_items) return false;
    const int per_tile = p.n_heads * p.n_batch;
    const int rest     = idx % per_tile;
    w.qtile = p.n_qtiles - 1 - idx / per_tile;
    w.head  = rest % p.n_heads;
    w.batch = rest / p.n_heads;
    w.q0    = w.qtile * kTile;
    const int last_row = min(w.q0 + kTile, p.n_q) - 1;
    w.n_tiles = min((p.n_kv + kTile - 1) / kTile, (last_row + p.causal_offset) / kTile + 1);
    return true;
}

__global__ void __launch_bounds__(kThreadsPf, 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * kVStages + 8];
    __shared__ float    half_max[2][2][kTile];  // [tile parity][column half][row]
    __shared__ uint32_t tmem_base_slot;
    __shared__ int      abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *      smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sQ = smem_base, sK = smem_base + kTileBytes, sV0 = sK + kTileBytes, sP = sV0 + kVStages * kTileBytes,
                   sOnes = sP + 2 * kTileBytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const uint32_t vfull0 = smem_u32(&bars[0]), vempty0 = smem_u32(&bars[kVStages]);
    const uint32_t bQ = smem_u32(&bars[2 * kVStages]), bSready = bQ + 8, bSfree = bQ + 16, bPready = bQ + 24, bPVdone = bQ + 32,
                   kfull = bQ + 48, kempty = bQ + 56;
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kVStages; ++s) {
            mbar_init(vfull0 + 8 * s, 1);
            mbar_init(vempty0 + 8 * s, 1);
        }
        mbar_init(kfull, 1);
        mbar_init(kempty, 1);
        mbar_init(bQ, kSoftmaxThreads / 32);  // one arrival per softmax warp
        mbar_init(bSready, 1);
        mbar_init(bSfree, kSoftmaxThreads / 32);
        mbar_init(bPready, kSoftmaxThreads / 32);
        mbar_init(bPVdone, 1);
        fence_mbar_init();
    }
    if (warp == 9) tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();  // barriers and TMEM are set up while the previous kernel drains; Q, K, V are read after this
    pdl_launch_dependents();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&tmem_base_slot);

    auto give_up = [&]() {
        atomicOr(p.status, kStatusTimeout);
        atomicExch(&abort_flag, 1);
    };
    auto aborted = [&]() { return *reinterpret_cast<volatile int *>(&abort_flag) != 0; };

    // The CTA is persistent: every role walks the same item sequence; T counts key tiles over all items
    // and fixes the phase of every barrier (one K copy, one S, one P and one P.V per tile).
    if (warp == 8) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
            WorkItem w;
            int      T  = 0;
            bool     ok = true;
            for (int round = 0; ok && work_item(p, round, w); ++round) {
                const int kvh = w.head / p.gqa;
                for (int j = 0; j < w.n_tiles && !aborted(); ++j, ++T) {
                    const int s = T % kVStages;
                    if (T >= 1 && !mbar_wait_spin(kempty, (T - 1) & 1)) { give_up(); ok = false; break; }
                    mbar_expect_tx(kfull, kTileBytes);
                    tma_load_5d(sK, &map_k, kfull, 0, j * kTile, kvh, w.batch, 0);
                    if (T >= kVStages && !mbar_wait_spin(vempty0 + 8 * s, ((T / kVStages) - 1) & 1)) { give_up(); ok = false; break; }
                    mbar_expect_tx(vfull0 + 8 * s, kTileBytes);
                    tma_load_5d(sV0 + s * kTileBytes, &map_v, vfull0 + 8 * s, 0, j * kTile, kvh, w.batch, 0);
                }
                if (aborted()) break;
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_f16(kTile, false), idesc_pv = idesc_f16(kHeadDim, true), idesc_sum = idesc_f16(16, false);
            // S = Q K^T of global tile T: four k-steps of 16 along head_dim, 32 bytes each inside the swizzle atom.
            // It is issued as soon as the softmax threads have taken S of tile T-1 out of TMEM, i.e. while
            // they are still busy with the exponentials of tile T-1.
            auto issue_qk = [&](int T) {
                if (!mbar_wait_spin(kfull, T & 1)) return false;
                if (T > 0 && !mbar_wait_spin(bSfree, (T - 1) & 1)) return false;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_f16(tmem, smem_desc_sw128(sQ + 32 * k), smem_desc_sw128(sK + 32 * k), idesc_qk, k > 0);
                tc_commit(bSready);
                tc_commit(kempty);  // the K tile may be refilled once Q.K^T has retired
                return true;
            };
            WorkItem w;
            int      T  = 0;
            bool     ok = true;
            for (int round = 0; ok && work_item(p, round, w); ++round) {
                // the first Q.K^T of an item needs the item's Q tile; later ones were issued one tile ahead
                if (!mbar_wait_spin(bQ, round & 1) || !issue_qk(T)) { give_up(); break; }
                for (int j = 0; j < w.n_tiles && !aborted(); ++j, ++T) {
                    if (j + 1 < w.n_tiles && !issue_qk(T + 1)) { give_up(); ok = false; break; }
                    const int      s  = T % kVStages;
                    const uint32_t sV = sV0 + s * kTileBytes;
                    if (!mbar_wait_spin(vfull0 + 8 * s, (T / kVStages) & 1)) { give_up(); ok = false; break; }
                    if (!mbar_wait_spin(bPready, T & 1)) { give_up(); ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < 8; ++k) {  // eight k-steps of 16 keys; P half-tiles of 64 keys, V rows 16 at a time
                        const uint64_t pd = smem_desc_sw128(sP + (k >> 2) * kTileBytes + 32 * (k & 3));
                        tc_mma_f16(tmem + kTile, pd, smem_desc_sw128(sV + 2048 * k), idesc_pv, j > 0 || k > 0);     // O += P V
                        tc_mma_f16(tmem + kTile + kHeadDim, pd, smem_desc_sw128(sOnes), idesc_sum, j > 0 || k > 0);  // row sums += P 1
                    }
                    tc_commit(bPVdone);
                    tc_commit(vempty0 + 8 * s);
                }
                if (aborted()) break;
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps: two threads per query row
        const int row  = 32 * (warp & 3) + lane;  // == TMEM lane; a warp may only touch lanes 32*(warp%4)..+31
        const int half = warp >> 2;               // 0: score columns 0-63 / output columns 0-31, 1: the rest
        const uint32_t t_row = tmem + ((uint32_t) (32 * (warp & 3)) << 16);  // this warp's lane quarter
        uint8_t * const q_dst = smem_gen + row * 128;
        uint8_t * const p_dst = smem_gen + (sP - smem_base) + half * kTileBytes + row * 128;

        // this thread's half of a Q row: f32 from memory, f16 into four 16-byte chunks at their swizzled places
        auto load_q = [&](const WorkItem & w, float4 (&qv)[8]) {
            const int qpos = w.q0 + row;
            if (qpos < p.n_q) {
                const float4 * src = reinterpret_cast<const float4 *>(p.q + (size_t) qpos * p.q_nb1 + (size_t) w.head * p.q_nb2 +
                                                                      (size_t) w.batch * p.q_nb3) + 8 * half;
#pragma unroll
                for (int i = 0; i < 8; ++i) qv[i] = src[i];
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) qv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        auto store_q = [&](const float4 (&qv)[8], int round) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = 4 * half + u;
                *reinterpret_cast<uint4 *>(q_dst + ((c ^ (row & 7)) << 4)) =
                    make_uint4(pack_half2(qv[2 * u].x, qv[2 * u].y), pack_half2(qv[2 * u].z, qv[2 * u].w),
                               pack_half2(qv[2 * u + 1].x, qv[2 * u + 1].y), pack_half2(qv[2 * u + 1].z, qv[2 * u + 1].w));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bQ);
            (void) round;
        };

        WorkItem w, wn;
        bool     have = work_item(p, 0, w);
        {
            const uint32_t one2 = 0x3C003C00u;
            *reinterpret_cast<uint4 *>(smem_gen + (sOnes - smem_base) + tid * 16) = make_uint4(one2, one2, one2, one2);
            if (have) {
                float4 qv[8];
                load_q(w, qv);
                store_q(qv, 0);
            }
        }
        int  T  = 0;
        bool ok = true;
        for (int round = 0; have && ok; ++round) {
            const int  qpos  = w.q0 + row;
            const bool live  = qpos < p.n_q;
            const int  limit = min(qpos + p.causal_offset, p.n_kv - 1);  // last key this row may see
            // The output row and the row sum accumulate in TMEM across all key tiles, both scaled by
            // 2^(-m_ref): their ratio does not depend on m_ref, so the reference maximum only has to keep
            // the weights inside f16 range.  It is raised (and the accumulated columns rescaled) only when a
            // tile's maximum exceeds it by more than 2^8, which after the first tile is rare.
            float m_ref = -INFINITY;
            for (int j = 0; j < w.n_tiles && !aborted(); ++j, ++T) {
                if (!mbar_wait_bounded(bSready, T & 1)) { give_up(); ok = false; break; }
                tc_fence_after();
                const int  k0     = j * kTile + 64 * half;  // first key of this thread's columns
                const bool masked = j * kTile + kTile - 1 > min(w.q0 + p.causal_offset, p.n_kv - 1);  // CTA-uniform: the tile may be cut
                // pass 1: maximum over this thread's 64 columns (two 32-column reads), then over the row through
                // shared memory.  S is read from TMEM again in pass 2 instead of being kept: 64 more live registers
                // would spill at two CTAs per SM.
                float v[32];
                float tmax = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    tmem_ld32(t_row + 64 * half + 32 * c, v);
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = k0 + 32 * c + i > limit ? -INFINITY : v[i];
                    }
                    float t0 = v[0], t1 = v[1], t2 = v[2], t3 = v[3];  // four chains instead of one long dependency
#pragma unroll
                    for (int i = 4; i < 32; i += 4) {
                        t0 = fmaxf(t0, v[i]); t1 = fmaxf(t1, v[i + 1]); t2 = fmaxf(t2, v[i + 2]); t3 = fmaxf(t3, v[i + 3]);
                    }
                    tmax = fmaxf(tmax, fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)));
                }
                half_max[T & 1][half][row] = tmax;
                named_bar_sync(1, kSoftmaxThreads);
                tmax = fmaxf(tmax, half_max[T & 1][half ^ 1][row]) * p.scale_log2;
                // the previous tile's P.V must have retired before P is overwritten (and before O is touched);
                // at the first tile of an item that wait was done when the previous item was read out
                if (j > 0 && !mbar_wait_bounded(bPVdone, (T - 1) & 1)) { give_up(); ok = false; break; }
                // tcgen05.ld/st are warp-collective: the decision to rescale is taken per warp (any lane), and lanes
                // that do not need it take part with a factor of 1
                const bool raise = j > 0 && tmax > m_ref + 8.0f;
                if (j == 0) {
                    m_ref = tmax;  // key 0 is visible to every row: finite
                } else if (__any_sync(0xffffffffu, raise)) {
                    const float f = raise ? ex2_approx(m_ref - tmax) : 1.0f;
                    if (raise) m_ref = tmax;
                    rescale_accumulators(t_row, half, f);
                }
                // pass 2: P = 2^(c*S - m_ref), f16, into this thread's 64-key half of the P tile, 8 keys (16 bytes) at a time
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    tmem_ld32(t_row + 64 * half + 32 * c, v);
                    if (c == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bSfree);  // S has been read for the last time: the next Q.K^T may overwrite it
                    }
                    if (masked) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = k0 + 32 * c + i > limit ? -INFINITY : v[i];
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint32_t h[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            h[i] = pack_half2(ex2_approx(fmaf(v[8 * u + 2 * i], p.scale_log2, -m_ref)),
                                              ex2_approx(fmaf(v[8 * u + 2 * i + 1], p.scale_log2, -m_ref)));
                        *reinterpret_cast<uint4 *>(p_dst + (((4 * c + u) ^ (row & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bPready);  // this warp's part of P is visible to the tensor core
            }
            if (!ok || aborted()) break;
            // item done: read the result out once the last P.V has retired, then bring in the next item's Q rows
            const bool have_next = work_item(p, round + 1, wn);
            if (!mbar_wait_bounded(bPVdone, (T - 1) & 1)) { give_up(); break; }
            // warp-collective TMEM reads by every lane; only rows that exist are stored
            tc_fence_after();
            const float l = tmem_ld1(t_row + kTile + kHeadDim);  // sum of exactly the rounded weights the tensor core used
            float o[32];
            tmem_ld32(t_row + kTile + 32 * half, o);
            tc_fence_before();
            if (live) {
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;
                float4 * out = reinterpret_cast<float4 *>(p.dst + (((size_t) w.batch * p.n_q + qpos) * p.n_heads + w.head) * kHeadDim + 32 * half);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    out[i] = make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
            }
            // every Q.K^T of this item has retired (its last S was consumed above), so the Q tile may be replaced
            if (have_next) {
                float4 qv[8];
                load_q(wn, qv);
                store_q(qv, round + 1);
            }
            have = have_next;
            w    = wn;
        }
    }

    // common exit: tensor-core work has been waited for by the softmax warps; release TMEM
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

bool tc_route_ok(const vox_attn_args * a) {
    const vox_tensor &k = a->k, &v = a->v;
    if (k.type != VOX_TYPE_F16 || v.type != VOX_TYPE_F16) return false;
    if (k.ne[2] != v.ne[2] || k.ne[3] != v.ne[3]) return false;
    if (a->q.ne[1] < 1 || k.ne[1] < 1) return false;
    // Q rows are read with 16-byte loads
    if ((reinterpret_cast<uintptr_t>(a->q.data) & 15) != 0 || a->q.nb[1] % 16 || a->q.nb[2] % 16 || a->q.nb[3] % 16) return false;
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
    p.n_batch  = (int) a->q.ne[3];
    p.n_qtiles = (p.n_q + kTile - 1) / kTile;
    const long long items = (long long) p.n_qtiles * p.n_heads * p.n_batch;
    VOX_REQUIRE(items < (1LL << 30), VOX_ATTN_INVALID_ARGUMENT, "too many query tiles");
    p.n_items = (int) items;
    // persistent CTAs, two per SM (100 KB of shared memory and 256 TMEM columns each)
    dim3 grid((unsigned) std::min<long long>(items, 2LL * e->sm_count));
    launch_pdl(prefill_tc_kernel, grid, dim3(kThreadsPf), kSmemPf, st, mk, mv, p);
    return check_launch(e, "prefill_tc_kernel");
}

}  // extern "C"
