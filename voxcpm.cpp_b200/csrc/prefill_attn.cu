// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), K/V fed by TMA.
//
// Replaces the n_q == n_kv call that MiniCPMModel::forward makes with the f16 mask from
// create_causal_mask (src/minicpm.cpp:602-620, 779-802 -> :708-710); the mask is implied by a
// causal offset instead of being materialised and re-read (512 KB per 512-token graph there).
// On the CPU this is ggml's tiled path (third_party/ggml/src/ggml-cpu/ops.cpp:8347-8633); ggml-cuda
// would run the mma.sync kernel flash_attn_ext_f16 (fattn-mma-f16.cuh:1459-1628).
//
// A work item = 128 rows: 16 consecutive tokens x the 8 query heads that share a kv head (row r = token r / 8, head
// r % 8; 128 tokens of one head when the GQA ratio is odd), walked over 128-key tiles, so that a K/V tile is fetched
// once for the whole group (the incumbent packs its GQA heads the same way, fattn-mma-f16.cuh:38-72).  CTAs are
// persistent, one per SM, and take items from a heaviest-first list in snake order; barriers, TMEM (464 of the 512
// columns) and the tile of ones are set up once.  A key tile is scored and weighted as two SCORE TILES of 64 keys
// (the second is left out where no row of the item can see it), each in one of six 64-column score buffers in TMEM:
// a buffer is held from Q.K^T until P.V has retired, several times longer than the softmax works on it, so it is the
// number of buffers that lets the tensor core, the softmax warps and the issuers run on different tiles at once.
// Sixteen warps in four warpgroups, which trade registers after launch (setmaxnreg: the launch allots 128 per thread,
// the two softmax groups take 168, the others keep 56 and 96):
//   warps 0-3, 8-11  softmax: one thread per query row (row r = TMEM lane r; warps w and w + 8 share a lane quarter).
//              Warps 0-3 take the even score tiles, warps 8-11 the odd ones.  Per tile a thread reads its 64 scores
//              from TMEM (tcgen05.ld), takes their maximum, and writes P = 2^(c*S - m_ref) back into TMEM (tcgen05.st)
//              over the tile's scores as two packed-f16 tiles hi + lo (~21 bits: one f16 per weight measured 2.3e-3 to
//              5e-3 of the output RMS on random sequences of 512 to 4096 tokens, outside the 2e-3 parity bound; hi + lo
//              measures under 6e-5): the tensor core takes the weights from there as the A operand of P.V, so they
//              never pass through shared memory.  The output row and the row sums accumulate in TMEM over all tiles (no per-tile
//              read-back); they are rescaled in place only when a tile's maximum exceeds the reference m_ref by more
//              than 2^8.  The reference of a row passes from the thread of one score tile to the thread of the next
//              (the other group) through shared memory and an mbarrier; it is handed on half-way through the
//              exponentials, so the two groups overlap there without starting them together.  These warps do
//              nothing else: from the last tile of an item they go straight to the first tile of the next.
//   warp 4     producer: one lane issues cp.async.bulk.tensor copies of 128-row K and V tiles into three-stage rings.
//   warp 6     score issuer: S = Q.K^T (tcgen05.mma kind::f16, M = 128, N = 64, 4 k-steps, both operands in shared
//              memory) into score buffer U % 6, up to six score tiles ahead of P.V and across item boundaries.
//   warp 5     output issuer: O += P.V and the row sums come from ONE instruction per 16 keys and weight part
//              (N = 80, 4 k-steps for hi, 4 for lo): P from TMEM, V read MN-major straight from its row-major tile,
//              and a tile of ones addressed as columns 64-79 of every 16-key step, which yields the sums of exactly
//              the rounded weights the tensor core used.  One thread issues both parts, so the order of the f32
//              accumulation, and with it every bit of the result, is the same in every run.  Completion is signalled
//              with tcgen05.commit.  (Warp 7 only fills the group.)
//              Both issuer warps run their loops with all 32 lanes (waits and votes by the warp, the instructions by
//              one elected lane): in warp-uniform control flow the descriptors live in uniform registers, where
//              tcgen05.mma takes them from.  Issued from inside a one-lane branch an instruction cost its thread about
//              80 clocks, now about 40 (a commit costs 46, a satisfied barrier wait 47: measured alone).
//   warps 12-15 in/out: one thread per query row again.  They keep the Q tiles of the next two items in shared
//              memory (f32 from memory, rounded to f16 once, exact when it already holds f16 values; the raw rows of
//              the item after those wait in a staging area, brought there by two bulk-tensor loads a whole item ahead) and read each
//              finished output row out of TMEM, normalise it and put it into an output staging tile, which two
//              bulk-tensor stores carry to its place (rows past n_q clipped by the copy), handing the columns back to
//              the issuer.
// What bounds it, measured by leaving parts out (developer builds, 2048 tokens x 2 sequences, 29.4 key tiles per CTA,
// one layer 41 us): barriers, commits and waits alone, with no copy, no MMA, no softmax arithmetic and no global
// traffic, 16.5 us (about 450 clocks per score tile although six are in flight and no single wait, arrive or commit
// costs more than 50 clocks to issue); with the MMAs 27 us; with Q in and results out as well 29 us (33 while a thread
// per row fetched and stored its 256 bytes itself); the softmax arithmetic adds the last 12.  The exponentials (16 per clock and SM) and the two conversions to packed f16 per pair of
// weights (32 per clock and SM, on the same unit) bound the arithmetic itself at 1175-1300 clocks per 128 x 128 tile
// with two or three warps per scheduler at work (measured alone; integer forms of the split, with shifts and byte
// permutes instead of conversions, measured slower: 1400-1900), against 2000 for the whole tile period.  Arrangements
// tried on this skeleton, none of which moved the 2048-token figure by more than 3 %: both softmax groups on the same
// tile with 64 keys per thread and a trade of maxima (the first form of this kernel); 128-key score tiles with
// three buffers; three softmax groups (640 threads, 120 registers each); handing the reference on before, during or
// after the exponentials; polling instead of parked waits in the issuers; two output accumulators so that an item's
// first P.V need not wait for the read-out of the item before.
// scale*log2(e) is applied to S in f32.  Accumulation is f32 everywhere.  195 KB of shared memory per CTA (as much
// with remainder tiles, which leave no room for the two staging areas: rows are then fetched and stored by their threads).  Every wait on a barrier is bounded; on expiry the
// status word is set and all roles fall through to the common exit, where the TMEM columns are released.  The
// register trade cannot block: what the softmax groups take, the other two have given up before (static_assert below).
//
// Three forms of the kernel share this code (template parameters):
//   kSplitP  the weights as hi + lo (the product path; a single f16 is kept for comparison);
//   kMask    an additive f16 mask tensor is read instead of implying the causal one: this is what vox_attn_forward
//            uses for the reference's own prefill call and for any other masked call with 32 or more keys.  A small
//            kernel first notes which key tiles the mask leaves anything of, and every role walks only those;
//   kVLo     K/V that are not f16 (q8_0 blocks, f32) are expanded by a small kernel into an f16 value tile and an f16
//            remainder tile each, Q is kept as value + remainder too, and the remainders take extra Q.K^T and P.V
//            passes (36 tcgen05.mma per tile instead of 20), so that nothing is lost to f16 rounding.
#include "tcgen05.cuh"

#include <algorithm>
#include <cstdlib>

using namespace vox;

namespace vox {
int launch_generic(vox_engine * e, const vox_attn_args * a, int causal_offset, cudaStream_t stream);
// the tensor-core kernel with an explicit additive mask (called by vox_attn_forward)
bool   prefill_mask_route_ok(const vox_attn_args * a);
size_t prefill_mask_workspace_bytes(const vox_attn_args * a);
size_t prefill_mask_workspace_min(const vox_attn_args * a);
int    launch_prefill_mask(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t stream);
bool   prefill_full_route_ok(const vox_attn_args * a);
size_t prefill_full_workspace_bytes(const vox_attn_args * a);
int    launch_prefill_full(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t stream);
}

namespace {

// Developer build only (-DVOX_ATTN_DEVELOPER -DVOX_PREFILL_PROFILE): per-role cycle counters (SM clock, summed over
// CTAs with atomics) that vox_debug_prefill_profile copies out.  Compiled out of the product library.
// With -DVOX_PREFILL_TRACE alone only the time stamps of CTA 0 are taken (one store per event: the counters cost the
// roles a hundred clocks per tile).
#if defined(VOX_ATTN_DEVELOPER) && (defined(VOX_PREFILL_PROFILE) || defined(VOX_PREFILL_TRACE))
__device__ unsigned long long g_prof[32];
// CTA 0, first 64 score tiles.  0 scores seen, 1 weights signalled, 2 weights seen by the output issuer, 3 its MMAs issued
// and committed, 4 buffer seen free by the score issuer, 5 its MMAs issued and committed; softmax thread: 11 before the
// wait for the scores, 6 scores loaded, 7 maximum taken, 8 reference seen, 9 weights computed, 10 their stores complete
// (12, 13: loop top at the other group's tile, own tile entered); output issuer: 14 loop top, 15 fenced, 16 MMAs issued,
// 17 commits issued; 18-21: weights signalled by each of the four warps of the tile's group
__device__ long long g_trace[22][64];
#define PROF_TRACE(k, T) do { if (blockIdx.x == 0 && (T) < 64) g_trace[k][T] = clock64(); } while (0)
#endif
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_PREFILL_PROFILE)
#define PROF_VARS long long pf_t = 0, pf_acc[12] = {0}
#define PROF_START() pf_t = clock64()
#define PROF_STOP(i) do { const long long pf_n = clock64(); pf_acc[i] += pf_n - pf_t; pf_t = pf_n; } while (0)
#define PROF_COUNT(i, n) pf_acc[i] += (n)
#define PROF_FLUSH(base, n) do { for (int pf_i = 0; pf_i < (n); ++pf_i) atomicAdd(&g_prof[(base) + pf_i], (unsigned long long) pf_acc[pf_i]); } while (0)
#else
#define PROF_VARS
#define PROF_START()
#define PROF_STOP(i)
#define PROF_COUNT(i, n)
#define PROF_FLUSH(base, n)
#if !(defined(VOX_ATTN_DEVELOPER) && defined(VOX_PREFILL_TRACE))
#define PROF_TRACE(k, T)
#endif
#endif

// Developer builds only (-DVOX_ATTN_DEVELOPER): VOX_PREFILL_NOSOFTMAX, VOX_PF_SKIP_QK, VOX_PF_SKIP_PV, VOX_PF_SKIP_LOAD and
// VOX_PF_SKIP_IO leave out the softmax arithmetic, the two kinds of MMA, the K/V copies and the global traffic of the
// in/out warps, one by one; the barrier protocol stays whole, the results are meaningless, the timings are the
// decomposition quoted in the header.  Compiled out of the product library.
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_PF_SKIP_PV)
#define VOX_PF_SKIP_PV_LO 1
#else
#define VOX_PF_SKIP_PV_LO 0
#endif
constexpr int kTile      = 128;            // query rows per item
constexpr int kKeys      = 128;            // keys per tile
constexpr int kQBytes    = kTile * 128;    // the item's [128][64] f16 Q tile
constexpr int kKvBytes   = kKeys * 128;    // one [128][64] f16 K or V tile
constexpr int kStages    = 6;              // most stages a K or V ring has (barrier slots)
constexpr int kSub       = 64;             // keys per score tile: a key tile is scored and weighted in two halves
constexpr int kSBufs     = 6;              // score buffers in TMEM
#ifndef VOX_PREFILL_GROUPS
#define VOX_PREFILL_GROUPS 2
#endif
#ifndef VOX_PREFILL_PUBLISH_AT
#define VOX_PREFILL_PUBLISH_AT 2
#endif
// After how many of its four blocks of 16 weights the thread of a score tile passes the row's reference on to the thread
// of the next tile, which waits for it before its own exponentials: 0 lets all groups run their exponentials at the same
// time (and then wait and load at the same time), 4 lets one group at a time run them; in between the groups overlap.
constexpr int kPublishAt = VOX_PREFILL_PUBLISH_AT;
constexpr int kGroups    = VOX_PREFILL_GROUPS;  // softmax warpgroups: score tile U is taken by group U % kGroups
constexpr int kSoftmaxThreads = 128 * kGroups;  // one thread per query row in each group
constexpr int kIoThreads = 128;
constexpr int kThreadsPf = 256 + kSoftmaxThreads;  // softmax 0, control (producer, two issuers, one idle warp), softmax 1, in/out, softmax 2
constexpr int kQBufs     = 2;              // Q tiles of two consecutive items
// Registers per thread after the warpgroups have traded (setmaxnreg).  One CTA per SM: the launch allots 128 x 512;
// what the softmax groups take beyond that, the other two have given up before (they do so first thing).
constexpr int kRegsLaunch = kGroups == 3 ? 96 : 128, kRegsSoftmax = kGroups == 3 ? 120 : 168, kRegsControl = kGroups == 3 ? 48 : 56,
              kRegsIo = kGroups == 3 ? 72 : 96;
static_assert(kRegsLaunch == 65536 / kThreadsPf / 8 * 8, "what a thread holds at launch");
static_assert(kGroups * (kRegsSoftmax - kRegsLaunch) <= (kRegsLaunch - kRegsControl) + (kRegsLaunch - kRegsIo), "the trade cannot block");
static_assert((kGroups * kRegsSoftmax + kRegsControl + kRegsIo) * 128 <= 65536, "the CTA's registers fit the SM");
// TMEM columns: six score buffers of 64 columns (score tile U uses buffer U % 6; its weights, packed f16, replace its
// scores: high parts in the first 32 columns, low parts in the last 32) and the output row with its row sum
constexpr int kTmemCols  = 512;
constexpr int kSCol      = 0;              // S: 6 x 64 columns
constexpr int kOCol      = kSBufs * kSub;  // O: 64 columns, row sums: 16 columns behind them
constexpr int kOnesBytes = 2048;           // 16 keys x 64 ones, addressed as columns 64-79 of every 16-key step of every V tile
// With kVLo (K/V expanded from q8_0 or f32) a K or V stage holds two tiles, the f16 values and what their rounding left
// over, and the rings are two stages deep instead of three (five stages measured 5 % slower than three: the rings
// are not what the kernel waits for) ...
#ifndef VOX_PREFILL_STAGES
#define VOX_PREFILL_STAGES 3
#endif
constexpr int stages_of(bool v_lo) { return v_lo ? 2 : VOX_PREFILL_STAGES; }
constexpr int v_stage_bytes(bool v_lo) { return v_lo ? 2 * kKvBytes : kKvBytes; }
// ... and a Q buffer holds the f16 tile and the remainder tile as well
constexpr int q_buf_bytes(bool v_lo) { return v_lo ? 2 * kQBytes : kQBytes; }
// Without remainder tiles there is room for a staging area the size of a raw Q tile (128 rows of 64 floats): the rows of
// the item after the two whose Q tiles are in place are copied there asynchronously (cp.async) a whole item ahead
constexpr int kQStageBytes = kTile * kHeadDim * 4;
// ... and for an output tile of the same size, from which finished rows leave by bulk-tensor stores (two 128-row halves of
// 128 bytes per row, in the 128-byte swizzle of the tensor map)
constexpr int kOutStageBytes = kTile * kHeadDim * 4;
constexpr int smem_pf(bool v_lo) {  // Q x 2, K ring, V ring, ones, Q staging, output staging
    return kQBufs * q_buf_bytes(v_lo) + stages_of(v_lo) * 2 * v_stage_bytes(v_lo) + kOnesBytes + (v_lo ? 0 : kQStageBytes + kOutStageBytes) + 1024;
}

struct PrefillParams {
    const uint8_t * q;
    size_t          q_nb1, q_nb2, q_nb3;
    float *         dst;
    int             n_q, n_kv, n_heads, gqa, causal_offset;
    int             n_batch, n_qtiles, n_items;
    // The 128 rows of an item are `tok` consecutive tokens x `pack` query heads that share a kv head (row r = token
    // r / pack, head r % pack): K and V tiles are fetched once for the whole group (the incumbent packs its GQA heads
    // the same way, third_party/ggml/src/ggml-cuda/fattn-mma-f16.cuh:38-72).  pack = 8, 4, 2 or 1, tok = 128 / pack.
    int             pack, tok, n_hgroups;
    float           scale_log2;
    int *           status;
    // additive f16 mask (kMask kernels): rows of n_kv values, planes broadcast over heads and sequences
    const uint8_t * mask;
    size_t          m_nb1, m_nb2, m_nb3;
    int             m_ne2, m_ne3;
    float           scale;
    // per (mask plane, query tile): 64 bytes, byte j set when key tile j holds a finite mask value for some row (NULL: not
    // known)
    const uint8_t * tile_live;
    // the same shape: byte j set when the mask adds 0 to every score of key tile j (the kernel then does not read it there)
    const uint8_t * tile_zero;
};

// Rare path of the softmax warps, kept out of line so that its registers do not weigh on the tile loop:
// multiply this thread's output row and row sum in TMEM by f.
__device__ __noinline__ void rescale_accumulators(uint32_t t_row, float f) {
    tc_fence_after();
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
        float o[32];
        tmem_ld32(t_row + kOCol + 32 * h, o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= f;
        tmem_st32(t_row + kOCol + 32 * h, o);
    }
    tmem_st1(t_row + kOCol + kHeadDim, tmem_ld1(t_row + kOCol + kHeadDim) * f);
    tc_fence_before();
}

// One unit of work: 128 rows = `tok` tokens (tile `qtile`) x `pack` heads of one sequence.  Items are numbered
// heaviest first (late query tiles see more keys); CTA c of G takes items c, 2G-1-c, 2G+c, ... so that
// a heavy first item is followed by a light one.
struct WorkItem {
    int                qtile, head, batch, n_tiles, q0;  // head: the first of the group; q0: the first token
    unsigned long long live;  // key tiles to walk, as bits (at most 64 when some are left out)
    unsigned long long zero;  // key tiles where the mask adds nothing for any row (known only together with `live`)
};
// 64 flag bytes (0 or 1, 16-byte aligned) -> a word with bit j = byte j: the multiplier gathers the low bits of eight bytes
// into the top byte of the product.
__device__ __forceinline__ unsigned long long bytes_to_bits(const uint8_t * flags) {
    const ulonglong2 * f = reinterpret_cast<const ulonglong2 *>(flags);
    unsigned long long bits = 0ull;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const ulonglong2 x = __ldg(f + i);
        bits |= ((x.x * 0x0102040810204080ull) >> 56) << (16 * i);
        bits |= ((x.y * 0x0102040810204080ull) >> 56) << (16 * i + 8);
    }
    return bits;
}

template <bool kMask>
__device__ __forceinline__ bool work_item(const PrefillParams & p, int round, WorkItem & w) {
    const int G = gridDim.x, c = blockIdx.x;
    const int idx = round * G + ((round & 1) ? G - 1 - c : c);
    if (idx >= p.n_items) return false;
    const int per_tile = p.n_hgroups * p.n_batch;
    const int rest     = idx % per_tile;
    w.qtile = p.n_qtiles - 1 - idx / per_tile;
    w.head  = (rest % p.n_hgroups) * p.pack;
    w.batch = rest / p.n_hgroups;
    w.q0    = w.qtile * p.tok;
    const int last_tok = min(w.q0 + p.tok, p.n_q) - 1;
    w.n_tiles = min((p.n_kv + kKeys - 1) / kKeys, (last_tok + p.causal_offset) / kKeys + 1);
    w.live    = ~0ull;
    w.zero    = 0ull;
    if (kMask && p.tile_live != nullptr) {  // only set for n_tiles <= 64; a tile where the mask hides every key from every row is left out
        unsigned long long seen = 0ull, zero = ~0ull;
        const int n_planes = min(p.pack, p.m_ne2);  // the heads of the group may read different planes of the mask
        for (int h = 0; h < n_planes; ++h) {
            const size_t at = (((size_t) (w.batch % p.m_ne3) * p.m_ne2 + ((w.head + h) % p.m_ne2)) * p.n_qtiles + w.qtile) * 64;
            seen |= bytes_to_bits(p.tile_live + at);
            zero &= bytes_to_bits(p.tile_zero + at);
        }
        const int n_kt = (p.n_kv + kKeys - 1) / kKeys;  // bytes of key tiles that do not exist were never written
        const unsigned long long valid = n_kt >= 64 ? ~0ull : (1ull << n_kt) - 1ull;
        seen &= valid;
        w.live = seen != 0 ? seen : 1ull;  // an item that sees nothing still walks one tile: its rows come out as zeros
        w.zero = zero & valid;
    }
    return true;
}

// Walks the key tiles of an item that are to be computed: j is the first live tile at or after `from`, or n_tiles.
// Only the mask-reading form leaves tiles out: for the others this is the identity at compile time.
template <bool kMask>
__device__ __forceinline__ int next_live(const WorkItem & w, int from) {
    if (!kMask || w.live == ~0ull) return from;
    const unsigned long long rest = from < 64 ? w.live >> from : 0ull;
    return rest ? from + __ffsll((long long) rest) - 1 : w.n_tiles;
}

// A counter modulo n with the parity of its turns: the slot and the barrier phase of tile number t are t % n and
// (t / n) & 1, kept by stepping instead of dividing (the roles' loop control is one dependent chain per tile, and a
// warp that runs it shares its scheduler with warps in their arithmetic).
struct Wheel {
    int      slot  = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void step(int n) {
        if (++slot == n) { slot = 0; phase ^= 1u; }
    }
};

// Score tiles (64 keys) of key tile j that an item walks: the second is left out when no row of the item can see a key
// of it (the diagonal tile of a causal item; the last tile of a key sequence that ends in its first half).
__device__ __forceinline__ int sub_tiles(const PrefillParams & p, const WorkItem & w, int j) {
    const int last_key = min(min(w.q0 + p.tok, p.n_q) - 1 + p.causal_offset, p.n_kv - 1);
    return last_key - j * kKeys >= kSub ? 2 : 1;
}

// kSplitP: the weights go to the tensor core as hi + lo (two f16 parts, ~21 bits) instead of one f16 (11 bits).
// kVLo: K and V come as two f16 tiles each, value + remainder (q8_0 blocks expanded exactly), and Q is kept as value +
// remainder too (the reference's accurate path for such operands keeps Q in f32); the remainders take a second and
// third Q.K^T pass and a third P.V pass.
// kMask: an additive f16 mask is read instead of implying the causal one; every key tile is walked, a row may see no
// key at all (its output is zero, third_party/ggml/src/ggml-cpu/ops.cpp:8333).
template <bool kSplitP, bool kVLo, bool kMask>
__global__ void __launch_bounds__(kThreadsPf, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                  const __grid_constant__ CUtensorMap map_klo, const __grid_constant__ CUtensorMap map_vlo,
                  const __grid_constant__ CUtensorMap map_o, const __grid_constant__ CUtensorMap map_q, const PrefillParams p) {
    constexpr int kSt = stages_of(kVLo), kVBytes = v_stage_bytes(kVLo), kQBufBytes = q_buf_bytes(kVLo);
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[4 * kStages + 3 * kSBufs + kQBufs + 2 + kGroups + 1];
    __shared__ float    row_ref[kGroups][kTile];  // [score tile % groups][row]: the row's reference maximum after that tile, for the thread that takes the next one
    __shared__ uint32_t tmem_base_slot;
    __shared__ int      abort_flag;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *      smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sQ = smem_base, sK0 = sQ + kQBufs * kQBufBytes, sV0 = sK0 + kSt * kVBytes, sOnes = sV0 + kSt * kVBytes, sStage = sOnes + kOnesBytes,
                   sOut = sStage + kQStageBytes;  // 1024-byte aligned: every area before it is a multiple of 1024 bytes but the ones (2048)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // Barriers.  Per ring stage (key tile T uses stage T % kSt): K landed / K stage free, V landed / V stage free; the
    // producer is the only waiter of the two "free" ones.  Per score buffer (score tile U uses buffer U % 6): scores ready
    // (Q.K^T retired), weights ready (one arrival per warp of the softmax group that took the tile), buffer free (P.V
    // retired: the weights have been used and the accumulators are at rest).  A barrier of buffer b completes once per
    // score tile of that buffer, and each of the three events of tile U + 6 needs the one its waiter is looking for in
    // tile U to have been seen, so no barrier can complete twice between two looks of a waiter (a parity wait cannot
    // tell two completed phases from none).  Per item: Q in place (one per Q buffer), output complete, output read.
    // Per score tile parity: the rows' reference maxima after the tile, published by the softmax group that took it for
    // the group that takes the next.
    const uint32_t kfull0 = smem_u32(&bars[0]), kempty0 = kfull0 + 8 * kStages, vfull0 = kempty0 + 8 * kStages,
                   vempty0 = vfull0 + 8 * kStages, bS0 = vempty0 + 8 * kStages, bP0 = bS0 + 8 * kSBufs, bF0 = bP0 + 8 * kSBufs,
                   bQ0 = bF0 + 8 * kSBufs, bO = bQ0 + 8 * kQBufs, bOfree = bO + 8, bM0 = bOfree + 8,
                   bQS = bM0 + 8 * kGroups;  // the raw rows of a Q tile have landed in the staging area
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(kfull0 + 8 * s, 1);
            mbar_init(kempty0 + 8 * s, 1);
            mbar_init(vfull0 + 8 * s, 1);
            mbar_init(vempty0 + 8 * s, 1);
        }
        for (int s = 0; s < kSBufs; ++s) {
            mbar_init(bS0 + 8 * s, 1);
            mbar_init(bP0 + 8 * s, 4);  // one arrival per softmax warp of the group that took the tile
            mbar_init(bF0 + 8 * s, 1);
        }
        for (int s = 0; s < kQBufs; ++s) mbar_init(bQ0 + 8 * s, kIoThreads / 32);  // one arrival per in/out warp
        mbar_init(bO, 1);
        mbar_init(bOfree, kIoThreads / 32);
        for (int s = 0; s < kGroups; ++s) mbar_init(bM0 + 8 * s, 4);  // the rows' references after a score tile published (tile U uses U % kGroups)
        mbar_init(bQS, 1);
        fence_mbar_init();
    }
    if (warp == 5) tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    if (tid == 128) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
        if (!kVLo) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_o)) : "memory");
        if (!kVLo) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
        if (kVLo) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_klo)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_vlo)) : "memory");
        }
    }
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
    // Looked at once per item, not per tile (a shared-memory load in a role's loop control waits behind the role's own
    // TMEM stores and barrier operations: it measured 380 clocks per tile in the softmax warps).  A role that another
    // role's give-up leaves waiting inside an item runs into its own bounded wait.
    auto aborted = [&]() { return *reinterpret_cast<volatile int *>(&abort_flag) != 0; };
    // the same for a whole warp that must stay together: every lane takes the same way out
    auto warp_aborted = [&]() { return __any_sync(0xffffffffu, aborted()) != 0; };
    auto warp_wait    = [&](uint32_t bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity)) != 0; };

    // The CTA is persistent: every role walks the same item sequence; T counts key tiles over all items
    // and fixes the phase of every per-tile barrier; `round` fixes the phase of the per-item ones.
    if (warp >= 12 && warp < 16) {
        // ------------------------------------------------------------------ in/out warps: Q tiles in, results out
        // One thread per query row, as in the softmax warps (warp 12+i may touch TMEM lanes 32i..32i+31).  They keep
        // the Q tiles of the next two items in shared memory and read each finished output out of TMEM, so that the
        // softmax warps go from the last tile of one item straight to the first tile of the next.
        regs_give<kRegsIo>();
        const int      row   = tid - 12 * 32;
        const uint32_t t_row = tmem + ((uint32_t) (32 * (warp & 3)) << 16);
        {
            const uint32_t one2 = 0x3C003C00u;
            for (int i = row; i < kOnesBytes / 16; i += kIoThreads)
                *reinterpret_cast<uint4 *>(smem_gen + (sOnes - smem_base) + i * 16) = make_uint4(one2, one2, one2, one2);
        }
        // this thread's Q row: f32 from memory, f16 into eight 16-byte chunks at their swizzled places
        auto load_q = [&](const WorkItem & w, int buf) {
            uint8_t * const q_dst = smem_gen + buf * kQBufBytes + row * 128;
            const int       qpos  = w.q0 + row / p.pack, head = w.head + row % p.pack;
            const float4 *  src   = reinterpret_cast<const float4 *>(p.q + (size_t) qpos * p.q_nb1 + (size_t) head * p.q_nb2 +
                                                                  (size_t) w.batch * p.q_nb3);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float4 qv[8];
#pragma unroll
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_PF_SKIP_IO)
                for (int i = 0; i < 8; ++i) qv[i] = make_float4(0.f, 0.f, 0.f, (float) (size_t) src * 0.f);
#else
                for (int i = 0; i < 8; ++i) qv[i] = qpos < p.n_q ? src[8 * h + i] : make_float4(0.f, 0.f, 0.f, 0.f);
#endif
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float    x[8] = {qv[2 * c].x, qv[2 * c].y, qv[2 * c].z, qv[2 * c].w, qv[2 * c + 1].x, qv[2 * c + 1].y, qv[2 * c + 1].z, qv[2 * c + 1].w};
                    uint32_t       hi[4], lo[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __half2 h2 = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
                        hi[i] = *reinterpret_cast<const uint32_t *>(&h2);
                        lo[i] = pack_half2(x[2 * i] - __low2float(h2), x[2 * i + 1] - __high2float(h2));
                    }
                    const int at = ((4 * h + c) ^ (row & 7)) << 4;
                    *reinterpret_cast<uint4 *>(q_dst + at) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    // what the rounding left over: a second tile, for operands whose reference path keeps Q in f32
                    if (kVLo) *reinterpret_cast<uint4 *>(q_dst + kQBytes + at) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bQ0 + 8 * buf);
        };
        // Without remainder tiles (kVLo) the raw rows travel through a staging area, asked for a whole item before they
        // are needed, so that a new Q tile costs the in/out warps a pass over shared memory instead of two round trips
        // to global memory between one item's output and the next.  Two bulk-tensor loads by one thread fill it (box =
        // 32 floats x the group's heads x the item's tokens: 128 rows of 128 bytes per half, in the 128-byte swizzle;
        // rows past n_q arrive as zeros).  The route to this kernel asks for 16-byte aligned Q rows and strides and a
        // 16-byte aligned output, which is all the two tensor maps need.
        constexpr bool  kStageQ   = !kVLo;
        constexpr bool  kTmaOut   = !kVLo;  // the same room holds the output staging tile
        uint8_t * const stage_tma = smem_gen + (sStage - smem_base) + row * 128;  // + half * 16 KB + swizzled chunk
        uint32_t        qs_phase  = 0;      // of the staging barrier
        bool            io_failed = false;  // set by all 128 threads together
        auto fetch_q = [&](const WorkItem & w) {
            named_bar_sync(1, kIoThreads);  // every thread has read the rows that were there
            if (row == 0) {
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_PF_SKIP_IO)
                mbar_arrive(bQS);
#else
                mbar_expect_tx(bQS, kQStageBytes);
                tma_load_5d(sStage, &map_q, bQS, 0, w.head, w.q0, w.batch, 0);
                tma_load_5d(sStage + kQStageBytes / 2, &map_q, bQS, 32, w.head, w.q0, w.batch, 0);
#endif
            }
        };
        auto convert_q = [&](const WorkItem &, int buf) {
            const bool got = mbar_wait_bounded(bQS, qs_phase);
            qs_phase ^= 1u;
            if (!named_bar_all(1, kIoThreads, got)) { give_up(); io_failed = true; return; }
            uint8_t * const q_dst = smem_gen + buf * kQBufBytes + row * 128;
            // chunk k (of 16) of this thread's raw row
            auto raw = [&](int k) {
                return *reinterpret_cast<const float4 *>(stage_tma + (k >> 3) * (kQStageBytes / 2) + (((k & 7) ^ (row & 7)) << 4));
            };
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 a = raw(8 * h + 2 * c), b = raw(8 * h + 2 * c + 1);
                    const int at = ((4 * h + c) ^ (row & 7)) << 4;
                    *reinterpret_cast<uint4 *>(q_dst + at) = make_uint4(pack_half2(a.x, a.y), pack_half2(a.z, a.w), pack_half2(b.x, b.y), pack_half2(b.z, b.w));
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bQ0 + 8 * buf);
        };
        WorkItem w, wn;
        for (int r = 0; r < kQBufs && !io_failed; ++r)
            if (work_item<kMask>(p, r, wn)) {
                if (kStageQ) { fetch_q(wn); convert_q(wn, r); }
                else load_q(wn, r);
            }
        if (kStageQ && !io_failed && work_item<kMask>(p, kQBufs, wn)) fetch_q(wn);
        for (int round = 0; !io_failed && work_item<kMask>(p, round, w); ++round) {
            // one decision for the 128 threads (they meet at barriers below): go on only if nobody has given up and
            // every thread has seen the item's output complete
            const bool seen = !aborted() && mbar_wait_bounded(bO, round & 1);
            if (!named_bar_all(1, kIoThreads, seen)) { give_up(); break; }
            tc_fence_after();
            const int   qpos = w.q0 + row / p.pack, head = w.head + row % p.pack;
#if defined(VOX_ATTN_DEVELOPER) && (defined(VOX_PF_SKIP_IO) || defined(VOX_PF_SKIP_STORE))
            const bool  live = qpos < 0;
#else
            const bool  live = qpos < p.n_q;
#endif
            const float l    = tmem_ld1(t_row + kOCol + kHeadDim);  // sum of exactly the rounded weights the tensor core used
            const float inv  = l > 0.0f ? 1.0f / l : 0.0f;
            if (kTmaOut) {
                // The row goes into the output staging tile, and two bulk-tensor stores (one per 128-byte half of the
                // rows) carry the tile to its place: box = 32 floats x the group's heads x the item's tokens, so rows
                // past n_q are clipped by the copy.  A thread per row writing 256 contiguous bytes of global memory
                // touched 32 lines per store instruction; measured with the stores left out, they cost 2 us per layer
                // at 512 tokens x 8 and 1.1 us at 512 x 1.
                uint8_t * const out_row = smem_gen + (sOut - smem_base) + row * 128;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t r[32];
                    tmem_ld32_sync(t_row + kOCol + 32 * h, r);
                    if (h == 0) {
                        // the stores of the item before have read the staging tile
                        if (row == 0 && round > 0) bulk_wait_read();
                        named_bar_sync(1, kIoThreads);
                    } else {  // both halves are in registers: the columns go back to the tensor core
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bOfree);
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *reinterpret_cast<float4 *>(out_row + h * (kOutStageBytes / 2) + ((c ^ (row & 7)) << 4)) =
                            make_float4(__uint_as_float(r[4 * c]) * inv, __uint_as_float(r[4 * c + 1]) * inv,
                                        __uint_as_float(r[4 * c + 2]) * inv, __uint_as_float(r[4 * c + 3]) * inv);
                }
                fence_proxy_async_smem();
                named_bar_sync(1, kIoThreads);
#if !(defined(VOX_ATTN_DEVELOPER) && (defined(VOX_PF_SKIP_IO) || defined(VOX_PF_SKIP_STORE)))
                if (row == 0) {
                    tma_store_5d(&map_o, sOut, 0, w.head, w.q0, w.batch, 0);
                    tma_store_5d(&map_o, sOut + kOutStageBytes / 2, 32, w.head, w.q0, w.batch, 0);
                    bulk_commit();
                }
#endif
            } else {
                float4 * out = reinterpret_cast<float4 *>(p.dst + (((size_t) w.batch * p.n_q + qpos) * p.n_heads + head) * kHeadDim);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t r[32];
                    tmem_ld32_sync(t_row + kOCol + 32 * h, r);
                    if (h == 1) {  // both halves are in registers: the columns go back to the tensor core
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bOfree);
                    }
                    if (live) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            out[8 * h + i] = make_float4(__uint_as_float(r[4 * i]) * inv, __uint_as_float(r[4 * i + 1]) * inv,
                                                         __uint_as_float(r[4 * i + 2]) * inv, __uint_as_float(r[4 * i + 3]) * inv);
                    }
                }
            }
            // The item's output is complete only after its last P.V, which needed its last weights, which needed its last
            // scores: every Q.K^T of this item has retired, and its Q buffer takes the item after next.
            if (work_item<kMask>(p, round + kQBufs, wn)) {
                if (kStageQ) {
                    convert_q(wn, round % kQBufs);  // its rows were asked for an item ago
                    if (!io_failed && work_item<kMask>(p, round + kQBufs + 1, wn)) fetch_q(wn);
                } else {
                    load_q(wn, round % kQBufs);
                }
            }
        }
        // the last stores have been performed (waiting only until they have read the staging tile measured the same)
        if (kTmaOut && row == 0) bulk_wait_all();
    } else if (warp >= 4 && warp < 8) {
        regs_give<kRegsControl>();
        if (warp == 4) {
            // -------------------------------------------------------------- producer
            if (lane == 0) {
                WorkItem w;
                int      T  = 0;
                Wheel    tw;
                bool     ok = true;
                PROF_VARS;
                PROF_START();
                for (int round = 0; ok && work_item<kMask>(p, round, w); ++round) {
                    const int kvh = w.head / p.gqa;
                    for (int j = next_live<kMask>(w, 0); j < w.n_tiles; j = next_live<kMask>(w, j + 1), ++T, tw.step(kSt)) {
                        const int      st = tw.slot;
                        const uint32_t ph = tw.phase ^ 1u;  // the stage's previous turn
                        PROF_STOP(0);
                        if (T >= kSt && !mbar_wait_bounded(kempty0 + 8 * st, ph)) { ok = false; break; }
                        PROF_STOP(1);
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_PF_SKIP_LOAD)
                        if (T >= kSt && !mbar_wait_bounded(vempty0 + 8 * st, ph)) { ok = false; break; }
                        mbar_arrive(kfull0 + 8 * st);
                        mbar_arrive(vfull0 + 8 * st);
                        continue;
#endif
                        mbar_expect_tx(kfull0 + 8 * st, kVBytes);
                        tma_load_5d(sK0 + st * kVBytes, &map_k, kfull0 + 8 * st, 0, j * kKeys, kvh, w.batch, 0);
                        if (kVLo) tma_load_5d(sK0 + st * kVBytes + kKvBytes, &map_klo, kfull0 + 8 * st, 0, j * kKeys, kvh, w.batch, 0);
                        PROF_STOP(0);
                        if (T >= kSt && !mbar_wait_bounded(vempty0 + 8 * st, ph)) { ok = false; break; }
                        PROF_STOP(2);
                        mbar_expect_tx(vfull0 + 8 * st, kVBytes);
                        tma_load_5d(sV0 + st * kVBytes, &map_v, vfull0 + 8 * st, 0, j * kKeys, kvh, w.batch, 0);
                        if (kVLo) tma_load_5d(sV0 + st * kVBytes + kKvBytes, &map_vlo, vfull0 + 8 * st, 0, j * kKeys, kvh, w.batch, 0);
                    }
                    if (aborted()) break;
                }
                if (!ok) give_up();
                PROF_STOP(0);
                PROF_FLUSH(0, 3);  // 0 issue, 1 wait K stage free, 2 wait V stage free
            }
        } else if (warp == 6) {
            // -------------------------------------------------------------- score issuer: S = Q.K^T
            // The whole warp walks the item sequence and waits on the barriers; one elected lane issues.  With the loop
            // in warp-uniform control flow the descriptors and TMEM addresses live in uniform registers, which is where
            // tcgen05.mma takes them from: issued from inside a one-lane branch every instruction first had its operands
            // moved over, and cost its thread some 80 clocks.  Every exit from the loops is taken by all lanes together
            // (votes on the waits' results and on the abort flag).  The warp runs up to three tiles ahead of P.V, across
            // item boundaries.  S of global tile Tq goes into score buffer Tq % 3: four k-steps of 16 along head_dim
            // (32 bytes each inside the swizzle atom), N = 128 keys.  The buffer last held the weights of tile Tq-3,
            // which P.V of that tile reads: its retirement is awaited first.
            {
                constexpr uint32_t idesc_qk = idesc_f16(kSub, false);
                const uint64_t     dQ = smem_desc_sw128(sQ), dK = smem_desc_sw128(sK0), dKlo = smem_desc_sw128(sK0 + kKvBytes);
                constexpr uint64_t kStepQK = 32 >> 4;          // 16 of head_dim inside the swizzle atom
                constexpr uint64_t kStage  = kVBytes >> 4;     // K stages are as large as V stages
                constexpr uint64_t kQBuf   = kQBufBytes >> 4;
                constexpr uint64_t kQLo    = kQBytes >> 4;     // from a Q tile to its remainder tile
                const bool leader = elect_one();
                constexpr uint64_t kSubK   = (kSub * 128) >> 4;  // from the first 64 keys of a K tile to the last
                WorkItem wq;
                int      Tk = 0, U = 0;  // key tiles and score tiles so far, over all items
                Wheel    tw, uw;         // their ring stage and score buffer
                bool     ok = true;
                PROF_VARS;
                PROF_START();
                for (int rq = 0; ok && work_item<kMask>(p, rq, wq); ++rq) {
                    PROF_STOP(0);
                    if (!warp_wait(bQ0 + 8 * (rq % kQBufs), (rq / kQBufs) & 1)) { ok = false; break; }  // the item's Q tile is in place
                    PROF_STOP(2);
                    const uint64_t dQi = dQ + (rq % kQBufs) * kQBuf;
                    for (int jq = next_live<kMask>(wq, 0); ok && jq < wq.n_tiles; jq = next_live<kMask>(wq, jq + 1), ++Tk, tw.step(kSt)) {
                        const int st = tw.slot, n_sub = sub_tiles(p, wq, jq);
                        PROF_STOP(0);
                        if (!warp_wait(kfull0 + 8 * st, tw.phase)) { ok = false; break; }
                        PROF_STOP(2);
                        for (int u = 0; u < n_sub; ++u, ++U, uw.step(kSBufs)) {
                            const int sb = uw.slot;
                            if (U >= kSBufs && !warp_wait(bF0 + 8 * sb, uw.phase ^ 1u)) { ok = false; break; }
                            PROF_STOP(1);
                            if (lane == 0) PROF_TRACE(4, U);
                            tc_fence_after();
                            const uint32_t dS  = tmem + kSCol + kSub * sb;
                            const uint64_t dKs = st * kStage + u * kSubK;
                            if (leader) {
#if !(defined(VOX_ATTN_DEVELOPER) && defined(VOX_PF_SKIP_QK))
#pragma unroll
                                for (int k = 0; k < 4; ++k) tc_mma_f16(dS, dQi + k * kStepQK, dK + dKs + k * kStepQK, idesc_qk, k > 0);
#endif
                                if (kVLo) {  // what rounding K to f16 left over
#pragma unroll
                                    for (int k = 0; k < 4; ++k) tc_mma_f16(dS, dQi + k * kStepQK, dKlo + dKs + k * kStepQK, idesc_qk, 1);
#pragma unroll
                                    for (int k = 0; k < 4; ++k)  // and what rounding Q to f16 left over
                                        tc_mma_f16(dS, dQi + kQLo + k * kStepQK, dK + dKs + k * kStepQK, idesc_qk, 1);
                                }
                                tc_commit(bS0 + 8 * sb);                          // Q.K^T has retired: the scores are there ...
                                if (u == n_sub - 1) tc_commit(kempty0 + 8 * st);  // ... and the K stage may be refilled
                            }
                            __syncwarp();
                            if (lane == 0) PROF_TRACE(5, U);
                            PROF_STOP(0);
                        }
                    }
                    if (!ok || warp_aborted()) break;
                }
                if (!ok) give_up();
                PROF_STOP(0);
                if (lane == 0) PROF_FLUSH(21, 3);  // 21 issue, 22 wait for the score buffer, 23 wait Q / K tile
            }
        } else if (warp == 5) {
            // -------------------------------------------------------------- output issuer: O += P.V, row sums += P.1
            // (whole warp in the loop, one elected lane issues: see the score issuer)
            {
                constexpr uint32_t idesc_pv = idesc_f16(kHeadDim + 16, true);
                // Descriptors are built once; a k-step or a ring stage is selected by adding its distance to the address
                // field, and the same distance comes off the leading byte offset, which then still points at the tile of ones.
                const uint64_t     dV = smem_desc_sw128_mn(sV0, sOnes - sV0);
                constexpr uint64_t kStepV   = 2048 >> 4;  // 16 keys
                constexpr uint64_t kStepVPv = kStepV - (kStepV << 16);
                constexpr uint64_t kVStep   = kVBytes >> 4;
                constexpr uint64_t kVStage  = kVStep - (kVStep << 16);
                // the remainder tile of a V stage: 64 columns, no tile of ones behind it
                const uint64_t     dVlo     = smem_desc_sw128_mn(sV0 + kKvBytes, 16);
                constexpr uint32_t idesc_lo = idesc_f16(kHeadDim, true);
                const bool leader = elect_one();
                PROF_VARS;
                WorkItem w;
                int      Tk = 0, U = 0;
                Wheel    tw, uw;
                bool     ok = true;
                PROF_START();
                for (int round = 0; ok && work_item<kMask>(p, round, w); ++round) {
                    const int j_first = next_live<kMask>(w, 0);
                    bool      first   = true;  // the item's first score tile: O is overwritten, not added to
                    for (int j = j_first; ok && j < w.n_tiles; ++Tk, tw.step(kSt)) {
                        const int st = tw.slot, n_sub = sub_tiles(p, w, j);
                        const int j_next = next_live<kMask>(w, j + 1);
                        PROF_STOP(0);
                        if (!warp_wait(vfull0 + 8 * st, tw.phase)) { ok = false; break; }
                        PROF_STOP(3);
                        const uint64_t dVs = dV + st * kVStage;
                        for (int u = 0; u < n_sub; ++u, ++U, uw.step(kSBufs)) {
                            const int sb = uw.slot;
                            if (lane == 0) PROF_TRACE(14, U);
                            if (!warp_wait(bP0 + 8 * sb, uw.phase)) { ok = false; break; }
                            PROF_STOP(4);
                            // the previous item's result has been read out of TMEM: its columns may be overwritten
                            if (first && round > 0 && !warp_wait(bOfree, (round - 1) & 1)) { ok = false; break; }
                            PROF_STOP(2);
                            if (lane == 0) PROF_TRACE(2, U);
                            tc_fence_after();
                            if (lane == 0) PROF_TRACE(15, U);
                            // O += P V and row sums += P 1 in one instruction per 16 keys: N = 80, columns 64-79 of the B
                            // operand are the tile of ones.  P: 8 TMEM columns of packed weights per k-step, the high parts
                            // in the first half of the score buffer, the low parts in the second half.
                            const uint32_t tP = tmem + kSCol + kSub * sb;
                            if (leader) {
#if !(defined(VOX_ATTN_DEVELOPER) && defined(VOX_PF_SKIP_PV))
#pragma unroll
                                for (int k = 0; k < kSub / 16; ++k)
                                    tc_mma_f16_ts(tmem + kOCol, tP + 8 * k, dVs + (4 * u + k) * kStepVPv, idesc_pv, !first || k > 0);
#endif
                                if (kSplitP && !(VOX_PF_SKIP_PV_LO)) {
#pragma unroll
                                    for (int k = 0; k < kSub / 16; ++k)
                                        tc_mma_f16_ts(tmem + kOCol, tP + kSub / 2 + 8 * k, dVs + (4 * u + k) * kStepVPv, idesc_pv, 1);
                                }
                                if (kVLo) {  // what rounding V to f16 left over, against the high parts of the weights
#pragma unroll
                                    for (int k = 0; k < kSub / 16; ++k)
                                        tc_mma_f16_ts(tmem + kOCol, tP + 8 * k, dVlo + st * kVStep + (4 * u + k) * kStepV, idesc_lo, 1);
                                }
                                PROF_TRACE(16, U);
                                tc_commit(bF0 + 8 * sb);  // P.V has retired: the score buffer may be reused, the accumulators are at rest ...
                                if (u == n_sub - 1) {
                                    tc_commit(vempty0 + 8 * st);                // ... the V stage may be refilled ...
                                    if (j_next >= w.n_tiles) tc_commit(bO);     // ... and the item's output is complete
                                }
                                PROF_TRACE(17, U);
                            }
                            __syncwarp();
                            if (lane == 0) PROF_TRACE(3, U);
                            first = false;
                            PROF_STOP(0);
                        }
                        j = j_next;
                    }
                    if (!ok || warp_aborted()) break;
                }
                if (!ok) give_up();
                PROF_STOP(0);
                if (lane == 0) PROF_FLUSH(4, 5);  // 4 issue, 6 wait output read, 7 wait V tile, 8 wait P
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps: one thread per query row
        // A key tile is scored and weighted as two score tiles of 64 keys; warps 0-3 take the even score tiles (global
        // count U), warps 8-11 the odd ones (a warp may touch the TMEM lanes of its quarter, warp % 4, so warps w and
        // w + 8 share rows).  The two groups are half a step apart, so each scheduler has one warp in its exponentials
        // (the special-function unit delivers 16 per clock: 1024 clocks for 128 x 128 weights) while the other waits
        // for scores, loads them or stores weights.  Six score buffers of 64 columns instead of three of 128: a buffer
        // is held from Q.K^T until P.V has retired, several times longer than the softmax works on it, and the number
        // of buffers over that time is what bounds the rate of tiles.
        regs_take<kRegsSoftmax>();
        const int      mine  = warp < 4 ? 0 : warp < 12 ? 1 : 2;             // this warpgroup takes the score tiles U % kGroups == mine
        const int      row   = 32 * (warp & 3) + lane;                       // == TMEM lane
        const uint32_t t_row = tmem + ((uint32_t) (32 * (warp & 3)) << 16);  // this warp's lane quarter

        WorkItem w;
        int      U  = 0;
        Wheel    uw;  // the score buffer of tile U and the phase of its barriers
        bool     ok = true;
        PROF_VARS;
        PROF_START();
        for (int round = 0; ok && work_item<kMask>(p, round, w); ++round) {
            const int  qpos  = w.q0 + row / p.pack;
            const int  limit = min(qpos + p.causal_offset, p.n_kv - 1);  // last key this row may see
            // The output row and the row sum accumulate in TMEM across all key tiles, both scaled by
            // 2^(-m_ref): their ratio does not depend on m_ref, so the reference maximum only has to keep
            // the weights inside f16 range.  It is raised (and the accumulated columns rescaled) only when a
            // tile's maximum exceeds it by more than 2^8, which after the first tile is rare.  The reference of a
            // row passes from the thread of score tile U to the thread of tile U + 1 through shared memory (row_ref).
            // this row of the mask (rows past n_q are computed on zeros and not stored: they borrow the last row)
            const uint8_t * mrow = nullptr;
            if (kMask)
                mrow = p.mask + (size_t) min(qpos, p.n_q - 1) * p.m_nb1 + (size_t) ((w.head + row % p.pack) % p.m_ne2) * p.m_nb2 +
                       (size_t) (w.batch % p.m_ne3) * p.m_nb3;
            bool  first = true;  // the item's first score tile sets the reference
            // last key every row of the item sees, and the key tile that holds it
            const int uncut = min(w.q0 + p.causal_offset, p.n_kv - 1), cut_from = uncut / kKeys;
            for (int j = next_live<kMask>(w, 0); ok && j < w.n_tiles; j = next_live<kMask>(w, j + 1)) {
                const int n_sub = sub_tiles(p, w, j);
                for (int u = 0; u < n_sub; ++u, ++U, uw.step(kSBufs)) {
                    const bool is_first = first;
                    first = false;
                    if (U % kGroups != mine && (warp & 3) == 0 && lane == 0) PROF_TRACE(12, U);  // loop top at the other group's tile
                    if (U % kGroups != mine) continue;  // another group's tile
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(13, U);
                    const int sb = uw.slot;
                    const int k0 = j * kKeys + kSub * u;  // the score tile's first key
                    // a key tile to which the mask adds nothing for any row of the item (most tiles of a causal mask) is not read
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_PF_FORCE_MREAD)
                    const bool m_read = kMask;
#else
                    const bool m_read = kMask && !(j < 64 && ((w.zero >> j) & 1ull));
#endif
                    // the scores are multiplied by `mul` on their way into the exponent: where the mask is read they have
                    // been put into natural units (scale * S + mask) first
                    const float mul = m_read ? 1.4426950408889634f : p.scale_log2;
                    uint4     mv[8];
                    if (kMask && m_read) {  // requested before the wait for the scores; chunks of 8 keys lie wholly inside or outside n_kv
                        const uint4 * mp = reinterpret_cast<const uint4 *>(mrow + (size_t) k0 * 2);
#pragma unroll
                        for (int c = 0; c < 8; ++c) mv[c] = k0 + 8 * c < p.n_kv ? __ldg(mp + c) : make_uint4(0u, 0u, 0u, 0u);
                    }
                    PROF_STOP(0);
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(11, U);
                    if (!mbar_wait_bounded(bS0 + 8 * sb, uw.phase)) { ok = false; break; }
                    PROF_STOP(1);
                    PROF_COUNT(7, 1);
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(0, U);
                    tc_fence_after();
#if defined(VOX_ATTN_DEVELOPER) && defined(VOX_PREFILL_NOSOFTMAX)  // developer build: the copy and MMA structure alone
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bP0 + 8 * sb);
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(1, U);
                    continue;
#endif
                    const uint32_t t_s    = t_row + kSCol + kSub * sb;  // the tile's score buffer
                    // uniform over the group: the tile may be cut (no key tile before the one that holds `uncut` can be)
                    const bool     masked = j >= cut_from && k0 + kSub - 1 > uncut;
                    // (Loading only the 32-column blocks some row of the warp can see, on the tiles the diagonal cuts, was
                    // measured against always loading all 64 columns: the extra code in the loop cost more than the
                    // loads it saved.)
                    uint32_t       r[kSub];
                    tmem_ld64_sync(t_s, r);
                    PROF_STOP(10);
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(6, U);
                    if (kMask && m_read) {
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint32_t w4[4] = {mv[c].x, mv[c].y, mv[c].z, mv[c].w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 m2 = __half22float2(*reinterpret_cast<const __half2 *>(&w4[i]));
                                r[8 * c + 2 * i]     = __float_as_uint(fmaf(__uint_as_float(r[8 * c + 2 * i]), p.scale, m2.x));
                                r[8 * c + 2 * i + 1] = __float_as_uint(fmaf(__uint_as_float(r[8 * c + 2 * i + 1]), p.scale, m2.y));
                            }
                        }
                    }
                    if (masked) {  // only the tiles the causal diagonal or the end of the keys cuts through
#pragma unroll
                        for (int i = 0; i < kSub; ++i)
                            if (k0 + i > limit) r[i] = 0xff800000u;
                    }
                    float cmax;
                    {
                        float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
                        for (int i = 0; i < kSub; i += 4) {
                            t0 = max3(t0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                            t1 = max3(t1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                        }
                        cmax = fmaxf(t0, t1) * mul;
                    }
                    // The row's reference after score tile U - 1, from the thread of the other group that took that
                    // tile.  The wait is made for every tile but the very first, also where the value is not used (first
                    // tile of an item): it keeps the two groups within one tile of each other, so that neither barrier
                    // can complete twice between two looks of its waiter, and a slot of row_ref is rewritten (tile U + 2)
                    // only after its reader (tile U + 1) has published in turn, which it does after reading.
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(7, U);
                    if (U > 0 && !mbar_wait_bounded(bM0 + 8 * ((U - 1) % kGroups), ((U - 1) / kGroups) & 1)) { ok = false; break; }
                    PROF_STOP(11);
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(8, U);
                    // The weights are written only after the whole tile has been looked at, so a raise of the
                    // reference needs no second pass.  tcgen05.ld/st are warp-collective: the decision to rescale is
                    // taken per warp (any lane), and lanes that do not need it take part with a factor of 1.
                    // With a mask a row may have seen no key yet: its reference stays -inf (any finite maximum then
                    // raises it, with a factor of 0 for accumulators that hold 0) and its weights are 2^(-inf - 0) = 0.
                    float m_ref;
                    if (is_first) {
                        m_ref = cmax;  // without a mask key 0 is visible to every row: finite
                    } else {
                        m_ref = row_ref[(U - 1) % kGroups][row];
                        const bool raise = cmax > m_ref + 8.0f;
                        if (__any_sync(0xffffffffu, raise)) {
                            const float f = raise ? ex2_approx(m_ref - cmax) : 1.0f;
                            if (raise) m_ref = cmax;
                            // the accumulators are at rest once P.V of the previous score tile has retired
                            if (!mbar_wait_bounded(bF0 + 8 * ((U - 1) % kSBufs), ((U - 1) / kSBufs) & 1)) { ok = false; break; }
                            rescale_accumulators(t_row, f);
                        }
                    }
                    if (kPublishAt == 0 || !kSplitP) {
                        row_ref[U % kGroups][row] = m_ref;
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bM0 + 8 * (U % kGroups));
                    }
                    const float m_sub = kMask && m_ref == -INFINITY ? 0.0f : m_ref;
                    // P = 2^(c*S - m_ref), 16 keys (8 columns of packed f16 pairs) at a time: k-step g of the score tile.
                    if (kSplitP) {
                        // hi + lo: two packed f16 tiles (hi: columns 0-31 of the buffer, lo: columns 32-63).  hi keeps the
                        // top 11 bits of the f32 weight (a mask: exact in f16 for every weight above 2^-14, and the weights
                        // that matter are >= 1 for the row's largest), lo is the exact remainder rounded to f16: together
                        // ~21 bits, so that the result does not depend on how the rounding errors of a few large weights
                        // happen to fall against the spread of V.  The thread holds every score of its row in registers,
                        // so the weights may overwrite the buffer in any order.
#pragma unroll
                        for (int g = 0; g < kSub / 16; ++g) {
                            uint32_t hi[8], lo[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float p0 = ex2_approx(fmaf(__uint_as_float(r[16 * g + 2 * i]), mul, -m_sub));
                                const float p1 = ex2_approx(fmaf(__uint_as_float(r[16 * g + 2 * i + 1]), mul, -m_sub));
                                const float h0 = __uint_as_float(__float_as_uint(p0) & 0xFFFFE000u);
                                const float h1 = __uint_as_float(__float_as_uint(p1) & 0xFFFFE000u);
                                hi[i] = pack_half2(h0, h1);
                                lo[i] = pack_half2(p0 - h0, p1 - h1);
                            }
                            tmem_st8_nowait(t_s + 8 * g, hi);
                            tmem_st8_nowait(t_s + kSub / 2 + 8 * g, lo);
                            if (g + 1 == kPublishAt) {  // see kPublishAt
                                row_ref[U % kGroups][row] = m_ref;
                                __syncwarp();
                                if (lane == 0) mbar_arrive(bM0 + 8 * (U % kGroups));
                            }
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < kSub / 16; ++g) {
                            uint32_t h[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                h[i] = pack_half2(ex2_approx(fmaf(__uint_as_float(r[16 * g + 2 * i]), mul, -m_sub)),
                                                  ex2_approx(fmaf(__uint_as_float(r[16 * g + 2 * i + 1]), mul, -m_sub)));
                            tmem_st8_nowait(t_s + 8 * g, h);
                        }
                    }
                    PROF_STOP(2);
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(9, U);
                    tmem_wait_st();
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(10, U);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bP0 + 8 * sb);  // this warp's rows of P are in TMEM
                    if ((warp & 3) == 0 && lane == 0) PROF_TRACE(1, U);
                    if (lane == 0) PROF_TRACE(18 + (warp & 3), U);  // every warp of the group
                    PROF_STOP(3);
                }
            }
            if (!ok) give_up();  // a wait of this thread ran out: raised once, here, to keep the tile loop short
            if (!ok || aborted()) break;
            PROF_COUNT(9, 1);
        }
        // 0 other, 1 wait S, 2 softmax blocks, 3 store wait + signal, 7 tiles, 9 items, 10 wait for the scores' load, 11 tile maximum + reference
        if (lane == 0 && mine == 0) PROF_FLUSH(9 + 0, 12);
    }

    // common exit: every role has left its loop; release TMEM
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// q8_0 K/V (34-byte blocks: f16 scale + 32 int8, third_party/ggml/src/ggml-common.h:221-224) and f32 K/V are expanded
// once per call into f16 tiles in the caller's workspace, [B][HK][n_kv][64] contiguous, and the tensor-core kernel
// runs on those.  One thread per 32 values; each value becomes an f16 and the f16 of what that rounding left over
// (exact for q8_0: d * q has at most 18 significant bits; 22 of 24 bits for f32).
struct DequantParams {
    const uint8_t * src[2];
    __half *        dst[2];
    __half *        rest[2];  // what rounding to f16 leaves over (exact: d * q has at most 18 significant bits)
    size_t          nb1[2], nb2[2], nb3[2];
    int             n_kv, n_kvh, n_batch;
    int             f32;  // source rows are 64 floats instead of two q8_0 blocks
};
__global__ void __launch_bounds__(256) q8_0_to_f16_kernel(const DequantParams p) {
    const long long n_blocks = 2LL * p.n_kv * p.n_kvh * p.n_batch;  // two blocks per 64-wide row
    const bool      is_v     = blockIdx.y != 0;                     // 0: K, 1: V
    const uint8_t * src      = is_v ? p.src[1] : p.src[0];
    __half *        dst      = is_v ? p.dst[1] : p.dst[0];
    const size_t    nb1 = is_v ? p.nb1[1] : p.nb1[0], nb2 = is_v ? p.nb2[1] : p.nb2[0], nb3 = is_v ? p.nb3[1] : p.nb3[0];
    for (long long i = (long long) blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks; i += (long long) gridDim.x * blockDim.x) {
        const int       blk = (int) (i & 1);
        const long long row = i >> 1;
        const int       pos = (int) (row % p.n_kv);
        const int       kvh = (int) ((row / p.n_kv) % p.n_kvh);
        const int       b   = (int) (row / ((long long) p.n_kv * p.n_kvh));
        const uint8_t * at = src + (size_t) pos * nb1 + (size_t) kvh * nb2 + (size_t) b * nb3;
        uint32_t        out[16], rest[16];
        if (p.f32) {
            const float4 * s = reinterpret_cast<const float4 *>(at + (size_t) blk * 128);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4  x  = s[j];
                const __half2 h0 = __floats2half2_rn(x.x, x.y), h1 = __floats2half2_rn(x.z, x.w);
                out[2 * j]      = *reinterpret_cast<const uint32_t *>(&h0);
                out[2 * j + 1]  = *reinterpret_cast<const uint32_t *>(&h1);
                rest[2 * j]     = pack_half2(x.x - __low2float(h0), x.y - __high2float(h0));
                rest[2 * j + 1] = pack_half2(x.z - __low2float(h1), x.w - __high2float(h1));
            }
        } else {
            const uint16_t * s = reinterpret_cast<const uint16_t *>(at + (size_t) blk * 34);
            const float      d = __half2float(__ushort_as_half(s[0]));
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint16_t two = s[1 + j];
                const float    x0 = d * (float) (signed char) (two & 0xff), x1 = d * (float) (signed char) (two >> 8);
                const __half2  h  = __floats2half2_rn(x0, x1);
                out[j]  = *reinterpret_cast<const uint32_t *>(&h);
                rest[j] = pack_half2(x0 - __low2float(h), x1 - __high2float(h));
            }
        }
        uint4 * o = reinterpret_cast<uint4 *>(dst + (size_t) row * 64 + (size_t) blk * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
        uint4 * r = reinterpret_cast<uint4 *>((is_v ? p.rest[1] : p.rest[0]) + (size_t) row * 64 + (size_t) blk * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = make_uint4(rest[4 * j], rest[4 * j + 1], rest[4 * j + 2], rest[4 * j + 3]);
    }
}

size_t q8_scratch_bytes(const vox_attn_args * a) {  // one tensor, rounded up so that the second one stays aligned
    const size_t bytes = (size_t) a->k.ne[1] * (size_t) a->k.ne[2] * (size_t) a->k.ne[3] * 128;
    return (bytes + 255) & ~(size_t) 255;
}

// K and V to expand: both q8_0 (whole blocks, rows at even addresses: the blocks are read as 16-bit words) or both
// f32 (rows read in 16-byte pieces), of equal shape
bool q8_route_ok(const vox_attn_args * a) {
    const vox_tensor &k = a->k, &v = a->v;
    if (k.type != v.type || (k.type != VOX_TYPE_Q8_0 && k.type != VOX_TYPE_F32)) return false;
    if (k.ne[1] != v.ne[1] || k.ne[2] != v.ne[2] || k.ne[3] != v.ne[3]) return false;
    if (a->q.ne[1] < 1 || k.ne[1] < 1) return false;
    if ((reinterpret_cast<uintptr_t>(a->q.data) & 15) != 0 || a->q.nb[1] % 16 || a->q.nb[2] % 16 || a->q.nb[3] % 16) return false;
    const uintptr_t unit = k.type == VOX_TYPE_F32 ? 16 : 2;
    for (const vox_tensor * t : {&k, &v})
        if (reinterpret_cast<uintptr_t>(t->data) % unit || t->nb[1] % unit || t->nb[2] % unit || t->nb[3] % unit) return false;
    if (k.type == VOX_TYPE_F32 && (k.nb[0] != 4 || v.nb[0] != 4)) return false;
    return true;
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

// Which key tiles of which query tiles the mask leaves anything of, and to which it adds nothing: per (mask plane, query
// tile) 64 flag bytes of each kind, byte j for keys 128j..128j+127.  The tensor-core kernel leaves the first kind's
// empty tiles out (with the reference's causal mask tensor that is half of them) and does not read the mask in the
// second kind's (all tiles below the diagonal).  Grid: (key tiles, query tiles, planes), one thread per row; every CTA
// writes its own two bytes, so nothing has to be cleared beforehand (words of bits set with atomics needed a memset
// node in front, and the two extra nodes per call cost a captured graph as much as the tiles they saved: 40 us per
// layer at 512 tokens x 8 with or without them).  Launched with programmatic dependency: it starts while the kernel
// before drains, reads the mask after that kernel has completed, and lets the tensor-core kernel's prologue start.
__global__ void __launch_bounds__(kTile) mask_tiles_kernel(const uint8_t * mask, size_t nb1, size_t nb2, size_t nb3, int ne2, int n_q,
                                                           int n_kv, int tok, uint8_t * live, uint8_t * zero) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.y * tok + threadIdx.x, k0 = blockIdx.x * kKeys;  // a query tile holds `tok` tokens
    const int i2 = blockIdx.z % ne2, i3 = blockIdx.z / ne2;
    int       any = 0, nonzero = 0;
    if (threadIdx.x < tok && row < n_q) {
        const uint4 * m = reinterpret_cast<const uint4 *>(mask + (size_t) row * nb1 + (size_t) i2 * nb2 + (size_t) i3 * nb3 + (size_t) k0 * 2);
#pragma unroll
        for (int c = 0; c < kKeys / 8; ++c) {
            if (k0 + 8 * c < n_kv) {  // n_kv is a multiple of 8: a piece lies wholly inside or outside
                const uint4    x    = __ldg(m + c);
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) any |= (w[i] & 0xffffu) != 0xfc00u || (w[i] >> 16) != 0xfc00u;
#pragma unroll
                for (int i = 0; i < 4; ++i) nonzero |= (w[i] & 0x7fff7fffu) != 0u;  // anything but +0 or -0
            }
        }
    }
    const int any_all = __syncthreads_or(any), nonzero_all = __syncthreads_or(nonzero);
    if (threadIdx.x == 0) {
        const size_t at = ((size_t) blockIdx.z * gridDim.y + blockIdx.y) * 64 + blockIdx.x;
        live[at] = any_all ? 1 : 0;
        zero[at] = nonzero_all ? 0 : 1;
    }
}

// query heads of one kv head that share an item's 128 rows: the largest of 8, 4, 2, 1 that divides the GQA ratio
int pack_of(const vox_attn_args * a) {
    const long long gqa = a->k.ne[2] > 0 ? a->q.ne[2] / a->k.ne[2] : 1;
    for (int pk = 8; pk > 1; pk >>= 1)
        if (gqa % pk == 0) return pk;
    return 1;
}
long long query_tiles_of(const vox_attn_args * a) {
    const int tok = kTile / pack_of(a);
    return (a->q.ne[1] + tok - 1) / tok;
}

#ifndef VOX_PREFILL_MASK_PREPASS_TILES
#define VOX_PREFILL_MASK_PREPASS_TILES 2048
#endif
constexpr long long kMaskPrepassTiles = VOX_PREFILL_MASK_PREPASS_TILES;  // see run_tc

// bytes of those flags, the "something visible" array and the "adds nothing" array behind it (0 when there are more
// than 64 key tiles: then every tile is walked and read)
size_t mask_tiles_bytes(const vox_attn_args * a) {
    const long long n_ktiles = (a->k.ne[1] + kKeys - 1) / kKeys, n_qtiles = query_tiles_of(a);
    if (a->mask.data == nullptr || n_ktiles > 64) return 0;
    return 2 * (((size_t) (a->mask.ne[2] * a->mask.ne[3] * n_qtiles * 64) + 255) & ~(size_t) 255);
}

// Host side of the tensor-core kernel: `with_mask` false implies the causal mask at `offset` (n_kv - n_q) or, with
// `causal` false, no mask at all; true reads a->mask.  q8_0 K/V are expanded into the workspace first; operands the kernel cannot take go to the general kernel.
int run_tc(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t st, bool with_mask,
           bool causal = true) {
    // every key visible (before the mask, if there is one) is a causal offset of n_kv
    const int offset = with_mask || !causal ? (int) a->k.ne[1] : (int) (a->k.ne[1] - a->q.ne[1]);
    // workspace: the live-tile words of the mask first (when it has room for them), then the expanded K/V
    const uint8_t * tile_live = nullptr, * tile_zero = nullptr;
    if (with_mask && workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0) {
        const size_t words = mask_tiles_bytes(a);
        const size_t rest  = q8_route_ok(a) ? 4 * q8_scratch_bytes(a) : 0;
        // worth its launch from a few thousand tiles on (512 tokens x 1 sequence is 512 tiles: not worth it)
        const long long tiles = ((a->k.ne[1] + kKeys - 1) / kKeys) * query_tiles_of(a) * (a->q.ne[2] / pack_of(a)) * a->q.ne[3];
        if (words > 0 && workspace_bytes >= words + rest && tiles >= kMaskPrepassTiles) {
            uint8_t * live = static_cast<uint8_t *>(workspace);
            const dim3 grid((unsigned) ((a->k.ne[1] + kKeys - 1) / kKeys), (unsigned) query_tiles_of(a),
                            (unsigned) (a->mask.ne[2] * a->mask.ne[3]));
            launch_pdl(mask_tiles_kernel, grid, dim3(kTile), 0, st, static_cast<const uint8_t *>(a->mask.data), a->mask.nb[1], a->mask.nb[2],
                       a->mask.nb[3], (int) a->mask.ne[2], (int) a->q.ne[1], (int) a->k.ne[1], kTile / pack_of(a), live, live + words / 2);
            int rc = check_launch(e, "mask_tiles_kernel");
            if (rc != VOX_ATTN_OK) return rc;
            tile_live       = live;
            tile_zero       = live + words / 2;
            workspace       = static_cast<uint8_t *>(workspace) + words;
            workspace_bytes -= words;
        }
    }
    // q8_0 K/V: expanded to f16 in the workspace first (without one of the size vox_attn_prefill_workspace_bytes
    // names, the general kernel takes the call, as it does for f32 K/V and unaligned strides)
    vox_tensor kf = a->k, vf = a->v;
    bool       v_lo = false;
    __half *   lo_data[2] = {nullptr, nullptr};
    if (q8_route_ok(a) && workspace != nullptr && workspace_bytes >= 4 * q8_scratch_bytes(a) &&
        (reinterpret_cast<uintptr_t>(workspace) & 15) == 0) {
        DequantParams dp;
        const size_t  one = q8_scratch_bytes(a);
        vox_tensor *  fs[2] = {&kf, &vf};
        const vox_tensor * qs[2] = {&a->k, &a->v};
        for (int i = 0; i < 2; ++i) {
            dp.src[i] = static_cast<const uint8_t *>(qs[i]->data);
            dp.dst[i] = reinterpret_cast<__half *>(static_cast<uint8_t *>(workspace) + i * one);
            dp.nb1[i] = qs[i]->nb[1]; dp.nb2[i] = qs[i]->nb[2]; dp.nb3[i] = qs[i]->nb[3];
            fs[i]->type  = VOX_TYPE_F16;
            fs[i]->data  = dp.dst[i];
            fs[i]->nb[0] = 2;
            fs[i]->nb[1] = 128;
            fs[i]->nb[2] = (size_t) a->k.ne[1] * 128;
            fs[i]->nb[3] = (size_t) a->k.ne[1] * (size_t) a->k.ne[2] * 128;
        }
        for (int i = 0; i < 2; ++i) dp.rest[i] = lo_data[i] = reinterpret_cast<__half *>(static_cast<uint8_t *>(workspace) + (2 + i) * one);
        v_lo = true;
        dp.n_kv = (int) a->k.ne[1]; dp.n_kvh = (int) a->k.ne[2]; dp.n_batch = (int) a->k.ne[3];
        dp.f32  = a->k.type == VOX_TYPE_F32;
        const long long n_blocks = 2LL * dp.n_kv * dp.n_kvh * dp.n_batch;
        const unsigned  gx = (unsigned) std::min<long long>((n_blocks + 255) / 256, 8LL * e->sm_count);
        q8_0_to_f16_kernel<<<dim3(gx, 2), 256, 0, st>>>(dp);
        int rc = check_launch(e, "q8_0_to_f16_kernel");
        if (rc != VOX_ATTN_OK) return rc;
    } else if (!tc_route_ok(a)) {
        return launch_generic(e, a, with_mask || !causal ? -1 : offset, st);
    }

    CUtensorMap    mk, mv, mklo, mvlo;
    const uint64_t dims[5] = {64, (uint64_t) a->k.ne[1], (uint64_t) a->k.ne[2], (uint64_t) a->k.ne[3], 1};
    const uint32_t box[5]  = {64, kKeys, 1, 1, 1};
    vox_tensor     kl = kf, vl = vf;  // the remainders: same shape and strides as the expanded tensors
    if (v_lo) { kl.data = lo_data[0]; vl.data = lo_data[1]; }
    const vox_tensor * ts[4] = {&kf, &vf, &kl, &vl};
    CUtensorMap *      ms[4] = {&mk, &mv, &mklo, &mvlo};
    for (int i = 0; i < (v_lo ? 4 : 2); ++i) {
        const uint64_t strides[4] = {ts[i]->nb[1], ts[i]->nb[2], ts[i]->nb[3],
                                     std::max<uint64_t>(ts[i]->nb[3] * (uint64_t) ts[i]->ne[3], 16)};
        int rc = make_tensor_map(e, ms[i], ts[i]->data, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != VOX_ATTN_OK) return rc;
    }
    if (!v_lo) { mklo = mk; mvlo = mv; }  // not read
    // Without remainder tiles in shared memory the raw Q rows come in and the results go out by bulk-tensor copies: Q as a
    // tensor map over (64 floats, heads, tokens, sequences) in whatever strides the caller's Q has, the output as
    // [batch][n_q][n_heads][64] f32; boxes of 32 floats x the heads of a group x the tokens of an item.  (With remainder
    // tiles the rows are fetched and stored by their threads and the two maps are not read.)
    CUtensorMap mq = mk, mo = mk;
    if (!v_lo) {
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(a->dst.data) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT, "dst must be 16-byte aligned");
        const uint32_t box[5] = {32, (uint32_t) pack_of(a), (uint32_t) (kTile / pack_of(a)), 1, 1};
        const uint64_t n_h = (uint64_t) a->q.ne[2], n_q = (uint64_t) a->q.ne[1], n_b = (uint64_t) a->q.ne[3], row_b = kHeadDim * 4;
        const uint64_t qd[5] = {kHeadDim, n_h, n_q, n_b, 1};
        const uint64_t qs[4] = {a->q.nb[2], a->q.nb[1], a->q.nb[3], std::max<uint64_t>(a->q.nb[3] * n_b, 16)};
        int rc = make_tensor_map(e, &mq, const_cast<void *>(a->q.data), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, qd, qs, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != VOX_ATTN_OK) return rc;
        const uint64_t os[4] = {row_b, n_h * row_b, n_q * n_h * row_b, n_b * n_q * n_h * row_b};
        rc = make_tensor_map(e, &mo, a->dst.data, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, qd, os, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != VOX_ATTN_OK) return rc;
    }
    if (!(e->attr_mask & (1u << 12))) {
        VOX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel<true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pf(false)));
        VOX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel<false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pf(false)));
        VOX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel<true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pf(true)));
        VOX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel<true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pf(false)));
        VOX_CUDA_TRY(cudaFuncSetAttribute(prefill_tc_kernel<true, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pf(true)));
        e->attr_mask |= 1u << 12;
    }
    // Developer setting (VOX_PREFILL_WEIGHTS=f16 when the engine was created): the weights as one f16 part (faster; on
    // long sequences of random data the result then misses the 2e-3 parity bound: 2.6e-3 at 640 keys).  The product
    // path splits them.
    const bool   split_p     = e->prefill_single_f16 == 0;
    PrefillParams p;
    p.q = static_cast<const uint8_t *>(a->q.data);
    p.q_nb1 = a->q.nb[1]; p.q_nb2 = a->q.nb[2]; p.q_nb3 = a->q.nb[3];
    p.dst = static_cast<float *>(a->dst.data);
    p.n_q = (int) a->q.ne[1]; p.n_kv = (int) a->k.ne[1]; p.n_heads = (int) a->q.ne[2];
    p.gqa = (int) (a->q.ne[2] / a->k.ne[2]); p.causal_offset = offset;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.scale  = a->scale;
    p.status = e->status_dev;
    p.mask   = with_mask ? static_cast<const uint8_t *>(a->mask.data) : nullptr;
    p.m_nb1 = a->mask.nb[1]; p.m_nb2 = a->mask.nb[2]; p.m_nb3 = a->mask.nb[3];
    p.m_ne2 = with_mask ? (int) a->mask.ne[2] : 1; p.m_ne3 = with_mask ? (int) a->mask.ne[3] : 1;
    p.tile_live = tile_live;
    p.tile_zero = tile_zero;
    p.n_batch  = (int) a->q.ne[3];
    p.pack      = pack_of(a);
    p.tok       = kTile / p.pack;
    p.n_hgroups = p.n_heads / p.pack;
    p.n_qtiles  = (int) query_tiles_of(a);
    const long long items = (long long) p.n_qtiles * p.n_hgroups * p.n_batch;
    VOX_REQUIRE(items < (1LL << 30), VOX_ATTN_INVALID_ARGUMENT, "too many query tiles");
    p.n_items = (int) items;
    // persistent CTAs, one per SM (all 512 TMEM columns, 131 KB of shared memory; 195 KB when K/V were expanded and every
    // operand tile comes with its remainder tile)
    dim3 grid((unsigned) std::min<long long>(items, (long long) e->sm_count));
    if (with_mask && v_lo) launch_pdl(prefill_tc_kernel<true, true, true>, grid, dim3(kThreadsPf), smem_pf(true), st, mk, mv, mklo, mvlo, mo, mq, p);
    else if (with_mask) launch_pdl(prefill_tc_kernel<true, false, true>, grid, dim3(kThreadsPf), smem_pf(false), st, mk, mv, mklo, mvlo, mo, mq, p);
    else if (v_lo) launch_pdl(prefill_tc_kernel<true, true, false>, grid, dim3(kThreadsPf), smem_pf(true), st, mk, mv, mklo, mvlo, mo, mq, p);
    else if (split_p) launch_pdl(prefill_tc_kernel<true, false, false>, grid, dim3(kThreadsPf), smem_pf(false), st, mk, mv, mklo, mvlo, mo, mq, p);
    else launch_pdl(prefill_tc_kernel<false, false, false>, grid, dim3(kThreadsPf), smem_pf(false), st, mk, mv, mklo, mvlo, mo, mq, p);
    return check_launch(e, "prefill_tc_kernel");
}

}  // namespace

namespace vox {

// The general kernel spreads its work over (query, head) pairs only and walks the keys one after another: 276 us for
// 16 queries over 512 keys, 2.2 ms for 32 over 4096 (a chunk of a prompt against a long cache), where the tensor-core
// kernel, with most rows of its 128-row tile idle, takes 10.7 and 68.5 us.  So the general kernel keeps only the
// short-key problems (LocEnc's 5 tokens, LocDiT's 9 or 18).
constexpr int kMinKeys = 32;

// An explicit mask goes to the tensor-core kernel when there are enough keys, the
// mask rows can be read in 16-byte pieces that lie wholly inside or outside n_kv, and K/V are f16 (or q8_0).
bool prefill_mask_route_ok(const vox_attn_args * a) {
    const vox_tensor & m = a->mask;
    if (m.data == nullptr || a->q.ne[1] < 1 || a->k.ne[1] < kMinKeys || a->k.ne[1] % 8) return false;
    if ((reinterpret_cast<uintptr_t>(m.data) & 15) != 0 || m.nb[1] % 16 || m.nb[2] % 16 || m.nb[3] % 16) return false;
    return tc_route_ok(a) || q8_route_ok(a);
}
size_t prefill_mask_workspace_bytes(const vox_attn_args * a) {
    if (!prefill_mask_route_ok(a)) return 0;
    return mask_tiles_bytes(a) + (q8_route_ok(a) ? 4 * q8_scratch_bytes(a) : 0);
}
// what the route cannot do without: room for the expanded K/V (the live-tile words are optional)
size_t prefill_mask_workspace_min(const vox_attn_args * a) {
    return prefill_mask_route_ok(a) && q8_route_ok(a) ? 4 * q8_scratch_bytes(a) : 0;
}
int launch_prefill_mask(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t stream) {
    return run_tc(e, a, workspace, workspace_bytes, stream, true);
}
// no mask, every key visible to every query (single-token calls have the decode kernel)
bool prefill_full_route_ok(const vox_attn_args * a) {
    return a->mask.data == nullptr && a->q.ne[1] >= 2 && a->k.ne[1] >= kMinKeys && (tc_route_ok(a) || q8_route_ok(a));
}
size_t prefill_full_workspace_bytes(const vox_attn_args * a) {
    return prefill_full_route_ok(a) && q8_route_ok(a) ? 4 * q8_scratch_bytes(a) : 0;
}
int launch_prefill_full(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t stream) {
    return run_tc(e, a, workspace, workspace_bytes, stream, false, false);
}

}  // namespace vox

extern "C" {

#if defined(VOX_ATTN_DEVELOPER) && (defined(VOX_PREFILL_PROFILE) || defined(VOX_PREFILL_TRACE))
int vox_debug_prefill_trace(long long * out) {
    return cudaMemcpyFromSymbol(out, g_trace, sizeof(long long) * 22 * 64) != cudaSuccess;
}
int vox_debug_prefill_profile(unsigned long long * out, int reset) {
    if (out && cudaMemcpyFromSymbol(out, g_prof, sizeof(unsigned long long) * 32) != cudaSuccess) return 1;
    if (reset) {
        unsigned long long zero[32] = {0};
        if (cudaMemcpyToSymbol(g_prof, zero, sizeof(zero)) != cudaSuccess) return 1;
    }
    return 0;
}
#endif

size_t vox_attn_prefill_workspace_bytes(const vox_attn_args * a) {
    if (!a || !vox_attn_supported(a) || a->mask.data != nullptr) return 0;
    return q8_route_ok(a) ? 4 * q8_scratch_bytes(a) : 0;  // K, V, and what rounding each to f16 leaves over
}

int vox_attn_prefill(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    VOX_REQUIRE(e && a, VOX_ATTN_INVALID_ARGUMENT, "vox_attn_prefill: null argument");
    VOX_REQUIRE(a->mask.data == nullptr, VOX_ATTN_INVALID_ARGUMENT,
                "vox_attn_prefill implies the causal mask; pass mask.data == NULL (use vox_attn_forward for explicit masks)");
    VOX_REQUIRE(vox_attn_supported(a), VOX_ATTN_INVALID_ARGUMENT, "%s", vox_attn_last_error_string());
    VOX_REQUIRE(a->q.data && a->k.data && a->v.data && a->dst.data, VOX_ATTN_INVALID_ARGUMENT, "null data pointer");
    VOX_REQUIRE(a->k.ne[1] >= a->q.ne[1], VOX_ATTN_INVALID_ARGUMENT, "n_kv %lld < n_q %lld", (long long) a->k.ne[1],
                (long long) a->q.ne[1]);
    return run_tc(e, a, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), false);
}

}  // extern "C"
