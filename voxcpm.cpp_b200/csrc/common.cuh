// Shared declarations of the attention engine: status handling, the engine object, and
// thin wrappers over the sm_100a PTX the kernels use (mbarrier, bulk-tensor copies,
// ldmatrix, mma).  Every device-side wait in this code base goes through mbar_wait_bounded or
// mbar_wait_spin, which compare the SM clock with a limit every few polls, give up when it is
// exceeded and report through the engine's status word instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <utility>
#include <vector>

#include "vox_attn.h"

namespace vox {

// ------------------------------------------------------------------ host side

void set_error(const char * fmt, ...);

#define VOX_CUDA_TRY(expr)                                                                   \
    do {                                                                                     \
        cudaError_t err__ = (expr);                                                          \
        if (err__ != cudaSuccess) {                                                          \
            ::vox::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, __LINE__); \
            return VOX_ATTN_CUDA_ERROR;                                                      \
        }                                                                                    \
    } while (0)

#define VOX_REQUIRE(cond, status, ...)          \
    do {                                        \
        if (!(cond)) {                          \
            ::vox::set_error(__VA_ARGS__);      \
            return (status);                    \
        }                                       \
    } while (0)

constexpr int kHeadDim = 64;
constexpr int kCounterSlots = 1 << 16;  // engine-owned split-KV tickets (operator calls on the caller's own tensors)
constexpr int kDecodeMaxSms = 148;      // a decode grid never spans more SMs than this (bounds its workspace)

// bits of the device status word
enum : int { kStatusTimeout = 1, kStatusBadState = 2 };

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace vox

struct vox_kv_cache;

struct vox_engine {
    int               device       = 0;
    int               sm_count     = 0;
    int *             status_host  = nullptr;  // pinned, mapped; kernels write through status_dev
    int *             status_dev   = nullptr;
    uint64_t          launches     = 0;
    int *             counters_dev = nullptr;  // kCounterSlots zeroed ints: split-KV arrival tickets
    uint32_t          attr_mask    = 0;      // kernels whose shared-memory attribute was set on this device
    // developer settings, read from the environment once, when the engine is created
    int               decode_early_tiles = -1;  // VOX_DECODE_EARLY: tiles a decode CTA requests before its dependency wait (-1: a full ring)
    int               linear_split = 0;         // VOX_LINEAR_SPLIT: CTAs along K of a vox_linear launch (0: chosen by shape)
    int               decode_cluster = 1;       // VOX_DECODE_CLUSTER=0: no cluster mode in decode launches of few pairs
    int               decode_wave[2] = {0, 0};  // VOX_DECODE_WAVE / VOX_DECODE_WAVE_Q8: CTAs per SM of a decode grid (0: all that fit)
    int               prefill_single_f16 = 0;   // VOX_PREFILL_WEIGHTS=f16: softmax weights as one f16 (comparison only)
    std::vector<vox_kv_cache *> caches;         // caches created from this engine (their ticket counters are reset after a failure)
    vox::encode_tiled_fn encode    = nullptr;
    // staging for the *_host entry points
    void *            stage_dev    = nullptr;
    size_t            stage_bytes  = 0;
    void *            stage_ws     = nullptr;
    size_t            stage_ws_bytes = 0;
};

namespace vox {

// 5-D tiled tensor map: dims/box in elements (dim 0 fastest), strides[i] = byte stride of dim i+1.
int make_tensor_map(const vox_engine * e, CUtensorMap * out, void * base, CUtensorMapDataType dt, const uint64_t dims[5],
                    const uint64_t strides[4], const uint32_t box[5], CUtensorMapSwizzle swizzle);

// Launch with programmatic dependent launch: the grid may be scheduled while the previous kernel of the
// stream is still draining, and its threads block in pdl_wait() until that kernel has completed and its
// writes are visible.  Every kernel launched this way calls pdl_wait() before its first global access.
// VOX_NO_PDL=1 in the environment turns the attribute off.
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);  // errors surface through check_launch
}

inline int check_launch(vox_engine * e, const char * what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        set_error("launch of %s failed: %s", what, cudaGetErrorString(err));
        return VOX_ATTN_CUDA_ERROR;
    }
    e->launches += 1;
    return VOX_ATTN_OK;
}

// ------------------------------------------------------------------ device side

#ifdef __CUDACC__

constexpr long long kWaitCycles = 4000000000LL;  // SM clock cycles before a wait gives up (~2 s at 1.9 GHz)

// programmatic dependent launch: wait for the preceding kernel of the stream / let the next one be scheduled
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void * p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bulk-tensor store shared -> global of one box of a tensor map (the innermost coordinate times the element size must be
// a multiple of 16 bytes, no coordinate may be negative; what lies beyond the tensor's extents is not written).  The
// writes to shared memory that fill the tile are made visible to the copy by fence_proxy_async_smem before the barrier
// that precedes the issue.  Stores are tracked in bulk groups of the issuing thread: bulk_wait_read returns once the
// committed groups have read their shared memory (it may be rewritten), bulk_wait_all once they have been performed.
__device__ __forceinline__ void tma_store_5d(const CUtensorMap * map, uint32_t src, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// A named barrier of n_threads that also votes: true when `mine` is true for every one of them.
__device__ __forceinline__ bool named_bar_all(int id, int n_threads, bool mine) {
    uint32_t all;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.and.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(all)
        : "r"(id), "r"(n_threads), "r"((uint32_t) mine)
        : "memory");
    return all != 0;
}

// One poll.  try_wait parks the thread in hardware until the phase completes or a time limit passes; the limit asked for
// here (the suspend-time hint, in ns) is long, so that a thread whose wait is long (a producer facing a full ring, a
// consumer ahead of the copies) polls rarely and leaves the issue slots to the warps that have work: with the default
// limit the waiting warps of the q8_0 decode kernel accounted for about a quarter of all instructions issued.  The
// thread wakes as soon as the phase completes, whatever the limit.
constexpr uint32_t kSuspendHintNs = 20000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}
// Returns false when the phase did not complete in time.  The loop polls back to back (each poll parks the thread,
// see above); every 16 failed polls the elapsed clock is checked against kWaitCycles (about two seconds).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit = kWaitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 0 && clock64() - t0 > limit) return false;
    }
}

// Same contract, polling with the non-blocking test_wait: lowest wake-up latency, for the few
// threads whose wait sits on a kernel's critical path.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 4095u) == 0 && clock64() - t0 > kWaitCycles) return false;
    }
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap * map, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap * map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2, uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t & r0, uint32_t & r1, uint32_t & r2,
                                                  uint32_t & r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
#ifndef VOX_MMA_ASM
#define VOX_MMA_ASM asm volatile
#endif
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    VOX_MMA_ASM(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// x ~= hi + lo with hi, lo representable in f16: carries ~22 bits of x through f16 MMAs
__device__ __forceinline__ void split_hi_lo(float x, float & hi, float & lo) {
    hi = __half2float(__float2half_rn(x));
    lo = x - hi;
}

// 2^x on the special-function unit: one MUFU instruction, relative error 2^-22, results below 2^-126 flushed
// to zero (exp2f adds range handling for arguments the kernels here never produce)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void named_bar_sync(int id, int n_threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

#endif  // __CUDACC__

}  // namespace vox
