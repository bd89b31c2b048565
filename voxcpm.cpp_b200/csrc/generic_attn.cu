// The operator entry (validation + routing) and the general kernel that covers the whole
// contract of ggml_flash_attn_ext as VoxCPM.cpp uses it: any n_q / n_kv, K/V in f32, f16 or
// q8_0 (34-byte blocks), arbitrary contiguous f16 mask with head/batch broadcast, byte strides.
//
// Replaces ggml_cuda_flash_attn_ext / ggml_cuda_get_best_fattn_kernel
// (third_party/ggml/src/ggml-cuda/fattn.cu:280-478) and, as arithmetic, the row-at-a-time loop of
// the CPU backend (third_party/ggml/src/ggml-cpu/ops.cpp:8109-8345) run with f32 operands:
// K and V are dequantised to f32 (d * q for q8_0), Q stays f32, accumulation is f32.
// Shapes with a dedicated kernel (decode, causal prefill) are routed there instead.
#include "kv_cache.cuh"

#include <algorithm>

using namespace vox;

namespace vox {
int    launch_decode_f16(vox_engine * e, const CUtensorMap & map_k, const CUtensorMap & map_v, int n_kv, int n_streams,
                         int n_heads, int n_kv_heads, const float * q, size_t q_nb_head, size_t q_nb_stream, float * dst,
                         float scale, const vox_tensor * mask, void * workspace, size_t workspace_bytes, cudaStream_t stream);
size_t decode_workspace_bytes(int n_streams, int n_heads, int n_kv_heads, int kv_bound);
bool   decode_mask_ok(const vox_attn_args * a);
// single-token calls over q8_0 K/V in block layout: taken apart into 64-row tiles in the workspace (decode_attn.cu)
bool   decode_q8_blocks_route_ok(const vox_attn_args * a);
size_t decode_q8_blocks_workspace_bytes(const vox_attn_args * a);
int    launch_decode_q8_blocks(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t stream);
// the tcgen05 prefill kernel reading an explicit mask (prefill_attn.cu)
bool   prefill_mask_route_ok(const vox_attn_args * a);
size_t prefill_mask_workspace_bytes(const vox_attn_args * a);
size_t prefill_mask_workspace_min(const vox_attn_args * a);
int    launch_prefill_mask(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t stream);
bool   prefill_full_route_ok(const vox_attn_args * a);
size_t prefill_full_workspace_bytes(const vox_attn_args * a);
int    launch_prefill_full(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, cudaStream_t stream);
}  // namespace vox

namespace {

struct GenericParams {
    const uint8_t *q, *k, *v, *mask;
    float *        dst;
    int            k_type, v_type;
    int64_t        n_q, n_kv, H, B, HK, HV, BK, BV;
    size_t         q_nb1, q_nb2, q_nb3, k_nb1, k_nb2, k_nb3, v_nb1, v_nb2, v_nb3, m_nb1, m_nb2, m_nb3;
    int64_t        m_ne2, m_ne3;
    float          scale;
    int            causal_offset;  // >= 0: key j visible to query i iff j <= i + causal_offset (no mask tensor)
};

// elements 2*lane, 2*lane+1 of one 64-wide K or V row, as f32
__device__ __forceinline__ float2 load_pair(const uint8_t * row, int type, int lane) {
    if (type == VOX_TYPE_F32) return *reinterpret_cast<const float2 *>(row + lane * 8);
    if (type == VOX_TYPE_F16) return __half22float2(*reinterpret_cast<const __half2 *>(row + lane * 4));
    // q8_0: block b = lane / 16 holds elements 32b .. 32b+31 after a 2-byte scale
    const uint8_t * blk = row + (lane >> 4) * 34;
    const float     d   = __half2float(*reinterpret_cast<const __half *>(blk));
    const char2     q   = *reinterpret_cast<const char2 *>(blk + 2 + (lane & 15) * 2);
    return make_float2((float) q.x * d, (float) q.y * d);
}

// One warp per (query row, head, batch); lane l owns dimensions 2l and 2l+1.
__global__ void __launch_bounds__(128) generic_attn_kernel(const GenericParams p) {
    const int       lane = threadIdx.x & 31;
    const long long row  = (long long) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long rows = p.n_q * p.H * p.B;
    if (row >= rows) return;
    const int64_t iq1 = row % p.n_q, iq2 = (row / p.n_q) % p.H, iq3 = row / (p.n_q * p.H);

    const float2 qv = *reinterpret_cast<const float2 *>(p.q + iq1 * p.q_nb1 + iq2 * p.q_nb2 + iq3 * p.q_nb3 + lane * 8);
    const uint8_t * kbase = p.k + (iq2 / (p.H / p.HK)) * p.k_nb2 + (iq3 / (p.B / p.BK)) * p.k_nb3;
    const uint8_t * vbase = p.v + (iq2 / (p.H / p.HV)) * p.v_nb2 + (iq3 / (p.B / p.BV)) * p.v_nb3;
    const __half *  mrow  = p.mask ? reinterpret_cast<const __half *>(p.mask + iq1 * p.m_nb1 + (iq2 % p.m_ne2) * p.m_nb2 +
                                                                     (iq3 % p.m_ne3) * p.m_nb3)
                                   : nullptr;
    int64_t n_vis = p.n_kv;
    if (p.causal_offset >= 0) n_vis = min(p.n_kv, iq1 + p.causal_offset + 1);

    float M = -INFINITY, S = 0.0f, a0 = 0.0f, a1 = 0.0f;
    for (int64_t ic = 0; ic < n_vis; ++ic) {
        const float mv = mrow ? __half2float(mrow[ic]) : 0.0f;
        if (mv == -INFINITY) continue;  // warp-uniform: every lane reads the same mask element
        const float2 kk = load_pair(kbase + ic * p.k_nb1, p.k_type, lane);
        float s = qv.x * kk.x + qv.y * kk.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        s = s * p.scale + mv;
        const float2 vv = load_pair(vbase + ic * p.v_nb1, p.v_type, lane);
        const float  Mn = fmaxf(M, s);
        const float  ms = __expf(M - Mn);  // M == -inf on the first visible key -> 0
        const float  vs = __expf(s - Mn);
        a0 = a0 * ms + vv.x * vs;
        a1 = a1 * ms + vv.y * vs;
        S  = S * ms + vs;
        M  = Mn;
    }
    const float inv = S == 0.0f ? 0.0f : 1.0f / S;  // fully masked row -> zeros (ops.cpp:8333)
    float * out = p.dst + ((iq3 * p.n_q + iq1) * p.H + iq2) * kHeadDim;
    *reinterpret_cast<float2 *>(out + lane * 2) = make_float2(a0 * inv, a1 * inv);
}

size_t type_size0(int t) { return t == VOX_TYPE_F32 ? 4 : t == VOX_TYPE_F16 ? 2 : 34; }
size_t row_size(int t) { return t == VOX_TYPE_F32 ? 256 : t == VOX_TYPE_F16 ? 128 : 68; }

// shape rules of ggml_flash_attn_ext (ggml.c:5281-5322) and of the CPU kernel (ops.cpp:8136-8154)
int validate(const vox_attn_args * a, bool need_data) {
    VOX_REQUIRE(a != nullptr, VOX_ATTN_INVALID_ARGUMENT, "args is null");
    const vox_tensor &q = a->q, &k = a->k, &v = a->v, &m = a->mask, &d = a->dst;
    VOX_REQUIRE(a->max_bias == 0.0f && a->logit_softcap == 0.0f && a->has_sinks == 0, VOX_ATTN_UNSUPPORTED,
                "max_bias, logit_softcap and sinks are not supported (VoxCPM.cpp never uses them)");
    VOX_REQUIRE(q.type == VOX_TYPE_F32, VOX_ATTN_UNSUPPORTED, "q must be f32");
    for (const vox_tensor * t : {&k, &v})
        VOX_REQUIRE(t->type == VOX_TYPE_F32 || t->type == VOX_TYPE_F16 || t->type == VOX_TYPE_Q8_0, VOX_ATTN_UNSUPPORTED,
                    "K/V type %d not supported (f32, f16, q8_0)", t->type);
    VOX_REQUIRE(q.ne[0] == kHeadDim && k.ne[0] == kHeadDim && v.ne[0] == kHeadDim, VOX_ATTN_UNSUPPORTED,
                "head_dim must be 64 (got q %lld, k %lld, v %lld)", (long long) q.ne[0], (long long) k.ne[0],
                (long long) v.ne[0]);
    for (const vox_tensor * t : {&q, &k, &v})
        for (int i = 0; i < 4; ++i) VOX_REQUIRE(t->ne[i] >= 0, VOX_ATTN_INVALID_ARGUMENT, "negative extent");
    VOX_REQUIRE(q.ne[1] > 0 && q.ne[2] > 0 && q.ne[3] > 0, VOX_ATTN_INVALID_ARGUMENT, "empty q");
    VOX_REQUIRE(k.ne[1] == v.ne[1], VOX_ATTN_INVALID_ARGUMENT, "K has %lld rows, V has %lld", (long long) k.ne[1],
                (long long) v.ne[1]);
    VOX_REQUIRE(k.ne[2] > 0 && v.ne[2] > 0 && q.ne[2] % k.ne[2] == 0 && q.ne[2] % v.ne[2] == 0, VOX_ATTN_INVALID_ARGUMENT,
                "n_head %lld is not a multiple of n_head_kv %lld / %lld", (long long) q.ne[2], (long long) k.ne[2],
                (long long) v.ne[2]);
    VOX_REQUIRE(k.ne[3] == q.ne[3] && v.ne[3] == q.ne[3], VOX_ATTN_INVALID_ARGUMENT, "batch extents differ");
    VOX_REQUIRE(q.nb[0] == 4 && k.nb[0] == type_size0(k.type) && v.nb[0] == type_size0(v.type), VOX_ATTN_INVALID_ARGUMENT,
                "input rows must be contiguous");
    VOX_REQUIRE(q.nb[1] % 8 == 0 && q.nb[2] % 8 == 0 && q.nb[3] % 8 == 0, VOX_ATTN_INVALID_ARGUMENT,
                "q strides must be multiples of 8 bytes");
    for (const vox_tensor * t : {&k, &v}) {
        const size_t al = t->type == VOX_TYPE_F32 ? 8 : t->type == VOX_TYPE_F16 ? 4 : 2;
        VOX_REQUIRE(t->nb[1] >= row_size(t->type) && t->nb[1] % al == 0 && t->nb[2] % al == 0 && t->nb[3] % al == 0,
                    VOX_ATTN_INVALID_ARGUMENT, "K/V strides are smaller than a row or misaligned");
    }
    if (m.data != nullptr || !need_data) {
        if (m.data != nullptr) {
            VOX_REQUIRE(m.type == VOX_TYPE_F16, VOX_ATTN_UNSUPPORTED, "mask must be f16");
            VOX_REQUIRE(m.ne[0] >= k.ne[1] && m.ne[1] >= q.ne[1], VOX_ATTN_INVALID_ARGUMENT,
                        "mask [%lld, %lld] is smaller than [n_kv %lld, n_q %lld]", (long long) m.ne[0], (long long) m.ne[1],
                        (long long) k.ne[1], (long long) q.ne[1]);
            VOX_REQUIRE(m.ne[2] > 0 && m.ne[3] > 0 && q.ne[2] % m.ne[2] == 0 && q.ne[3] % m.ne[3] == 0,
                        VOX_ATTN_INVALID_ARGUMENT, "mask does not broadcast over heads/batch");
            // contiguity as ggml_is_contiguous sees it: strides of extent-1 axes do not matter
            VOX_REQUIRE(m.nb[0] == 2 && (m.ne[1] == 1 || m.nb[1] == (size_t) m.ne[0] * 2) &&
                            (m.ne[2] == 1 || m.nb[2] == (size_t) m.ne[0] * 2 * m.ne[1]) &&
                            (m.ne[3] == 1 || m.nb[3] == (size_t) m.ne[0] * 2 * m.ne[1] * m.ne[2]),
                        VOX_ATTN_INVALID_ARGUMENT, "mask must be contiguous");
        }
    }
    VOX_REQUIRE(d.type == VOX_TYPE_F32 && d.ne[0] == kHeadDim && d.ne[1] == q.ne[2] && d.ne[2] == q.ne[1] &&
                    d.ne[3] == q.ne[3],
                VOX_ATTN_INVALID_ARGUMENT, "dst must be f32 [64, n_head, n_q, batch]");
    VOX_REQUIRE(d.nb[0] == 4 && d.nb[1] == 256 && d.nb[2] == 256 * (size_t) d.ne[1] && d.nb[3] == d.nb[2] * (size_t) d.ne[2],
                VOX_ATTN_INVALID_ARGUMENT, "dst must be contiguous");
    if (need_data) {
        VOX_REQUIRE(q.data && d.data && (k.ne[1] == 0 || (k.data && v.data)), VOX_ATTN_INVALID_ARGUMENT, "null data pointer");
        VOX_REQUIRE((reinterpret_cast<uintptr_t>(q.data) & 7) == 0 && (reinterpret_cast<uintptr_t>(d.data) & 15) == 0,
                    VOX_ATTN_INVALID_ARGUMENT, "q must be 8-byte and dst 16-byte aligned");
    }
    return VOX_ATTN_OK;
}

// n_q == 1, f16 K/V with 16-byte-aligned strides, no mask or one whose rows can be read two values at a time,
// GQA <= 8: the split-KV decode kernel
bool decode_route_ok(const vox_attn_args * a) {
    const vox_tensor &q = a->q, &k = a->k, &v = a->v;
    if (q.ne[1] != 1 || !decode_mask_ok(a)) return false;
    if (q.ne[3] * k.ne[2] > kCounterSlots) return false;
    if (k.type != VOX_TYPE_F16 || v.type != VOX_TYPE_F16) return false;
    if (k.ne[2] != v.ne[2] || q.ne[2] / k.ne[2] > 8) return false;
    if (k.ne[1] < 1) return false;
    for (const vox_tensor * t : {&k, &v}) {
        if ((reinterpret_cast<uintptr_t>(t->data) & 15) != 0) return false;
        if (t->nb[1] % 16 || t->nb[2] % 16 || t->nb[3] % 16) return false;
    }
    return true;
}

}  // namespace

namespace vox {

int launch_generic(vox_engine * e, const vox_attn_args * a, int causal_offset, cudaStream_t stream) {
    GenericParams p;
    p.q = (const uint8_t *) a->q.data; p.k = (const uint8_t *) a->k.data; p.v = (const uint8_t *) a->v.data;
    p.mask = (const uint8_t *) a->mask.data; p.dst = (float *) a->dst.data;
    p.k_type = a->k.type; p.v_type = a->v.type;
    p.n_q = a->q.ne[1]; p.n_kv = a->k.ne[1]; p.H = a->q.ne[2]; p.B = a->q.ne[3];
    p.HK = a->k.ne[2]; p.HV = a->v.ne[2]; p.BK = a->k.ne[3]; p.BV = a->v.ne[3];
    p.q_nb1 = a->q.nb[1]; p.q_nb2 = a->q.nb[2]; p.q_nb3 = a->q.nb[3];
    p.k_nb1 = a->k.nb[1]; p.k_nb2 = a->k.nb[2]; p.k_nb3 = a->k.nb[3];
    p.v_nb1 = a->v.nb[1]; p.v_nb2 = a->v.nb[2]; p.v_nb3 = a->v.nb[3];
    p.m_nb1 = a->mask.nb[1]; p.m_nb2 = a->mask.nb[2]; p.m_nb3 = a->mask.nb[3];
    p.m_ne2 = a->mask.data ? a->mask.ne[2] : 1; p.m_ne3 = a->mask.data ? a->mask.ne[3] : 1;
    p.scale = a->scale; p.causal_offset = causal_offset;
    const long long rows = p.n_q * p.H * p.B;
    generic_attn_kernel<<<(unsigned) ((rows + 3) / 4), 128, 0, stream>>>(p);
    return check_launch(e, "generic_attn_kernel");
}

}  // namespace vox

extern "C" {

int vox_attn_supported(const vox_attn_args * a) { return validate(a, false) == VOX_ATTN_OK ? 1 : 0; }

size_t vox_attn_workspace_bytes(const vox_attn_args * a) {
    if (validate(a, false) != VOX_ATTN_OK) return 0;
    if (decode_route_ok(a))
        return decode_workspace_bytes((int) a->q.ne[3], (int) a->q.ne[2], (int) a->k.ne[2], (int) a->k.ne[1]);
    if (decode_q8_blocks_route_ok(a)) return decode_q8_blocks_workspace_bytes(a);
    return a->mask.data ? prefill_mask_workspace_bytes(a) : prefill_full_workspace_bytes(a);
}

int vox_attn_forward(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes, void * stream) {
    VOX_REQUIRE(e != nullptr, VOX_ATTN_INVALID_ARGUMENT, "engine is null");
    int rc = validate(a, true);
    if (rc != VOX_ATTN_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (decode_route_ok(a) && workspace != nullptr &&
        workspace_bytes >= decode_workspace_bytes((int) a->q.ne[3], (int) a->q.ne[2], (int) a->k.ne[2], (int) a->k.ne[1])) {
        // K/V of the caller described to the copy engine exactly as given: rows beyond n_kv are
        // out of bounds for the descriptor and read as zeros
        CUtensorMap    mk, mv;
        const uint64_t dims[5] = {64, (uint64_t) a->k.ne[1], (uint64_t) a->k.ne[2], (uint64_t) a->k.ne[3], 1};
        const uint32_t box[5]  = {64, kKvTile, 1, 1, 1};
        const vox_tensor * ts[2] = {&a->k, &a->v};
        CUtensorMap *      ms[2] = {&mk, &mv};
        for (int i = 0; i < 2; ++i) {
            const uint64_t strides[4] = {ts[i]->nb[1], ts[i]->nb[2], ts[i]->nb[3],
                                         std::max<uint64_t>(ts[i]->nb[3] * (uint64_t) ts[i]->ne[3], 16)};
            rc = make_tensor_map(e, ms[i], ts[i]->data, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc != VOX_ATTN_OK) return rc;
        }
        return launch_decode_f16(e, mk, mv, (int) a->k.ne[1], (int) a->q.ne[3], (int) a->q.ne[2], (int) a->k.ne[2],
                                 (const float *) a->q.data, a->q.nb[2], a->q.nb[3], (float *) a->dst.data, a->scale,
                                 a->mask.data ? &a->mask : nullptr, workspace, workspace_bytes, st);
    }
    if (decode_q8_blocks_route_ok(a) && workspace != nullptr && workspace_bytes >= decode_q8_blocks_workspace_bytes(a))
        return launch_decode_q8_blocks(e, a, workspace, workspace_bytes, st);
    // large masked problems over f16 / q8_0 K/V: the tensor-core kernel reads the mask (q8_0 needs the workspace)
    if (prefill_mask_route_ok(a) && workspace_bytes >= prefill_mask_workspace_min(a) &&
        (prefill_mask_workspace_min(a) == 0 || workspace != nullptr))
        return launch_prefill_mask(e, a, workspace, workspace_bytes, st);
    if (prefill_full_route_ok(a) && workspace_bytes >= prefill_full_workspace_bytes(a) &&
        (prefill_full_workspace_bytes(a) == 0 || workspace != nullptr))
        return launch_prefill_full(e, a, workspace, workspace_bytes, st);
    return launch_generic(e, a, -1, st);
}

int vox_attn_forward_host(vox_engine * e, const vox_attn_args * a, void * stream) {
    VOX_REQUIRE(e != nullptr, VOX_ATTN_INVALID_ARGUMENT, "engine is null");
    int rc = validate(a, false);
    if (rc != VOX_ATTN_OK) return rc;
    VOX_REQUIRE(a->q.data && a->dst.data && (a->k.ne[1] == 0 || (a->k.data && a->v.data)), VOX_ATTN_INVALID_ARGUMENT,
                "null data pointer");
    VOX_CUDA_TRY(cudaSetDevice(e->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // each host tensor is copied as one span with its strides unchanged
    auto span = [](const vox_tensor & t) {
        size_t end = 0;
        const size_t e0 = t.type == VOX_TYPE_Q8_0 ? (size_t) (t.ne[0] / 32) * 34 : (size_t) t.ne[0] * t.nb[0];
        end = e0;
        for (int i = 1; i < 4; ++i)
            if (t.ne[i] > 0) end += (size_t) (t.ne[i] - 1) * t.nb[i];
        for (int i = 0; i < 4; ++i)
            if (t.ne[i] == 0) return (size_t) 0;
        return end;
    };
    const size_t qb = span(a->q), kb = span(a->k), vb = span(a->v), mb = a->mask.data ? span(a->mask) : 0, ob = span(a->dst);
    auto up = [](size_t x) { return (x + 255) & ~(size_t) 255; };
    const size_t total = up(qb) + up(kb) + up(vb) + up(mb) + up(ob);
    if (total > e->stage_bytes) {
        if (e->stage_dev) cudaFree(e->stage_dev);
        e->stage_dev = nullptr; e->stage_bytes = 0;
        cudaError_t err = cudaMalloc(&e->stage_dev, total);
        if (err != cudaSuccess) { cudaGetLastError(); set_error("staging allocation of %zu bytes failed", total); return VOX_ATTN_OUT_OF_MEMORY; }
        e->stage_bytes = total;
    }
    vox_attn_args d = *a;
    uint8_t * base = static_cast<uint8_t *>(e->stage_dev);
    d.q.data = base; d.k.data = base + up(qb); d.v.data = base + up(qb) + up(kb);
    d.mask.data = a->mask.data ? base + up(qb) + up(kb) + up(vb) : nullptr;
    d.dst.data = base + up(qb) + up(kb) + up(vb) + up(mb);
    const size_t ws = vox_attn_workspace_bytes(&d);
    if (ws > e->stage_ws_bytes) {
        if (e->stage_ws) cudaFree(e->stage_ws);
        e->stage_ws = nullptr; e->stage_ws_bytes = 0;
        cudaError_t err = cudaMalloc(&e->stage_ws, ws);
        if (err != cudaSuccess) { cudaGetLastError(); set_error("workspace allocation of %zu bytes failed", ws); return VOX_ATTN_OUT_OF_MEMORY; }
        e->stage_ws_bytes = ws;
    }
    VOX_CUDA_TRY(cudaMemcpyAsync(d.q.data, a->q.data, qb, cudaMemcpyHostToDevice, st));
    if (kb) VOX_CUDA_TRY(cudaMemcpyAsync(d.k.data, a->k.data, kb, cudaMemcpyHostToDevice, st));
    if (vb) VOX_CUDA_TRY(cudaMemcpyAsync(d.v.data, a->v.data, vb, cudaMemcpyHostToDevice, st));
    if (mb) VOX_CUDA_TRY(cudaMemcpyAsync(d.mask.data, a->mask.data, mb, cudaMemcpyHostToDevice, st));
    rc = vox_attn_forward(e, &d, e->stage_ws, e->stage_ws_bytes, stream);
    if (rc != VOX_ATTN_OK) return rc;
    VOX_CUDA_TRY(cudaMemcpyAsync(a->dst.data, d.dst.data, ob, cudaMemcpyDeviceToHost, st));
    return vox_engine_sync_status(e, stream);
}

}  // extern "C"
