// TEST INFRASTRUCTURE — not part of the shipped attention engine.
//
// Thin C entry points around the reference's own vendored ggml CPU backend, so that the
// unmodified reference implementation of the attention operator
// (third_party/ggml/src/ggml-cpu/ops.cpp:8109-8853, reached through
// ggml_flash_attn_ext, third_party/ggml/src/ggml.c:5281-5322) can be driven from
// ctypes.  Nothing here restates any arithmetic: tensors are created with the public
// ggml API, pointed at caller memory, and executed with ggml_graph_compute.
//
// The file is compiled together with the reference's ggml sources (where they lie in the
// reference checkout) by oracle/Makefile into oracle/_ref/libvoxref_<isa>.so.
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "ggml.h"
#include "ggml-cpu.h"

extern "C" {
// declared in the reference's src/ggml-quants.h (C linkage)
void quantize_row_q8_0_ref(const float * x, void * y, int64_t k);
void dequantize_row_q8_0(const void * x, float * y, int64_t k);
}

namespace {

ggml_type to_type(int t) {
    switch (t) {
        case 0: return GGML_TYPE_F32;
        case 1: return GGML_TYPE_F16;
        case 8: return GGML_TYPE_Q8_0;
        default: return GGML_TYPE_COUNT;
    }
}

}  // namespace

extern "C" {

// Number of bytes of one K or V tensor [D, n_kv, HK, B] of the given type.
int64_t voxref_kv_bytes(int type, int64_t D, int64_t n_kv, int64_t HK, int64_t B) {
    ggml_type t = to_type(type);
    if (t == GGML_TYPE_COUNT) return -1;
    return (int64_t) ggml_row_size(t, D) * n_kv * HK * B;
}

void voxref_quantize_q8_0(const float * x, void * y, int64_t n) { quantize_row_q8_0_ref(x, y, n); }
void voxref_dequantize_q8_0(const void * x, float * y, int64_t n) { dequantize_row_q8_0(x, y, n); }
void voxref_fp32_to_fp16(const float * x, uint16_t * y, int64_t n) { ggml_fp32_to_fp16_row(x, (ggml_fp16_t *) y, n); }
void voxref_fp16_to_fp32(const uint16_t * x, float * y, int64_t n) { ggml_fp16_to_fp32_row((const ggml_fp16_t *) x, y, n); }

// Run `n_layers` independent attention nodes (one graph, as the reference's runtime lays
// its layers out) `iters` times on the reference CPU backend.
//
//   q    : n_layers x [D, n_q,  H,  B] f32, contiguous
//   k, v : n_layers x [D, n_kv, HK, B] of `kv_type` (0 f32, 1 f16, 8 q8_0), contiguous
//   mask : NULL or one shared [n_kv, n_q, mask_ne2, mask_ne3] f16 tensor, contiguous
//   out  : n_layers x [D, H, n_q, B] f32 (the operator's permuted result layout)
//   ms   : if non-NULL receives `iters` wall-clock durations in milliseconds
//
// use_ref != 0 forces the reference's row-at-a-time path (ggml_backend_cpu_set_use_ref
// semantics, ops.cpp:8752-8753).  Returns 0 on success.
int voxref_attn(int n_layers, const float * q, const void * k, const void * v, const uint16_t * mask,
                int kv_type, int64_t D, int64_t n_q, int64_t n_kv, int64_t H, int64_t HK, int64_t B,
                int64_t mask_ne2, int64_t mask_ne3, float scale, int n_threads, int iters,
                int use_ref, float * out, double * ms) {
    const ggml_type kt = to_type(kv_type);
    if (kt == GGML_TYPE_COUNT || n_layers <= 0 || iters <= 0) return 1;

    const size_t n_tensors = (size_t) n_layers * 4 + 8;
    ggml_init_params ip = {
        /*.mem_size   =*/ ggml_tensor_overhead() * n_tensors + ggml_graph_overhead_custom(4 * n_layers + 16, false) + 4096,
        /*.mem_buffer =*/ nullptr,
        /*.no_alloc   =*/ true,
    };
    ggml_context * ctx = ggml_init(ip);
    if (!ctx) return 2;

    const size_t q_bytes  = sizeof(float) * D * n_q * H * B;
    const size_t kv_bytes = ggml_row_size(kt, D) * n_kv * HK * B;
    const size_t o_bytes  = sizeof(float) * D * H * n_q * B;

    ggml_tensor * tm = nullptr;
    if (mask) {
        tm = ggml_new_tensor_4d(ctx, GGML_TYPE_F16, n_kv, n_q, mask_ne2, mask_ne3);
        tm->data = (void *) mask;
    }

    ggml_cgraph * gf = ggml_new_graph_custom(ctx, 4 * n_layers + 16, false);
    for (int l = 0; l < n_layers; ++l) {
        ggml_tensor * tq = ggml_new_tensor_4d(ctx, GGML_TYPE_F32, D, n_q, H, B);
        ggml_tensor * tk = ggml_new_tensor_4d(ctx, kt, D, n_kv, HK, B);
        ggml_tensor * tv = ggml_new_tensor_4d(ctx, kt, D, n_kv, HK, B);
        tq->data = (char *) q + l * q_bytes;
        tk->data = (char *) k + l * kv_bytes;
        tv->data = (char *) v + l * kv_bytes;
        ggml_tensor * to = ggml_flash_attn_ext(ctx, tq, tk, tv, tm, scale, 0.0f, 0.0f);
        to->data = (char *) out + l * o_bytes;
        ggml_build_forward_expand(gf, to);
    }

    ggml_cplan plan = ggml_graph_plan(gf, n_threads, nullptr);
    plan.use_ref = use_ref != 0;
    std::vector<uint8_t> work(plan.work_size + 64);
    plan.work_data = work.data();

    int rc = 0;
    for (int it = 0; it < iters; ++it) {
        auto t0 = std::chrono::steady_clock::now();
        if (ggml_graph_compute(gf, &plan) != GGML_STATUS_SUCCESS) { rc = 3; break; }
        auto t1 = std::chrono::steady_clock::now();
        if (ms) ms[it] = std::chrono::duration<double, std::milli>(t1 - t0).count();
    }
    ggml_free(ctx);
    return rc;
}

// ggml_rope_ext exactly as MiniCPMModel::apply_rope issues it (src/minicpm.cpp:582-600): NEOX pairing,
// n_dims = D, freq_scale 1, ext_factor 0, beta_fast 32, beta_slow 1.
//   x            : [D, n_heads, n_tok] f32, contiguous (the projection layout)
//   positions    : n_tok int32
//   freq_factors : NULL or D/2 floats
//   out          : same shape as x
int voxref_rope(const float * x, int64_t D, int64_t n_heads, int64_t n_tok, const int32_t * positions,
                const float * freq_factors, int n_ctx_orig, float freq_base, float attn_factor, int n_threads, float * out) {
    ggml_init_params ip = {
        /*.mem_size   =*/ ggml_tensor_overhead() * 8 + ggml_graph_overhead_custom(16, false) + 4096,
        /*.mem_buffer =*/ nullptr,
        /*.no_alloc   =*/ true,
    };
    ggml_context * ctx = ggml_init(ip);
    if (!ctx) return 2;
    ggml_tensor * tx = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, D, n_heads, n_tok);
    ggml_tensor * tp = ggml_new_tensor_1d(ctx, GGML_TYPE_I32, n_tok);
    ggml_tensor * tf = nullptr;
    tx->data = (void *) x;
    tp->data = (void *) positions;
    if (freq_factors) {
        tf = ggml_new_tensor_1d(ctx, GGML_TYPE_F32, D / 2);
        tf->data = (void *) freq_factors;
    }
    ggml_tensor * to = ggml_rope_ext(ctx, tx, tp, tf, (int) D, GGML_ROPE_TYPE_NEOX, n_ctx_orig, freq_base, 1.0f, 0.0f,
                                     attn_factor, 32.0f, 1.0f);
    to->data = out;
    ggml_cgraph * gf = ggml_new_graph_custom(ctx, 16, false);
    ggml_build_forward_expand(gf, to);
    ggml_cplan plan = ggml_graph_plan(gf, n_threads, nullptr);
    std::vector<uint8_t> work(plan.work_size + 64);
    plan.work_data = work.data();
    const int rc = ggml_graph_compute(gf, &plan) == GGML_STATUS_SUCCESS ? 0 : 3;
    ggml_free(ctx);
    return rc;
}

// ggml_mul_mat(w, x) exactly as MiniCPMModel::attention_forward issues it for the Q/K/V projection
// (src/minicpm.cpp:660): w [k, n_out] f16 (a weight row per output feature), x [k, n_tok] f32, out [n_out, n_tok] f32.
int voxref_mul_mat_f16(const uint16_t * w, const float * x, int64_t k, int64_t n_out, int64_t n_tok, int n_threads, float * out) {
    ggml_init_params ip = {
        /*.mem_size   =*/ ggml_tensor_overhead() * 8 + ggml_graph_overhead_custom(16, false) + 4096,
        /*.mem_buffer =*/ nullptr,
        /*.no_alloc   =*/ true,
    };
    ggml_context * ctx = ggml_init(ip);
    if (!ctx) return 2;
    ggml_tensor * tw = ggml_new_tensor_2d(ctx, GGML_TYPE_F16, k, n_out);
    ggml_tensor * tx = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, k, n_tok);
    tw->data = (void *) w;
    tx->data = (void *) x;
    ggml_tensor * to = ggml_mul_mat(ctx, tw, tx);
    to->data = out;
    ggml_cgraph * gf = ggml_new_graph_custom(ctx, 16, false);
    ggml_build_forward_expand(gf, to);
    ggml_cplan plan = ggml_graph_plan(gf, n_threads, nullptr);
    std::vector<uint8_t> work(plan.work_size + 64);
    plan.work_data = work.data();
    const int rc = ggml_graph_compute(gf, &plan) == GGML_STATUS_SUCCESS ? 0 : 3;
    ggml_free(ctx);
    return rc;
}

// MiniCPMModel::rms_norm (src/minicpm.cpp:572-580): ggml_rms_norm(x, eps), then ggml_mul with the weight.
//   x, out [k, n_tok] f32, w [k] f32
int voxref_rms_norm_mul(const float * x, const float * w, float eps, int64_t k, int64_t n_tok, int n_threads, float * out) {
    ggml_init_params ip = {
        /*.mem_size   =*/ ggml_tensor_overhead() * 8 + ggml_graph_overhead_custom(16, false) + 4096,
        /*.mem_buffer =*/ nullptr,
        /*.no_alloc   =*/ true,
    };
    ggml_context * ctx = ggml_init(ip);
    if (!ctx) return 2;
    ggml_tensor * tx = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, k, n_tok);
    ggml_tensor * tw = ggml_new_tensor_1d(ctx, GGML_TYPE_F32, k);
    tx->data = (void *) x;
    tw->data = (void *) w;
    std::vector<float> normed((size_t) k * n_tok);
    ggml_tensor * tn = ggml_rms_norm(ctx, tx, eps);
    tn->data = normed.data();
    ggml_tensor * to = ggml_mul(ctx, tn, tw);
    to->data = out;
    ggml_cgraph * gf = ggml_new_graph_custom(ctx, 16, false);
    ggml_build_forward_expand(gf, to);
    ggml_cplan plan = ggml_graph_plan(gf, n_threads, nullptr);
    std::vector<uint8_t> work(plan.work_size + 64);
    plan.work_data = work.data();
    const int rc = ggml_graph_compute(gf, &plan) == GGML_STATUS_SUCCESS ? 0 : 3;
    ggml_free(ctx);
    return rc;
}

// ggml_swiglu_split(gate, up) as MiniCPMModel::mlp_forward issues it (src/minicpm.cpp:738-741).  gate, up, out [n, n_tok] f32
int voxref_swiglu(const float * gate, const float * up, int64_t n, int64_t n_tok, int n_threads, float * out) {
    ggml_init_params ip = {
        /*.mem_size   =*/ ggml_tensor_overhead() * 8 + ggml_graph_overhead_custom(16, false) + 4096,
        /*.mem_buffer =*/ nullptr,
        /*.no_alloc   =*/ true,
    };
    ggml_context * ctx = ggml_init(ip);
    if (!ctx) return 2;
    ggml_tensor * tg = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, n, n_tok);
    ggml_tensor * tu = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, n, n_tok);
    tg->data = (void *) gate;
    tu->data = (void *) up;
    ggml_tensor * to = ggml_swiglu_split(ctx, tg, tu);
    to->data = out;
    ggml_cgraph * gf = ggml_new_graph_custom(ctx, 16, false);
    ggml_build_forward_expand(gf, to);
    ggml_cplan plan = ggml_graph_plan(gf, n_threads, nullptr);
    std::vector<uint8_t> work(plan.work_size + 64);
    plan.work_data = work.data();
    const int rc = ggml_graph_compute(gf, &plan) == GGML_STATUS_SUCCESS ? 0 : 3;
    ggml_free(ctx);
    return rc;
}

}  // extern "C"
