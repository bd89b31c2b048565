// Rotary position embedding for the decode step: the (cos, sin) table of one step's positions.
//
// MiniCPMModel::apply_rope (src/minicpm.cpp:582-600) issues ggml_rope_ext with GGML_ROPE_TYPE_NEOX,
// freq_scale 1, ext_factor 0, optional per-frequency factors and attn_factor on cos and sin, once for Q and once
// for K in every layer; ggml recomputes the same cos/sin cache each time (ggml_rope_cache_init,
// third_party/ggml/src/ggml-cpu/ops.cpp:5613-5629; rope_neox in ggml-cuda/rope.cu).  The angles depend on the
// position only, so here they are computed once per step for all streams and every layer's decode launch applies
// them to Q and to the arriving K row (decode_attn.cu).
#include "common.cuh"

#include <cmath>

using namespace vox;

namespace {

// One thread per (stream, frequency).  theta_i is built by i successive f32 multiplications, as the reference's
// loop builds it, so that the angle is the same float the reference takes the cosine of.
__global__ void rope_table_kernel(const int32_t * positions, int pos_offset, int n_streams, float theta_scale, float attn_factor,
                                  const float * freq_factors, float * table) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_wait();  // the positions may come from the kernel before
    pdl_launch_dependents();
    if (idx >= n_streams * (kHeadDim / 2)) return;
    const int s = idx / (kHeadDim / 2), i = idx % (kHeadDim / 2);
    float     theta = (float) (positions[s] + pos_offset);
    for (int k = 0; k < i; ++k) theta = __fmul_rn(theta, theta_scale);
    const float ff = freq_factors ? freq_factors[i] : 1.0f;
    const float th = __fdiv_rn(theta, ff);
    table[2 * idx + 0] = __fmul_rn(cosf(th), attn_factor);
    table[2 * idx + 1] = __fmul_rn(sinf(th), attn_factor);
}

}  // namespace

extern "C" int vox_rope_table(vox_engine * e, const vox_rope_config * cfg, const int32_t * positions, int pos_offset, int n_streams,
                              float * table, void * stream) {
    VOX_REQUIRE(e && cfg && positions && table, VOX_ATTN_INVALID_ARGUMENT, "vox_rope_table: null argument");
    VOX_REQUIRE(n_streams > 0, VOX_ATTN_INVALID_ARGUMENT, "n_streams must be positive");
    VOX_REQUIRE(cfg->freq_base > 0.0f, VOX_ATTN_INVALID_ARGUMENT, "freq_base must be positive");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(table) & 7) == 0, VOX_ATTN_INVALID_ARGUMENT, "table must be 8-byte aligned");
    VOX_CUDA_TRY(cudaSetDevice(e->device));
    const float theta_scale = powf(cfg->freq_base, -2.0f / kHeadDim);  // ops.cpp:5778
    const int   n           = n_streams * (kHeadDim / 2);
    launch_pdl(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), positions, pos_offset,
               n_streams, theta_scale, cfg->attn_factor, cfg->freq_factors, table);
    return check_launch(e, "rope_table_kernel");
}
