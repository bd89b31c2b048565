// Causal prefill attention entry.
//
// Replaces the n_q == n_kv call that MiniCPMModel::forward makes with the f16 mask from
// create_causal_mask (src/minicpm.cpp:602-620, 779-802 -> :708-710); the mask is implied by a
// causal offset instead of being materialised and re-read (512 KB per 512-token graph there).
#include "common.cuh"

using namespace vox;

namespace vox {
int launch_generic(vox_engine * e, const vox_attn_args * a, int causal_offset, cudaStream_t stream);
}

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
    const int offset = (int) (a->k.ne[1] - a->q.ne[1]);
    return launch_generic(e, a, offset, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
