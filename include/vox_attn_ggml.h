/* vox_attn_ggml.h — the operator behind a ggml graph node (C++, header only).
 *
 * For a host that already holds ggml tensors: fills vox_attn_args from a GGML_OP_FLASH_ATTN_EXT node
 * exactly as ggml's own backends read it (sources 0-3 = q, k, v, mask, source 4 = sinks, op_params =
 * scale, max_bias, logit_softcap; third_party/ggml/src/ggml.c:5281-5322) and calls the engine.  It
 * replaces `case GGML_OP_FLASH_ATTN_EXT` of the CUDA backend's op switch
 * (third_party/ggml/src/ggml-cuda/ggml-cuda.cu:2721-2722 -> fattn.cu:460-478) and its capability
 * query (ggml-cuda.cu:4852-4853 -> fattn.cu:480-482).
 *
 * Needs the reference's "ggml.h" on the include path (only the struct ggml_tensor and the type
 * enumerators are used: nothing of ggml is linked) and libvoxattn.so at link time.
 */
#ifndef VOX_ATTN_GGML_H
#define VOX_ATTN_GGML_H

#include <string.h>

#include "ggml.h"
#include "vox_attn.h"

static_assert((int) GGML_TYPE_F32 == (int) VOX_TYPE_F32 && (int) GGML_TYPE_F16 == (int) VOX_TYPE_F16 &&
                  (int) GGML_TYPE_Q8_0 == (int) VOX_TYPE_Q8_0,
              "vox_type is numbered as ggml_type");

/* the fields of ggml_tensor the operator reads (ggml.h:655-687); a null tensor (no mask) gives data == NULL */
static inline vox_tensor vox_tensor_from_ggml(const struct ggml_tensor * t) {
    vox_tensor v;
    memset(&v, 0, sizeof(v));
    if (t == NULL) return v;
    v.type = (int32_t) t->type;
    for (int i = 0; i < 4; ++i) {
        v.ne[i] = t->ne[i];
        v.nb[i] = t->nb[i];
    }
    v.data = t->data; /* device pointer of the backend buffer */
    return v;
}

static inline vox_attn_args vox_attn_args_from_ggml(const struct ggml_tensor * dst) {
    vox_attn_args a;
    memset(&a, 0, sizeof(a));
    a.q    = vox_tensor_from_ggml(dst->src[0]);
    a.k    = vox_tensor_from_ggml(dst->src[1]);
    a.v    = vox_tensor_from_ggml(dst->src[2]);
    a.mask = vox_tensor_from_ggml(dst->src[3]);
    a.dst  = vox_tensor_from_ggml(dst);
    memcpy(&a.scale, (const float *) dst->op_params + 0, sizeof(float));
    memcpy(&a.max_bias, (const float *) dst->op_params + 1, sizeof(float));
    memcpy(&a.logit_softcap, (const float *) dst->op_params + 2, sizeof(float));
    a.has_sinks = dst->src[4] != NULL;
    return a;
}

/* ggml_cuda_flash_attn_ext_supported */
static inline bool vox_flash_attn_ext_supported(const struct ggml_tensor * dst) {
    if (dst == NULL || dst->op != GGML_OP_FLASH_ATTN_EXT) return false;
    const vox_attn_args a = vox_attn_args_from_ggml(dst);
    return vox_attn_supported(&a) != 0;
}

/* scratch the node needs (the caller's pool allocation, fattn-common.cuh:808-818) */
static inline size_t vox_flash_attn_ext_workspace_bytes(const struct ggml_tensor * dst) {
    const vox_attn_args a = vox_attn_args_from_ggml(dst);
    return vox_attn_workspace_bytes(&a);
}

/* ggml_cuda_flash_attn_ext: returns a vox_status */
static inline int vox_flash_attn_ext(vox_engine * engine, const struct ggml_tensor * dst, void * workspace, size_t workspace_bytes,
                                     void * cuda_stream) {
    if (dst == NULL || dst->op != GGML_OP_FLASH_ATTN_EXT) return VOX_ATTN_INVALID_ARGUMENT;
    const vox_attn_args a = vox_attn_args_from_ggml(dst);
    return vox_attn_forward(engine, &a, workspace, workspace_bytes, cuda_stream);
}

#endif /* VOX_ATTN_GGML_H */
