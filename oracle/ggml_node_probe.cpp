// TEST INFRASTRUCTURE.  Builds a GGML_OP_FLASH_ATTN_EXT node by hand, as ggml_flash_attn_ext would
// (third_party/ggml/src/ggml.c:5281-5322: sources q, k, v, mask; op_params scale, max_bias, logit_softcap;
// result [D, H, n_q, B] f32), with the reference's own struct ggml_tensor from its ggml.h, and hands it to the
// engine through include/vox_attn_ggml.h.  Nothing of ggml is linked: the header alone is used, which is how a
// backend of the reference would include it.  The parity test drives this through ctypes with device pointers.
#include "vox_attn_ggml.h"

namespace {

size_t type_size(int type) { return type == GGML_TYPE_F32 ? 4 : type == GGML_TYPE_F16 ? 2 : 34; }
int64_t block_size(int type) { return type == GGML_TYPE_Q8_0 ? 32 : 1; }

// a contiguous tensor: nb[0] = type size, nb[1] = nb[0] * ne[0] / block size, nb[i] = nb[i-1] * ne[i-1]
void describe(ggml_tensor & t, int type, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3, void * data) {
    memset(&t, 0, sizeof(t));
    t.type  = (ggml_type) type;
    t.ne[0] = ne0; t.ne[1] = ne1; t.ne[2] = ne2; t.ne[3] = ne3;
    t.nb[0] = type_size(type);
    t.nb[1] = t.nb[0] * (size_t) (ne0 / block_size(type));
    t.nb[2] = t.nb[1] * (size_t) ne1;
    t.nb[3] = t.nb[2] * (size_t) ne2;
    t.data  = data;
}

}  // namespace

extern "C" {

size_t vox_probe_sizeof_ggml_tensor(void) { return sizeof(ggml_tensor); }

// what = 0: run the node; 1: capability query only (returns 1 / 0); 2: workspace bytes (through *ws_out)
int vox_probe_flash_attn_ext(vox_engine * engine, int what, int kv_type, int64_t n_q, int64_t n_kv, int64_t n_heads,
                             int64_t n_kv_heads, int64_t n_batch, void * q, void * k, void * v, void * mask, int64_t mask_ne2,
                             int64_t mask_ne3, float scale, float max_bias, float logit_softcap, void * dst_data, void * workspace,
                             size_t workspace_bytes, size_t * ws_out, void * cuda_stream) {
    ggml_tensor tq, tk, tv, tm, dst;
    describe(tq, GGML_TYPE_F32, 64, n_q, n_heads, n_batch, q);
    describe(tk, kv_type, 64, n_kv, n_kv_heads, n_batch, k);
    describe(tv, kv_type, 64, n_kv, n_kv_heads, n_batch, v);
    describe(tm, GGML_TYPE_F16, n_kv, n_q, mask_ne2, mask_ne3, mask);
    describe(dst, GGML_TYPE_F32, 64, n_heads, n_q, n_batch, dst_data);  // permuted against q (ggml.c:5308-5310)
    dst.op     = GGML_OP_FLASH_ATTN_EXT;
    dst.src[0] = &tq;
    dst.src[1] = &tk;
    dst.src[2] = &tv;
    dst.src[3] = mask ? &tm : nullptr;
    const float params[3] = {scale, max_bias, logit_softcap};
    memcpy(dst.op_params, params, sizeof(params));
    if (what == 1) return vox_flash_attn_ext_supported(&dst) ? 1 : 0;
    if (what == 2) {
        if (ws_out) *ws_out = vox_flash_attn_ext_workspace_bytes(&dst);
        return 0;
    }
    return vox_flash_attn_ext(engine, &dst, workspace, workspace_bytes, cuda_stream);
}

}  // extern "C"
