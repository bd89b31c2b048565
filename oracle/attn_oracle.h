/* TEST INFRASTRUCTURE — a CPU restatement of the reference's attention operator.
 *
 * This header and attn_oracle.c exist only so that tests, the smoke check and the
 * benchmark's cpu_baseline leg can check the CUDA engine.  Nothing in the shipped engine
 * includes, links or calls it.
 *
 * Parity status: PINNED.  tests/test_oracle.py compares every path below with the
 * reference's own ggml CPU backend (compiled unmodified into oracle/_ref) where that
 * library is present, and with committed fixtures generated from it
 * (tests/golden/, made by tests/golden/make_golden.py) everywhere.
 */
#ifndef VOX_ATTN_ORACLE_H
#define VOX_ATTN_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types, numbered as the reference numbers them (ggml.h enum ggml_type) */
enum { VOXO_F32 = 0, VOXO_F16 = 1, VOXO_Q8_0 = 8 };

/* which of the reference's code paths to restate */
enum {
    VOXO_PATH_AUTO     = 0, /* the selection rule of ops.cpp:8755-8756, 8812-8820          */
    VOXO_PATH_ROW      = 1, /* row-at-a-time, as shipped (ops.cpp:8109-8345): Q converted to */
                            /* K's dot type, fp16 accumulator when V is f16                */
    VOXO_PATH_ROW_F32  = 2, /* the same loop as the reference runs it on F32-typed K/V      */
                            /* holding the dequantised values: f32 Q, f32 accumulator      */
    VOXO_PATH_TILED    = 3, /* 64x64 tiles, all f32 (ops.cpp:8347-8633)                    */
    VOXO_PATH_F64      = 4, /* plain softmax(QK^T)V in double; cross-check only            */
    VOXO_PATH_SPLIT_KV = 5  /* VOXO_PATH_ROW over n_chunks KV ranges + merge                */
                            /* (ops.cpp:8758-8786, 8637-8705)                              */
};

/* a tensor in the reference's terms: type, extents, byte strides (ggml.h:655-687) */
typedef struct {
    int          type;
    int64_t      ne[4];
    size_t       nb[4];
    const void * data;
} voxo_tensor;

uint16_t voxo_fp32_to_fp16(float f);
float    voxo_fp16_to_fp32(uint16_t h);

/* 34-byte blocks: fp16 scale + 32 int8 (ggml-common.h:221-224) */
void voxo_quantize_row_q8_0(const float * x, void * y, int64_t n);   /* ggml-quants.c:199-222 */
void voxo_dequantize_row_q8_0(const void * x, float * y, int64_t n); /* ggml-quants.c:401-415 */

/* softmax(scale * Q K^T + mask) V with GQA broadcast.
 *   q    [D, n_q,  H,  B] f32        k, v [D, n_kv, HK, B] f32 | f16 | q8_0
 *   mask NULL or [n_kv, n_q, ne2, ne3] f16 (broadcast: head %% ne2, batch %% ne3)
 *   dst  [D, H, n_q, B] f32, contiguous (the operator's permuted result, ops.cpp:8342)
 * n_chunks is used by VOXO_PATH_SPLIT_KV only.  Returns 0, or non-zero for a shape or
 * type the reference would reject. */
int voxo_flash_attn_ext(const voxo_tensor * q, const voxo_tensor * k, const voxo_tensor * v,
                        const voxo_tensor * mask, float scale, int path, int n_chunks, float * dst);

/* f16 causal mask [total_len, n_tok] for query positions pos[0..n_tok)
 * (src/minicpm.cpp:602-620): -inf where key > query, -0 elsewhere. */
void voxo_causal_mask(const int32_t * pos, int n_tok, int total_len, uint16_t * mask);

/* f16 block-diagonal mask [2*seq, 2*seq] that isolates the two CFG branches packed along
 * the sequence axis (src/locdit.cpp:63-130): 0 inside a branch, -inf across. */
void voxo_cfg_pair_mask(int seq, uint16_t * mask);

/* KV-cache append semantics: n rows of D floats stored as f16 (GGML_FP32_TO_FP16) or
 * q8_0 (quantize_row_q8_0_ref), what ggml_cpy into an f16 / q8_0 cache tensor does
 * (src/minicpm.cpp:684-685). */
void voxo_kv_store(const float * x, int64_t n_rows, int64_t D, int type, void * dst);

/* Rotary position embedding as MiniCPMModel::apply_rope asks for it (src/minicpm.cpp:582-600:
 * ggml_rope_ext, GGML_ROPE_TYPE_NEOX, freq_scale 1, ext_factor 0, optional per-frequency
 * factors, attn_factor on cos and sin).
 *   voxo_rope_table: table[p][i] = (cos, sin) of theta_i / ff_i, times attn_factor, for
 *     n_pos positions and i < n_dims/2, with theta_0 = pos and theta_{i+1} = theta_i *
 *     powf(freq_base, -2/n_dims) (ggml_rope_cache_init, rope_yarn:
 *     third_party/ggml/src/ggml-cpu/ops.cpp:5596-5629, theta_scale at :5778).
 *   voxo_rope_neox: rotates n_rows rows of n_dims floats in place, pairing element i with
 *     element i + n_dims/2 (rotate_pairs, ops.cpp:5701-5718); row r uses the table entry of
 *     position index pos_index[r]. */
void voxo_rope_table(const int32_t * pos, int64_t n_pos, int n_dims, float freq_base, float attn_factor,
                     const float * freq_factors, float * table);
void voxo_rope_neox(float * x, int64_t n_rows, int n_dims, const float * table, const int32_t * pos_index);

#ifdef __cplusplus
}
#endif
/* ggml_mul_mat with f16 weights (ggml-cpu.c:217, vec.cpp:264): activations rounded to f16, f32 accumulation.
 *   x [n_tok][k] f32, w [n_out][k] f16 bits, out [n_tok][n_out] f32 */
void voxo_mul_mat_f16(const float * x, const uint16_t * w, int64_t n_tok, int64_t k, int64_t n_out, float * out);
/* MiniCPMModel::rms_norm (src/minicpm.cpp:572-580): ggml_rms_norm, then ggml_mul with the weight.  x, out [n_tok][k], w [k] */
void voxo_rms_norm_mul(const float * x, const float * w, float eps, int64_t n_tok, int64_t k, float * out);
/* ggml_swiglu_split(gate, up): silu(gate) * up, element by element */
void voxo_swiglu(const float * gate, const float * up, int64_t n, float * out);

#endif
