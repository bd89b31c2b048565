/* vox_attn.h — C ABI of the B200 (sm_100a) attention engine for VoxCPM.cpp.
 *
 * The engine implements the operator that VoxCPM.cpp reaches through
 * ggml_flash_attn_ext (third_party/ggml/include/ggml.h:2311-2330, called from
 * src/minicpm.cpp:708-710 for the backbone LM, the residual LM, LocEnc and LocDiT):
 *
 *     dst = softmax(scale * Q K^T + mask) V      with GQA broadcast of K/V heads
 *
 * plus the KV cache that feeds it (MiniCPMKVCache, include/voxcpm/minicpm.h:44-84) and the
 * batched forms VoxCPM.cpp's loops need (one launch for many synthesis streams; one launch
 * for all layers and both CFG branches of a LocDiT timestep).
 *
 * Conventions
 *   - plain C, no CUDA or torch types: device pointers are void*, a CUDA stream is passed
 *     as void* (cudaStream_t), NULL meaning the legacy default stream;
 *   - tensors are described as ggml describes them: element type, ne[4] extents with
 *     dim 0 fastest, nb[4] strides in BYTES (ggml.h:655-687);
 *   - every function returns a vox_status; nothing aborts, nothing falls back to the CPU;
 *   - all launches are asynchronous on the caller's stream; an engine (and everything
 *     created from it) belongs to one device and may be used by one host thread at a time.
 */
#ifndef VOX_ATTN_H
#define VOX_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    VOX_ATTN_OK                  = 0,
    VOX_ATTN_INVALID_ARGUMENT    = 1, /* null pointer, bad extent/stride, out-of-range index   */
    VOX_ATTN_UNSUPPORTED         = 2, /* valid for the reference operator, not built here       */
    VOX_ATTN_WORKSPACE_TOO_SMALL = 3,
    VOX_ATTN_CUDA_ERROR          = 4, /* a CUDA runtime/driver call failed; see error string    */
    VOX_ATTN_TIMEOUT             = 5, /* a bounded device-side wait ran out (status word)       */
    VOX_ATTN_OUT_OF_MEMORY       = 6,
    VOX_ATTN_DEVICE_STATE        = 7  /* a kernel found device-side state that does not fit the call: a
                                         stream's kv_len beyond its cache rows (status word); the row was
                                         not stored                                                     */
} vox_status;

/* numbered as ggml numbers them (ggml.h enum ggml_type) */
typedef enum {
    VOX_TYPE_F32  = 0,
    VOX_TYPE_F16  = 1,
    VOX_TYPE_Q8_0 = 8  /* 34-byte blocks: fp16 scale + 32 int8 (ggml-common.h:221-224) */
} vox_type;

/* mirrors the fields of ggml_tensor the operator reads (ggml.h:655-687) */
typedef struct {
    int32_t type;   /* vox_type */
    int64_t ne[4];
    size_t  nb[4];  /* bytes */
    void *  data;   /* device pointer (host pointer for the *_host entry points) */
} vox_tensor;

/* replaces the argument list of ggml_flash_attn_ext (ggml.h:2322-2330):
 *   q    [D, n_q,  H,  B] f32          k, v [D, n_kv, HK, B] f32 | f16 | q8_0, rows contiguous
 *   mask data==NULL, or [n_kv, n_q, ne2, ne3] f16 contiguous, broadcast over heads/batch
 *   dst  [D, H, n_q, B] f32  (permuted against q exactly as the reference result is)      */
typedef struct {
    vox_tensor q, k, v, mask, dst;
    float      scale;
    float      max_bias;      /* must be 0: ALiBi is never used by VoxCPM.cpp             */
    float      logit_softcap; /* must be 0                                                  */
    int32_t    has_sinks;     /* must be 0 (ggml_flash_attn_ext_add_sinks is never called)  */
} vox_attn_args;

typedef struct vox_engine   vox_engine;
typedef struct vox_kv_cache vox_kv_cache;
typedef struct vox_group    vox_group;

/* ---------------------------------------------------------------- engine --------------- */

/* Replaces backend selection in VoxCPMBackend (src/backend.cpp:146-205): binds to one CUDA
 * device, fails with VOX_ATTN_UNSUPPORTED unless it is compute capability 10.x. */
int  vox_engine_create(int device, vox_engine ** out);
void vox_engine_destroy(vox_engine * e);

/* Text of the last failure on the calling thread (replaces GGML_ASSERT / CUDA_CHECK abort
 * messages, third_party/ggml/src/ggml-cuda/common.cuh CUDA_CHECK). */
const char * vox_attn_last_error_string(void);
const char * vox_attn_status_string(int status);

/* Kernel launches issued through this engine so far (the launch-count metric). */
uint64_t vox_engine_launch_count(const vox_engine * e);

/* Synchronise `stream` and fold the device status word into a status: VOX_ATTN_TIMEOUT when
 * a kernel's bounded wait gave up.  Replaces the ggml_status returned by
 * ggml_backend_graph_compute (src/backend.cpp:564-570).  Clears the word. */
int vox_engine_sync_status(vox_engine * e, void * stream);

/* Failure-path self-test without a fault: launches one thread that waits, for at most limit_cycles SM
 * clock cycles (<= 2e9), on a barrier nothing ever arrives at.  The wait gives up the way every bounded
 * wait of the engine's kernels does: it raises the device status word and the kernel returns normally.
 * The next vox_engine_sync_status reports VOX_ATTN_TIMEOUT and the context stays usable.  (The reference
 * has no counterpart: a stuck ggml-cuda kernel ends in the driver's watchdog or not at all.) */
int vox_engine_selftest_wait(vox_engine * e, long long limit_cycles, void * stream);

/* ---------------------------------------------------------------- generic operator ----- */

/* Replaces ggml_cuda_flash_attn_ext_supported (third_party/ggml/src/ggml-cuda/fattn.cu:480-482).
 * Pure host function: 1 if vox_attn_forward accepts these operands, else 0. */
int vox_attn_supported(const vox_attn_args * a);

/* Scratch bytes vox_attn_forward needs for these operands (replaces the pool allocations of
 * launch_fattn, third_party/ggml/src/ggml-cuda/fattn-common.cuh:808-818). */
size_t vox_attn_workspace_bytes(const vox_attn_args * a);

/* Replaces ggml_cuda_flash_attn_ext (fattn.cu:460-478) / ggml_compute_forward_flash_attn_ext
 * (third_party/ggml/src/ggml-cpu/ops.cpp:8838-8853).  Routes by shape: n_q==1 with f16 K/V, or
 * q8_0 K/V and the workspace vox_attn_workspace_bytes names (the blocks are taken apart into tiles
 * there) -> split-KV decode kernel; 32 or more keys with a mask (the
 * reference's prefill call, src/minicpm.cpp:708-710, with the tensor create_causal_mask built, or
 * any other additive f16 mask whose rows start on 16-byte boundaries, n_kv a multiple of 8) ->
 * tcgen05 kernel, which reads the mask (see vox_attn_prefill for the form that implies it; q8_0
 * and f32 K/V need the workspace vox_attn_workspace_bytes names; with that workspace a small kernel
 * first marks the key tiles the mask hides altogether, which are then not walked, and those it adds
 * nothing to, which are then not read), and so do two or more queries
 * over 32 or more keys without a mask; anything else the contract allows (any
 * n_q/n_kv, f32/f16/q8_0 K/V, arbitrary f16 mask, strides) -> general kernel.  Never allocates. */
int vox_attn_forward(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes,
                     void * stream);

/* Same operator with HOST tensors: copies q/k/v/mask to the device, runs, copies dst back and
 * synchronises.  Uses engine-owned staging buffers that grow on demand. */
int vox_attn_forward_host(vox_engine * e, const vox_attn_args * a, void * stream);

/* Causal prefill without a materialised mask (the mask MiniCPMModel::create_causal_mask builds,
 * src/minicpm.cpp:602-620, is implied: key j visible to query i iff j <= i + n_kv - n_q).
 * q [D, n_q, H, B] f32; k, v [D, n_kv, HK, B] f16, or q8_0 / f32 when a workspace of
 * vox_attn_prefill_workspace_bytes is passed (they are expanded there into f16 value + remainder
 * tiles first): runs on tcgen05/TMEM.  Unaligned strides, and q8_0 / f32 K/V without a workspace,
 * take the general kernel. */
int vox_attn_prefill(vox_engine * e, const vox_attn_args * a, void * workspace, size_t workspace_bytes,
                     void * stream);
size_t vox_attn_prefill_workspace_bytes(const vox_attn_args * a);

/* ---------------------------------------------------------------- KV cache ------------- */

/* Replaces MiniCPMKVCache (src/minicpm.cpp:144-271).  Storage is f16 or q8_0 instead of the
 * reference's F32 and holds many independent streams:
 *   f16 : K and V as [layer][stream][kv_head][pos][64] halves
 *   q8_0: [layer][stream][kv_head][tile], a tile = 64 rows in one span of 8704 bytes: the bytes
 *         of K (each q + 128), the bytes of V, two f16 scales per row of K, then of V — the
 *         values of block_q8_0, laid out so that the decode kernel fetches a tile with one
 *         bulk copy; vox_kv_export / vox_kv_import speak the reference's 34-byte blocks.      */
typedef struct {
    int32_t n_layers, n_streams, n_kv_heads, head_dim /* 64 */, max_len, type /* F16 | Q8_0 */;
} vox_kv_config;

int  vox_kv_create(vox_engine * e, const vox_kv_config * cfg, vox_kv_cache ** out); /* MiniCPMKVCache::init  */
void vox_kv_destroy(vox_kv_cache * c);
int  vox_kv_clear(vox_kv_cache * c, int stream_id /* -1: all */, void * stream);    /* MiniCPMKVCache::clear */
size_t vox_kv_bytes(const vox_kv_cache * c);                                        /* ::buffer_size         */

/* Replaces ggml_cpy into get_k_batch/get_v_batch views (src/minicpm.cpp:684-685, 222-236) and
 * the concat(past, cur) that follows (:696-701): rounds f32 rows to f16 (GGML_FP32_TO_FP16) or
 * quantises them (quantize_row_q8_0_ref, third_party/ggml/src/ggml-quants.c:199-222) in place.
 *   k, v      [D, HK, n_tok, n_streams] f32 on the device; strides in bytes
 *   positions device array [n_streams]: first cache row written for each stream (NULL: `pos0`)
 * Rows land at positions[s] .. positions[s]+n_tok-1 of every stream s < n_streams. */
int vox_kv_append(vox_kv_cache * c, int layer, int n_streams, int n_tok, const int32_t * positions, int pos0,
                  const float * k, const float * v, size_t nb_head, size_t nb_tok, size_t nb_stream,
                  void * stream);

/* Replaces MiniCPMKVCache::get_k / get_v (src/minicpm.cpp:200-212): describes the first
 * seq_len rows of one stream's K and V for `layer` as operator tensors [64, seq_len, HK, 1].
 * Only an f16 cache can be viewed as a ggml tensor; a q8_0 cache returns UNSUPPORTED (use
 * vox_attn_decode, or vox_kv_export to get block_q8_0 rows). */
int vox_kv_view(const vox_kv_cache * c, int layer, int stream_id, int seq_len, vox_tensor * k, vox_tensor * v);

/* Host <-> cache in the reference's storage formats (f16 rows, or block_q8_0 rows of 68 bytes),
 * rows ordered [kv_head][pos].  Replaces backend.tensor_get/tensor_set on raw_k_cache()
 * (src/minicpm.cpp:252-271).  Synchronous. */
int vox_kv_export(const vox_kv_cache * c, int layer, int stream_id, int n_pos, void * k_host, void * v_host);
int vox_kv_import(vox_kv_cache * c, int layer, int stream_id, int n_pos, const void * k_host, const void * v_host);
int vox_kv_copy_from(vox_kv_cache * dst, const vox_kv_cache * src, void * stream); /* ::copy_from */

/* ---------------------------------------------------------------- rotary embedding ------ */

/* Rotary position embedding of the decode step.  MiniCPMModel::apply_rope (src/minicpm.cpp:582-600)
 * issues ggml_rope_ext (GGML_ROPE_TYPE_NEOX, n_dims = 64, freq_scale 1, ext_factor 0) on Q and on K
 * in every layer, each time rebuilding the cos/sin cache of the token's position.  Here the table is
 * built once per step and the decode launch rotates Q and the arriving K row itself.
 *   freq_base     llama.rope.freq_base
 *   attn_factor   1, or the magnitude factor apply_rope derives beyond the original context
 *   freq_factors  device pointer to 32 floats (rope_short_factor / rope_long_factor), or NULL    */
typedef struct {
    float         freq_base;
    float         attn_factor;
    const float * freq_factors;
} vox_rope_config;

/* table[s][i] = (cos, sin)(theta_i / freq_factors[i]) * attn_factor for stream s at position
 * positions[s] + pos_offset, i < 32; theta_0 = position, theta_{i+1} = theta_i * freq_base^(-2/64)
 * (ggml_rope_cache_init).  positions is a device array; table is device memory of
 * n_streams * 64 floats.  One launch. */
int vox_rope_table(vox_engine * e, const vox_rope_config * cfg, const int32_t * positions, int pos_offset,
                   int n_streams, float * table, void * stream);

/* ---------------------------------------------------------------- Q/K/V projection ------ */

/* The three graph nodes in front of attention in MiniCPMModel::attention_forward (src/minicpm.cpp:644-701), for the
 * single-token step of n_streams streams in ONE launch (plus a small one that rounds the activations to f16):
 * ggml_mul_mat(qkv_proj, hidden) (:660-686, or q_proj / k_proj / v_proj stacked into one matrix), apply_rope on q and
 * k (:688-689, :582-600) and the ggml_cpy of the new K and V rows into the cache views (:684-685).  The reference
 * runs them per stream, reading the projection weights once per stream and step; here they are read once per step.
 * Arithmetic as ggml's CPU backend does it for f16 weights (activations rounded to f16, f32 accumulation:
 * third_party/ggml/src/ggml-cpu/ggml-cpu.c:217, ggml-cpu/vec.cpp:264), on tcgen05 tensor cores.
 *   x          [hidden, n_streams] f32: the normed hidden state of each stream's token; x_nb_stream bytes apart
 *   w_qkv      [hidden, (H + 2 HK) * 64] f16 in ggml's layout (a weight row per output feature, hidden contiguous;
 *              Q rows first, then K, then V, as qkv_proj stores them); w_nb_row bytes between rows; w_type VOX_TYPE_F16
 *   rope_table optional, from vox_rope_table for these streams' positions: q and k leave rotated (NULL: not rotated)
 *   q          out [64, H, n_streams] f32 contiguous: what vox_attn_decode reads with q_nb_head = 256, q_nb_stream = H * 256
 *   cache, layer, positions   the K and V rows go straight into the cache (converted as vox_kv_append converts them),
 *              stream s's at row positions[s] + pos_offset (device array): the decode call that follows then takes
 *              kv_len = that row + 1 and no k_new / v_new.  Or, with cache == NULL:
 *   k_new, v_new   out [64, HK, n_streams] f32 contiguous, for the decode launch's own store (its k_new / v_new;
 *              with rope_table given here, pass none there).
 * workspace: vox_qkv_workspace_bytes (the f16 copy of x), 16-byte aligned.  Never allocates. */
typedef struct {
    int32_t         n_streams, hidden, n_heads, n_kv_heads, head_dim /* 64 */;
    const float *   x;
    size_t          x_nb_stream;
    const void *    w_qkv;
    size_t          w_nb_row;
    int32_t         w_type;
    const float *   rope_table;
    float *         q;
    float *         k_new;
    float *         v_new;
    vox_kv_cache *  cache;
    int32_t         layer;
    const int32_t * positions;
    int32_t         pos_offset; /* added to every positions[s] (-1 when positions holds the lengths after the step) */
} vox_qkv_args;

size_t vox_qkv_workspace_bytes(int n_streams, int hidden);
int    vox_qkv_project(vox_engine * e, const vox_qkv_args * a, void * workspace, size_t workspace_bytes, void * stream);

/* ---------------------------------------------------------------- linear layers of a step - */

/* The other weight matrices of a decoder layer, for the single-token step of n_tokens streams in ONE launch each (plus a
 * small one that rounds the activations to f16): the reference runs ggml_mul_mat per stream, reading every matrix once
 * per stream and step.
 *   VOX_LINEAR_PLAIN     out = W x                          ggml_mul_mat (e.g. o_proj, src/minicpm.cpp:715)
 *   VOX_LINEAR_RESIDUAL  out = residual + scale * (W x)     + ggml_scale and ggml_add of layer_forward (:765-768, :773-776)
 *   VOX_LINEAR_SWIGLU    out = silu(W_gate x) * (W_up x)    ggml_mul_mat(gate_up_proj) + ggml_swiglu_split (:718-746);
 *                        w holds 2 * n_out rows, the gate rows first, as gate_up_proj stores them
 * With norm_weight given, x is first normalised as MiniCPMModel::rms_norm does (:572-580: ggml_rms_norm with norm_eps,
 * then ggml_mul with the weight).  Arithmetic as ggml's CPU backend (activations rounded to f16, exact products, f32
 * sums), on tcgen05 tensor cores; the order of the f32 sums differs, so results agree to about 1e-6 of their RMS.
 *   x     [k_dim, n_tokens] f32, x_nb_token bytes between tokens
 *   w     [k_dim, rows] f16 in ggml's layout (a row per output feature, k_dim contiguous), w_nb_row bytes between rows
 *   out   [n_out, n_tokens] f32, out_nb_token bytes between tokens; residual likewise (may be out itself)
 *   x_type, out_type   VOX_TYPE_F32 (0, the default) or VOX_TYPE_F16.  The product rounds its activations to f16 in any
 *         case, so a layer whose output only feeds another product (the SwiGLU output in front of down_proj) may leave
 *         as f16 and enter the next call as f16: same values, no conversion launch, half the bytes.  f16 x comes without
 *         norm_weight; f16 out comes without a residual.
 * k_dim a multiple of 64; n_out a multiple of 64 (32 for SwiGLU).
 * workspace: vox_linear_workspace_bytes (the f16 copy of x; none needed for f16 x), 16-byte aligned.  Never allocates. */
enum vox_linear_mode { VOX_LINEAR_PLAIN = 0, VOX_LINEAR_RESIDUAL = 1, VOX_LINEAR_SWIGLU = 2 };
typedef struct {
    int32_t       n_tokens, k_dim, n_out;
    int32_t       mode;
    const void *  x;
    size_t        x_nb_token;
    const void *  w;
    size_t        w_nb_row;
    int32_t       w_type; /* VOX_TYPE_F16 */
    void *        out;
    size_t        out_nb_token;
    const float * residual;
    size_t        res_nb_token;
    float         scale;
    const float * norm_weight; /* [k_dim] f32 or NULL */
    float         norm_eps;
    int32_t       x_type, out_type;
} vox_linear_args;

size_t vox_linear_workspace_bytes(int n_tokens, int k_dim);
int    vox_linear(vox_engine * e, const vox_linear_args * a, void * workspace, size_t workspace_bytes, void * stream);

/* ---------------------------------------------------------------- decode --------------- */

/* One-token attention for n_streams independent streams in ONE launch (the K/V rows of all
 * streams are cut into equal runs, one per CTA; the CTA that finishes a stream's last run folds
 * the partial results).  Replaces the n_q==1 call made by MiniCPMModel::forward_step
 * (src/minicpm.cpp:813-846) once per stream.
 *   q        [D, 1, H, n_streams] f32 (strides q_nb_head, q_nb_stream in bytes)
 *   kv_len   device array [n_streams]: rows of each stream that are visible (after append)
 *   kv_bound host-known upper bound of every kv_len (sizes the grid; <= max_len)
 *   dst      [D, H, 1, n_streams] f32, contiguous
 *   k_new, v_new  optional (both or neither), [D, HK, n_streams] f32 with strides new_nb_head,
 *            new_nb_stream in bytes: the token's own K/V rows.  The reference stores them with
 *            ggml_cpy just before the attention node (src/minicpm.cpp:684-701); given here, the
 *            decode launch does that store itself: stream s's row goes to position kv_len[s]-1
 *            (converted exactly as vox_kv_append converts it) and takes part in this call's
 *            attention, so no append launch is needed.  A stream whose kv_len exceeds the cache
 *            capacity writes nothing and raises the engine's status (vox_engine_sync_status).
 *            The cache is written: do not run two such calls on one layer concurrently.
 *   rope_table  optional: the table vox_rope_table built for these streams' positions
 *            (kv_len - 1).  q and k_new are then the projections BEFORE the rotary embedding
 *            and the launch rotates them (element i with element i + 32) as it reads them;
 *            v_new is stored as it is.  NULL: q and k_new are already rotated.
 *   stream_order  optional device array, a permutation of [0, n_streams): the order in which the
 *            streams are laid end to end before the rows are cut into runs.  Every CTA gets an equal
 *            share of the rows whatever the order, so it only decides which streams share a CTA;
 *            the outputs agree to rounding of the f32 folds (NULL: 0, 1, 2, ...).
 *   flags    VOX_DECODE_CACHE_STABLE: a promise that neither kv_len nor any cache row this call reads
 *            was written by the kernel launched just before it on the same stream (q, k_new and
 *            v_new may have been).  True for the layers of a model, where a projection GEMM
 *            precedes attention and the cache rows are at least one step old.  The launch then
 *            requests its first K/V tiles before its programmatic-dependency wait, i.e. while the
 *            previous kernel drains.                                                           */
#define VOX_DECODE_CACHE_STABLE 1u
typedef struct {
    const vox_kv_cache * cache;
    int32_t         layer;
    int32_t         n_streams;
    int32_t         n_heads;
    const int32_t * kv_len;
    int32_t         kv_bound;
    const float *   q;
    size_t          q_nb_head, q_nb_stream;
    float *         dst;
    float           scale;
    const float *   k_new;
    const float *   v_new;
    size_t          new_nb_head, new_nb_stream;
    uint32_t        flags;
    const float *   rope_table;
    const int32_t * stream_order;
} vox_decode_args;

size_t vox_attn_decode_workspace_bytes(int n_streams, int n_heads, int n_kv_heads, int kv_bound);
int    vox_attn_decode(vox_engine * e, const vox_decode_args * a, void * workspace, size_t workspace_bytes,
                       void * stream);

/* vox_attn_decode for callers that cannot allocate device memory and so have no workspace to
 * pass: a real-time audio thread that must stay out of the allocator, a host that gave all device
 * memory to its own arena at start-up, a plugin that is handed nothing but its inputs and
 * outputs.  It has no counterpart in the reference.  Same arguments and results as
 * vox_attn_decode; the split-KV partials go to a 4 MiB array built into the library (each GPU
 * that loads the library holds it until the process exits), and the call performs no allocation
 * of any kind.  The arguments are validated exactly as vox_attn_decode validates them, before
 * anything is derived from them.
 *   - A launch needs two partial slots per CTA of a grid that never exceeds one wave (2 x CTAs x
 *     n_heads / n_kv_heads x 264 bytes: 2.4 MiB on a 148-SM device with 8 heads per kv head).  A
 *     call whose plan needs more than 4 MiB (ask vox_attn_decode_workspace_bytes) returns
 *     VOX_ATTN_WORKSPACE_TOO_SMALL and launches nothing.
 *   - The engine's device must be the current device.  The first call on a device looks up the
 *     array's device address; make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Nothing in it needs clearing between calls, but
 *     two calls whose kernels overlap on the GPU (different streams) overwrite each other's
 *     partials: keep calls on one stream, or order them yourself. */
int    vox_attn_decode_static(vox_engine * e, const vox_decode_args * a, void * stream);

/* ---------------------------------------------------------------- LocDiT --------------- */

/* All attention of ONE CFM timestep in ONE launch: every layer, both CFG branches, every head,
 * for n_streams patches.  Replaces the 8 ggml_flash_attn_ext nodes (18 packed tokens +
 * block-diagonal mask) that LocDiTModel::forward_cfg_pair_projected emits per evaluation
 * (src/locdit.cpp:401-464, 63-130) inside UnifiedCFM::solve_euler (src/unified_cfm.cpp:88-149).
 * Bidirectional, no mask, f32 in and out.
 *   q   [D, seq, H,  2, n_layers, n_streams] f32 contiguous
 *   k,v [D, seq, HK, 2, n_layers, n_streams] f32 contiguous
 *   dst [D, H, seq, 2, n_layers, n_streams] f32 contiguous                                  */
typedef struct {
    int32_t       n_streams, n_layers, n_heads, n_kv_heads, seq /* <= 16 */, head_dim /* 64 */;
    const float * q;
    const float * k;
    const float * v;
    float *       dst;
    float         scale;
} vox_locdit_args;

int vox_attn_locdit_step(vox_engine * e, const vox_locdit_args * a, void * stream);

/* ---------------------------------------------------------------- stream groups -------- */

/* A group is the set of synthesis streams one GPU serves: a backbone cache, a residual-LM
 * cache, per-stream lengths, and the step that VoxCPMRuntime::decode (src/voxcpm.cpp:1027-1128)
 * performs as far as attention is concerned: per layer append + decode attention for both LM
 * stacks, then cfm_steps LocDiT launches for the patch. */
typedef struct {
    int32_t n_streams;
    int32_t base_layers, res_layers;       /* 24, 6 */
    int32_t n_heads, n_kv_heads, head_dim; /* 16, 2, 64 */
    int32_t max_len;
    int32_t kv_type;                       /* VOX_TYPE_F16 | VOX_TYPE_Q8_0 */
    int32_t locdit_layers, locdit_seq, cfm_steps; /* 8, 9, 10 */
    /* Timesteps at the start of a patch that evaluate no network: UnifiedCFM::solve_euler with
     * cfg-zero-star sets dphi_dt = 0 for step <= max(1, 0.04 * (n_steps + 1)) (src/unified_cfm.cpp:107-116),
     * i.e. 1 of 10.  Those steps issue no launch, move no data in vox_group_step_host and leave their
     * slice of dit_out untouched.  0: every timestep evaluates the network. */
    int32_t cfm_zero_init_steps;
} vox_group_config;

/* Device (or, for vox_group_step_host, pinned host) buffers of one step.
 *   lm_q      [D, 1, H,  S, L] f32   L = base_layers + res_layers, S = n_streams
 *   lm_k_new  [D, HK, 1, S, L] f32   rows appended at position kv_len[s] before attending
 *   lm_v_new  same
 *   lm_out    [D, H, 1, S, L] f32
 *   lm_hidden [hidden, S, L] f32   (only with vox_group_set_qkv_weights, instead of the three inputs above)
 *   dit_q     [D, seq, H,  2, locdit_layers, S, cfm_steps] f32;  dit_k, dit_v with HK
 *   dit_out   [D, H, seq, 2, locdit_layers, S, cfm_steps] f32
 * vox_group_step skips the LM stacks when lm_q is NULL and the LocDiT patch when dit_q is NULL.  */
typedef struct {
    const float * lm_q;
    const float * lm_k_new;
    const float * lm_v_new;
    float *       lm_out;
    const float * dit_q;
    const float * dit_k;
    const float * dit_v;
    float *       dit_out;
    /* With projection weights set (vox_group_set_qkv_weights): [hidden, S, L] f32, the normed hidden state of every
     * stream's token for every LM layer, INSTEAD of lm_q / lm_k_new / lm_v_new (which must then be NULL).  Every layer
     * becomes projection (with the rotary embedding when the group has it set) + decode attention. */
    const float * lm_hidden;
} vox_step_buffers;

int  vox_group_create(vox_engine * e, const vox_group_config * cfg, vox_group ** out);
void vox_group_destroy(vox_group * g);
vox_kv_cache * vox_group_cache(vox_group * g, int stack /* 0 backbone, 1 residual */);
/* Set every stream's current length (host array [n_streams]); synchronous. */
int vox_group_set_kv_len(vox_group * g, const int32_t * kv_len);
int vox_group_get_kv_len(const vox_group * g, int32_t * kv_len);
/* Fill both caches' first kv_len[s] rows of every stream with N(0,1) values from a counter-based
 * generator seeded with `seed` (synthetic prompt state for benchmarks). */
int vox_group_fill_synthetic(vox_group * g, uint64_t seed, void * stream);
size_t vox_group_step_bytes(const vox_group * g, int which /* 0 lm in, 1 lm out, 2 dit in, 3 dit out */);
/* Rotary embedding inside the step: with a configuration set, lm_q and lm_k_new of vox_step_buffers are the
 * projections BEFORE apply_rope (src/minicpm.cpp:582-600); each step builds one cos/sin table for the
 * streams' positions (one launch) and every layer's decode launch rotates Q and the arriving K row.
 * freq_factors_host: 32 floats on the host (copied), or NULL.  cfg == NULL switches it off again. */
int vox_group_set_rope(vox_group * g, const vox_rope_config * cfg, const float * freq_factors_host);
/* Q/K/V projection inside the step (src/minicpm.cpp:660-686 for every LM layer): w is a device array of
 * base_layers + res_layers matrices [hidden, (H + 2 HK) * 64] f16 in ggml's layout, nb_layer bytes apart, rows nb_row
 * bytes apart (they stay the caller's).  vox_group_step then takes lm_hidden of vox_step_buffers.  w == NULL: off. */
int vox_group_set_qkv_weights(vox_group * g, const void * w, int hidden, size_t nb_row, size_t nb_layer);

/* Position-independent step (the reference rebuilds and re-reserves its step graph at every position,
 * src/voxcpm.cpp:485-513).  Lengths live on the device and are advanced there, so the launch sequence of
 * vox_group_step depends on the position only through the sizes of its grids.  vox_group_set_bound fixes
 * those to "lengths up to kv_bound" (0: back to the exact longest stream): a step can then be captured
 * into a CUDA graph (cudaStreamBeginCapture on the stream handed to vox_group_step; the programmatic
 * dependencies between the launches are captured with them) and replayed for every position until a stream
 * reaches the bound.  A captured step records launches only; after each replay of an advancing step call
 * vox_group_advance(g, 1) so that the host copy of the lengths follows the device. */
int vox_group_set_bound(vox_group * g, int kv_bound);
int vox_group_advance(vox_group * g, int steps);

/* One decode step on device buffers.  advance != 0 stores the new rows and grows every stream
 * by one position; advance == 0 attends to the current rows only (lengths fixed).
 * Launches: one per LM layer (it stores the arriving row and folds the split-KV partials itself), one
 * length update, one rotary table when set, one per CFM step. */
int vox_group_step(vox_group * g, const vox_step_buffers * dev, int advance, void * stream);
/* The same step from pinned HOST buffers: H2D of the inputs, the launches, D2H of the outputs,
 * overlapped on the group's own streams; returns after the outputs have landed. */
int vox_group_step_host(vox_group * g, const vox_step_buffers * host, int advance);

/* Longest-processing-time partition of streams over GPUs by KV length (pure host function):
 * owner[s] in [0, n_gpus) such that the per-GPU sums of kv_len are balanced. */
int vox_partition_streams(const int32_t * kv_len, int n_streams, int n_gpus, int32_t * owner);

#ifdef __cplusplus
}
#endif
#endif /* VOX_ATTN_H */
