// Stream groups: the synthesis streams one GPU serves and the attention part of one decode
// step for all of them at once.
//
// Replaces, for attention, the per-stream loop of VoxCPMRuntime::decode
// (src/voxcpm.cpp:1027-1128): there each stream rebuilds a ggml graph per position
// (:485-544), runs 24 + 6 single-token attention nodes and one unrolled CFM solve with
// 8 attention nodes per evaluation.  Here every LM layer is ONE decode launch for ALL streams of
// the group (it stores the arriving K/V row and folds the split-KV partials itself), and every CFM
// timestep that evaluates the network is one launch.  Streams never exchange data, so several GPUs
// each run their own group with no collective; vox_partition_streams assigns streams to GPUs.
#include "kv_cache.cuh"

#include <algorithm>
#include <cstring>
#include <new>
#include <numeric>
#include <vector>

using namespace vox;

namespace vox {
int kv_fill_synthetic(vox_kv_cache * c, const int32_t * kv_len_dev, uint64_t seed, cudaStream_t stream);
}

struct vox_group {
    vox_engine *     e = nullptr;
    vox_group_config cfg{};
    vox_kv_cache *   cache[2]  = {nullptr, nullptr};  // backbone, residual LM
    int32_t *        kv_len_dev = nullptr;            // [n_streams] rows visible to attention
    std::vector<int32_t> kv_len_host;
    int              kv_bound  = 0;                   // longest stream (host copy)
    int              grid_bound = 0;                  // vox_group_set_bound: grids are sized for this length instead (0: exact)
    void *           workspace = nullptr;
    size_t           workspace_bytes = 0;
    // rotary embedding inside the step (vox_group_set_rope): one table per step, applied by every layer's decode
    bool             rope_on = false;
    vox_rope_config  rope{};
    float *          rope_factors = nullptr;          // device copy of the 32 per-frequency factors
    float *          rope_table   = nullptr;          // [n_streams][32][2]
    // Q/K/V projection inside the step (vox_group_set_qkv_weights): the caller's weights, and the group's own rows for
    // one layer's q, k, v and the f16 copy of its activations
    const uint8_t *  qkv_w = nullptr;
    int              qkv_hidden = 0;
    size_t           qkv_nb_row = 0, qkv_nb_layer = 0;
    float *          proj_q = nullptr;                // [S][H][64], then [S][HK][64] x 2
    void *           proj_ws = nullptr;
    size_t           proj_ws_bytes = 0;
    // vox_group_step_host: device mirrors of the step buffers, two copy streams, events
    uint8_t *        dev_buf   = nullptr;
    size_t           dev_off[8] = {0};
    cudaStream_t     st_compute = nullptr, st_copy = nullptr, st_back = nullptr;  // launches, host-to-device, device-to-host
    cudaEvent_t      ev_lm_in = nullptr, ev_dit_in[16] = {nullptr}, ev_lm_done = nullptr, ev_dit_done[16] = {nullptr};
};

namespace {

__global__ void add_scalar_kernel(int32_t * a, int n, int delta, int cap) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    if (i < n) a[i] = min(a[i] + delta, cap);
}

size_t lm_layers(const vox_group_config & c) { return (size_t) c.base_layers + c.res_layers; }

size_t step_bytes(const vox_group_config & c, int which) {
    const size_t S = c.n_streams, D = c.head_dim;
    switch (which) {
        case 0: return lm_layers(c) * S * (c.n_heads + 2 * (size_t) c.n_kv_heads) * D * 4;            // q + k_new + v_new
        case 1: return lm_layers(c) * S * c.n_heads * D * 4;                                            // lm_out
        case 2: return (size_t) (c.cfm_steps - c.cfm_zero_init_steps) * S * c.locdit_layers * 2 * c.locdit_seq * (c.n_heads + 2 * (size_t) c.n_kv_heads) * D * 4;
        case 3: return (size_t) (c.cfm_steps - c.cfm_zero_init_steps) * S * c.locdit_layers * 2 * c.locdit_seq * c.n_heads * D * 4;
        default: return 0;
    }
}

}  // namespace

extern "C" {

int vox_group_create(vox_engine * e, const vox_group_config * cfg, vox_group ** out) {
    VOX_REQUIRE(e && cfg && out, VOX_ATTN_INVALID_ARGUMENT, "vox_group_create: null argument");
    *out = nullptr;
    VOX_REQUIRE(cfg->n_streams > 0 && cfg->base_layers >= 0 && cfg->res_layers >= 0, VOX_ATTN_INVALID_ARGUMENT,
                "bad stream/layer counts");
    VOX_REQUIRE(cfg->head_dim == kHeadDim, VOX_ATTN_UNSUPPORTED, "head_dim %d not supported (64 only)", cfg->head_dim);
    VOX_REQUIRE(cfg->n_heads > 0 && cfg->n_kv_heads > 0 && cfg->n_heads % cfg->n_kv_heads == 0 &&
                    cfg->n_heads / cfg->n_kv_heads <= 8,
                VOX_ATTN_UNSUPPORTED, "head counts %d/%d not supported", cfg->n_heads, cfg->n_kv_heads);
    VOX_REQUIRE(cfg->cfm_steps >= 0 && cfg->cfm_steps <= 16, VOX_ATTN_UNSUPPORTED, "cfm_steps %d not supported (0..16)", cfg->cfm_steps);
    VOX_REQUIRE(cfg->cfm_zero_init_steps >= 0 && cfg->cfm_zero_init_steps <= cfg->cfm_steps, VOX_ATTN_INVALID_ARGUMENT,
                "cfm_zero_init_steps %d must lie in [0, cfm_steps]", cfg->cfm_zero_init_steps);
    VOX_REQUIRE(cfg->locdit_seq >= 1 && cfg->locdit_seq <= 16 && cfg->locdit_layers >= 0, VOX_ATTN_UNSUPPORTED, "LocDiT shape not supported");
    VOX_CUDA_TRY(cudaSetDevice(e->device));

    vox_group * g = new (std::nothrow) vox_group();
    VOX_REQUIRE(g != nullptr, VOX_ATTN_OUT_OF_MEMORY, "out of host memory");
    g->e = e;
    g->cfg = *cfg;
    g->kv_len_host.assign(cfg->n_streams, 0);
    int rc = VOX_ATTN_OK;
    const int layers[2] = {cfg->base_layers, cfg->res_layers};
    for (int s = 0; s < 2 && rc == VOX_ATTN_OK; ++s) {
        if (layers[s] == 0) continue;
        vox_kv_config kc = {layers[s], cfg->n_streams, cfg->n_kv_heads, cfg->head_dim, cfg->max_len, cfg->kv_type};
        rc = vox_kv_create(e, &kc, &g->cache[s]);
    }
    if (rc == VOX_ATTN_OK) {
        // the grid of a decode launch, and with it the workspace, only grows with the bound
        g->workspace_bytes = std::max<size_t>(256, vox_attn_decode_workspace_bytes(cfg->n_streams, cfg->n_heads, cfg->n_kv_heads, cfg->max_len));
        cudaError_t err = cudaMalloc(&g->workspace, g->workspace_bytes);
        if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void **>(&g->kv_len_dev), sizeof(int32_t) * cfg->n_streams);
        if (err == cudaSuccess) err = cudaMemset(g->kv_len_dev, 0, sizeof(int32_t) * cfg->n_streams);
        if (err != cudaSuccess) {
            cudaGetLastError();
            set_error("group allocation failed: %s", cudaGetErrorString(err));
            rc = VOX_ATTN_OUT_OF_MEMORY;
        }
    }
    if (rc != VOX_ATTN_OK) {
        vox_group_destroy(g);
        return rc;
    }
    *out = g;
    return VOX_ATTN_OK;
}

void vox_group_destroy(vox_group * g) {
    if (!g) return;
    cudaSetDevice(g->e->device);
    for (int s = 0; s < 2; ++s) vox_kv_destroy(g->cache[s]);
    if (g->workspace) cudaFree(g->workspace);
    if (g->kv_len_dev) cudaFree(g->kv_len_dev);
    if (g->rope_factors) cudaFree(g->rope_factors);
    if (g->rope_table) cudaFree(g->rope_table);
    if (g->proj_q) cudaFree(g->proj_q);
    if (g->proj_ws) cudaFree(g->proj_ws);
    if (g->dev_buf) cudaFree(g->dev_buf);
    if (g->st_compute) cudaStreamDestroy(g->st_compute);
    if (g->st_copy) cudaStreamDestroy(g->st_copy);
    if (g->st_back) cudaStreamDestroy(g->st_back);
    if (g->ev_lm_in) cudaEventDestroy(g->ev_lm_in);
    if (g->ev_lm_done) cudaEventDestroy(g->ev_lm_done);
    for (int i = 0; i < 16; ++i) {
        if (g->ev_dit_in[i]) cudaEventDestroy(g->ev_dit_in[i]);
        if (g->ev_dit_done[i]) cudaEventDestroy(g->ev_dit_done[i]);
    }
    delete g;
}

vox_kv_cache * vox_group_cache(vox_group * g, int stack) { return (g && stack >= 0 && stack < 2) ? g->cache[stack] : nullptr; }

int vox_group_set_kv_len(vox_group * g, const int32_t * kv_len) {
    VOX_REQUIRE(g && kv_len, VOX_ATTN_INVALID_ARGUMENT, "null argument");
    int bound = 0;
    for (int s = 0; s < g->cfg.n_streams; ++s) {
        VOX_REQUIRE(kv_len[s] >= 0 && kv_len[s] <= g->cfg.max_len, VOX_ATTN_INVALID_ARGUMENT,
                    "kv_len[%d] = %d exceeds the capacity %d", s, kv_len[s], g->cfg.max_len);
        bound = std::max(bound, kv_len[s]);
    }
    VOX_CUDA_TRY(cudaSetDevice(g->e->device));
    VOX_CUDA_TRY(cudaMemcpy(g->kv_len_dev, kv_len, sizeof(int32_t) * g->cfg.n_streams, cudaMemcpyHostToDevice));
    memcpy(g->kv_len_host.data(), kv_len, sizeof(int32_t) * g->cfg.n_streams);
    g->kv_bound = bound;
    return VOX_ATTN_OK;
}

int vox_group_get_kv_len(const vox_group * g, int32_t * kv_len) {
    VOX_REQUIRE(g && kv_len, VOX_ATTN_INVALID_ARGUMENT, "null argument");
    memcpy(kv_len, g->kv_len_host.data(), sizeof(int32_t) * g->cfg.n_streams);
    return VOX_ATTN_OK;
}

int vox_group_fill_synthetic(vox_group * g, uint64_t seed, void * stream) {
    VOX_REQUIRE(g != nullptr, VOX_ATTN_INVALID_ARGUMENT, "group is null");
    for (int s = 0; s < 2; ++s) {
        if (!g->cache[s]) continue;
        int rc = kv_fill_synthetic(g->cache[s], g->kv_len_dev, seed + 7919u * s, static_cast<cudaStream_t>(stream));
        if (rc != VOX_ATTN_OK) return rc;
    }
    return VOX_ATTN_OK;
}

int vox_group_set_bound(vox_group * g, int kv_bound) {
    VOX_REQUIRE(g != nullptr, VOX_ATTN_INVALID_ARGUMENT, "null group");
    VOX_REQUIRE(kv_bound == 0 || (kv_bound >= g->kv_bound && kv_bound <= g->cfg.max_len), VOX_ATTN_INVALID_ARGUMENT,
                "bound %d must lie between the longest stream (%d) and the capacity (%d), or be 0", kv_bound, g->kv_bound, g->cfg.max_len);
    g->grid_bound = kv_bound;
    return VOX_ATTN_OK;
}

int vox_group_advance(vox_group * g, int steps) {
    VOX_REQUIRE(g != nullptr && steps >= 0, VOX_ATTN_INVALID_ARGUMENT, "bad argument");
    const int limit = g->grid_bound > 0 ? g->grid_bound : g->cfg.max_len;
    VOX_REQUIRE(g->kv_bound + steps <= limit, VOX_ATTN_INVALID_ARGUMENT, "%d more rows would exceed %d", steps, limit);
    for (auto & x : g->kv_len_host) x += steps;
    g->kv_bound += steps;
    return VOX_ATTN_OK;
}

int vox_group_set_rope(vox_group * g, const vox_rope_config * cfg, const float * freq_factors_host) {
    VOX_REQUIRE(g != nullptr, VOX_ATTN_INVALID_ARGUMENT, "null group");
    if (cfg == nullptr) {  // back to "the caller rotates"
        g->rope_on = false;
        return VOX_ATTN_OK;
    }
    VOX_REQUIRE(cfg->freq_base > 0.0f, VOX_ATTN_INVALID_ARGUMENT, "freq_base must be positive");
    VOX_CUDA_TRY(cudaSetDevice(g->e->device));
    if (!g->rope_table) VOX_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&g->rope_table), sizeof(float) * 64 * g->cfg.n_streams));
    g->rope = *cfg;
    g->rope.freq_factors = nullptr;
    if (freq_factors_host != nullptr) {
        if (!g->rope_factors) VOX_CUDA_TRY(cudaMalloc(reinterpret_cast<void **>(&g->rope_factors), sizeof(float) * 32));
        VOX_CUDA_TRY(cudaMemcpy(g->rope_factors, freq_factors_host, sizeof(float) * 32, cudaMemcpyHostToDevice));
        g->rope.freq_factors = g->rope_factors;
    }
    g->rope_on = true;
    return VOX_ATTN_OK;
}

int vox_group_set_qkv_weights(vox_group * g, const void * w, int hidden, size_t nb_row, size_t nb_layer) {
    VOX_REQUIRE(g != nullptr, VOX_ATTN_INVALID_ARGUMENT, "null group");
    if (w == nullptr) {
        g->qkv_w = nullptr;
        return VOX_ATTN_OK;
    }
    const vox_group_config & c = g->cfg;
    VOX_REQUIRE(hidden > 0 && hidden % 64 == 0, VOX_ATTN_UNSUPPORTED, "hidden size %d is not a multiple of 64", hidden);
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(w) & 15) == 0 && nb_row % 16 == 0 && nb_row >= (size_t) hidden * 2 && nb_layer % 16 == 0,
                VOX_ATTN_INVALID_ARGUMENT, "weight rows must be 16-byte aligned and at least hidden halves apart");
    VOX_CUDA_TRY(cudaSetDevice(g->e->device));
    if (!g->proj_q) {
        const size_t rows = (size_t) c.n_streams * (c.n_heads + 2 * (size_t) c.n_kv_heads) * c.head_dim * sizeof(float);
        cudaError_t err = cudaMalloc(reinterpret_cast<void **>(&g->proj_q), rows);
        if (err != cudaSuccess) { cudaGetLastError(); set_error("projection rows allocation of %zu bytes failed", rows); return VOX_ATTN_OUT_OF_MEMORY; }
    }
    const size_t ws = vox_qkv_workspace_bytes(c.n_streams, hidden);
    if (ws > g->proj_ws_bytes) {
        if (g->proj_ws) cudaFree(g->proj_ws);
        g->proj_ws = nullptr; g->proj_ws_bytes = 0;
        cudaError_t err = cudaMalloc(&g->proj_ws, ws);
        if (err != cudaSuccess) { cudaGetLastError(); set_error("projection workspace allocation of %zu bytes failed", ws); return VOX_ATTN_OUT_OF_MEMORY; }
        g->proj_ws_bytes = ws;
    }
    g->qkv_w = static_cast<const uint8_t *>(w);
    g->qkv_hidden = hidden; g->qkv_nb_row = nb_row; g->qkv_nb_layer = nb_layer;
    return VOX_ATTN_OK;
}

size_t vox_group_step_bytes(const vox_group * g, int which) { return g ? step_bytes(g->cfg, which) : 0; }

int vox_group_step(vox_group * g, const vox_step_buffers * b, int advance, void * stream) {
    VOX_REQUIRE(g && b, VOX_ATTN_INVALID_ARGUMENT, "null argument");
    const vox_group_config & c = g->cfg;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t S = c.n_streams, D = c.head_dim;
    const float  scale = 1.0f / sqrtf((float) c.head_dim);  // src/minicpm.cpp:708-710
    // a null lm_q skips the LM stacks, a null dit_q skips the LocDiT patch (partial steps for profiling)
    const bool   project = b->lm_hidden != nullptr;  // the step starts from hidden states: projection + attention per layer
    if (project) {
        VOX_REQUIRE(g->qkv_w != nullptr, VOX_ATTN_INVALID_ARGUMENT, "lm_hidden needs vox_group_set_qkv_weights first");
        VOX_REQUIRE(!b->lm_q && !b->lm_k_new && !b->lm_v_new, VOX_ATTN_INVALID_ARGUMENT, "give lm_hidden or lm_q / lm_k_new / lm_v_new, not both");
        VOX_REQUIRE(advance, VOX_ATTN_INVALID_ARGUMENT, "a step from hidden states produces the new K/V rows: it advances");
    }
    const int    L = (b->lm_q || project) ? c.base_layers + c.res_layers : 0;
    VOX_REQUIRE(L > 0 || !advance, VOX_ATTN_INVALID_ARGUMENT, "advance needs the LM step buffers");
    if (L > 0) VOX_REQUIRE(b->lm_out && (!advance || project || (b->lm_k_new && b->lm_v_new)), VOX_ATTN_INVALID_ARGUMENT, "LM step buffers are null");
    if (advance) {
        VOX_REQUIRE(g->kv_bound + 1 <= c.max_len, VOX_ATTN_INVALID_ARGUMENT, "a stream would outgrow the cache capacity %d", c.max_len);
    }
    const int longest = g->kv_bound + (advance ? 1 : 0);
    VOX_REQUIRE(g->grid_bound == 0 || longest <= g->grid_bound, VOX_ATTN_INVALID_ARGUMENT,
                "a stream of %d rows exceeds the bound %d set with vox_group_set_bound", longest, g->grid_bound);
    const int bound = g->grid_bound > 0 ? g->grid_bound : longest;
    // A step that is being captured into a CUDA graph only records launches: the lengths on the device move when
    // the graph is replayed, and the host copy is moved by vox_group_advance after each replay.
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    VOX_CUDA_TRY(cudaStreamIsCapturing(st, &capture));
    const bool capturing = capture != cudaStreamCaptureStatusNone;
    if (advance) {  // the appended row becomes visible to this step's attention
        // a replayed step may run past the capacity before the host looks again: the length then stops one beyond it,
        // which the decode launch reports (it stores nothing for such a stream)
        launch_pdl(add_scalar_kernel, dim3((c.n_streams + 255) / 256), dim3(256), 0, st, g->kv_len_dev, c.n_streams, 1, c.max_len + 1);
        int rc = check_launch(g->e, "add_scalar_kernel");
        if (rc != VOX_ATTN_OK) return rc;
    }
    if (L > 0 && g->rope_on) {  // the angles of this step's positions (kv_len - 1), once for all layers
        int rc = vox_rope_table(g->e, &g->rope, g->kv_len_dev, -1, c.n_streams, g->rope_table, stream);
        if (rc != VOX_ATTN_OK) return rc;
    }
    for (int l = 0; l < L; ++l) {
        const int      stack = l < c.base_layers ? 0 : 1;
        const int      layer = stack == 0 ? l : l - c.base_layers;
        vox_kv_cache * kc    = g->cache[stack];
        vox_decode_args da = {};
        da.k_new = da.v_new = nullptr;
        da.new_nb_head = da.new_nb_stream = 0;
        // from the second layer on, the kernel before this one is the previous layer's decode: it wrote
        // neither the lengths nor this layer's rows (layer 0 follows the length update)
        da.flags = l > 0 ? VOX_DECODE_CACHE_STABLE : 0u;
        da.rope_table = g->rope_on ? g->rope_table : nullptr;
        da.stream_order = nullptr;  // every CTA of a decode launch streams an equal share of the rows whatever the order
        if (advance && !project) {  // the token's K/V rows are stored by the decode launch itself (position kv_len-1)
            da.k_new = b->lm_k_new + (size_t) l * S * c.n_kv_heads * D;
            da.v_new = b->lm_v_new + (size_t) l * S * c.n_kv_heads * D;
            da.new_nb_head = D * 4; da.new_nb_stream = (size_t) c.n_kv_heads * D * 4;
        }
        da.cache = kc; da.layer = layer; da.n_streams = c.n_streams; da.n_heads = c.n_heads;
        da.kv_len = g->kv_len_dev; da.kv_bound = bound;
        if (project) {
            // this layer's Q and new K/V rows from the hidden states: one projection launch for all streams (rotated when
            // the group applies the rotary embedding); the decode launch then stores the rows and attends
            vox_qkv_args qa;
            memset(&qa, 0, sizeof(qa));
            qa.n_streams = c.n_streams; qa.hidden = g->qkv_hidden; qa.n_heads = c.n_heads; qa.n_kv_heads = c.n_kv_heads; qa.head_dim = c.head_dim;
            qa.x = b->lm_hidden + (size_t) l * S * g->qkv_hidden; qa.x_nb_stream = (size_t) g->qkv_hidden * 4;
            qa.w_qkv = g->qkv_w + (size_t) l * g->qkv_nb_layer; qa.w_nb_row = g->qkv_nb_row; qa.w_type = VOX_TYPE_F16;
            qa.rope_table = g->rope_on ? g->rope_table : nullptr;
            qa.q = g->proj_q;
            qa.k_new = g->proj_q + S * c.n_heads * D;
            qa.v_new = qa.k_new + S * c.n_kv_heads * D;
            int rc = vox_qkv_project(g->e, &qa, g->proj_ws, g->proj_ws_bytes, stream);
            if (rc != VOX_ATTN_OK) return rc;
            da.k_new = qa.k_new; da.v_new = qa.v_new;
            da.new_nb_head = D * 4; da.new_nb_stream = (size_t) c.n_kv_heads * D * 4;
            da.rope_table = nullptr;  // applied by the projection
        }
        da.q = project ? g->proj_q : b->lm_q + (size_t) l * S * c.n_heads * D;
        da.q_nb_head = D * 4; da.q_nb_stream = (size_t) c.n_heads * D * 4;
        da.dst = b->lm_out + (size_t) l * S * c.n_heads * D;
        da.scale = scale;
        int rc = vox_attn_decode(g->e, &da, g->workspace, g->workspace_bytes, stream);
        if (rc != VOX_ATTN_OK) return rc;
    }
    if (advance && !capturing) {
        for (auto & x : g->kv_len_host) x += 1;
        g->kv_bound += 1;
    }
    if (c.cfm_steps > 0 && c.locdit_layers > 0 && b->dit_q) {
        VOX_REQUIRE(b->dit_k && b->dit_v && b->dit_out, VOX_ATTN_INVALID_ARGUMENT, "LocDiT step buffers are null");
        const size_t q_step  = S * c.locdit_layers * 2 * c.locdit_seq * c.n_heads * D;
        const size_t kv_step = S * c.locdit_layers * 2 * c.locdit_seq * c.n_kv_heads * D;
        // the first cfm_zero_init_steps timesteps evaluate no network (UnifiedCFM::solve_euler with cfg-zero-star,
        // src/unified_cfm.cpp:107-116: dphi_dt = 0 there), so they issue nothing and leave their slice of dit_out alone
        for (int t = c.cfm_zero_init_steps; t < c.cfm_steps; ++t) {
            vox_locdit_args la;
            la.n_streams = c.n_streams; la.n_layers = c.locdit_layers; la.n_heads = c.n_heads; la.n_kv_heads = c.n_kv_heads;
            la.seq = c.locdit_seq; la.head_dim = c.head_dim;
            la.q = b->dit_q + t * q_step; la.k = b->dit_k + t * kv_step; la.v = b->dit_v + t * kv_step;
            la.dst = b->dit_out + t * q_step; la.scale = scale;
            int rc = vox_attn_locdit_step(g->e, &la, stream);
            if (rc != VOX_ATTN_OK) return rc;
        }
    }
    return VOX_ATTN_OK;
}

// Host-buffer form: inputs cross PCIe on one copy stream while the compute stream works on what has
// already landed (LM inputs first, then one CFM timestep at a time); outputs return on a second copy
// stream as each part finishes, so both directions of the link are busy at once.
int vox_group_step_host(vox_group * g, const vox_step_buffers * h, int advance) {
    VOX_REQUIRE(g && h, VOX_ATTN_INVALID_ARGUMENT, "null argument");
    const vox_group_config & c = g->cfg;
    VOX_CUDA_TRY(cudaSetDevice(g->e->device));
    const size_t S = c.n_streams, D = c.head_dim, L = lm_layers(c);
    const size_t lm_q_b = L * S * c.n_heads * D * 4, lm_kv_b = L * S * c.n_kv_heads * D * 4;
    const size_t dq_step = S * c.locdit_layers * 2 * c.locdit_seq * c.n_heads * D * 4;
    const size_t dkv_step = S * c.locdit_layers * 2 * c.locdit_seq * c.n_kv_heads * D * 4;
    const size_t T = c.cfm_steps;
    if (!g->dev_buf) {
        const size_t sizes[8] = {lm_q_b, lm_kv_b, lm_kv_b, lm_q_b, dq_step * T, dkv_step * T, dkv_step * T, dq_step * T};
        size_t off = 0;
        for (int i = 0; i < 8; ++i) { g->dev_off[i] = off; off += (sizes[i] + 255) & ~(size_t) 255; }
        cudaError_t err = cudaMalloc(reinterpret_cast<void **>(&g->dev_buf), std::max<size_t>(off, 256));
        if (err != cudaSuccess) { cudaGetLastError(); set_error("step staging allocation of %zu bytes failed", off); return VOX_ATTN_OUT_OF_MEMORY; }
        VOX_CUDA_TRY(cudaStreamCreateWithFlags(&g->st_compute, cudaStreamNonBlocking));
        VOX_CUDA_TRY(cudaStreamCreateWithFlags(&g->st_copy, cudaStreamNonBlocking));
        VOX_CUDA_TRY(cudaStreamCreateWithFlags(&g->st_back, cudaStreamNonBlocking));
        VOX_CUDA_TRY(cudaEventCreateWithFlags(&g->ev_lm_in, cudaEventDisableTiming));
        VOX_CUDA_TRY(cudaEventCreateWithFlags(&g->ev_lm_done, cudaEventDisableTiming));
        for (int i = 0; i < 16; ++i) {
            VOX_CUDA_TRY(cudaEventCreateWithFlags(&g->ev_dit_in[i], cudaEventDisableTiming));
            VOX_CUDA_TRY(cudaEventCreateWithFlags(&g->ev_dit_done[i], cudaEventDisableTiming));
        }
    }
    uint8_t * d = g->dev_buf;
    vox_step_buffers dev = {};
    dev.lm_q = (const float *) (d + g->dev_off[0]); dev.lm_k_new = (const float *) (d + g->dev_off[1]);
    dev.lm_v_new = (const float *) (d + g->dev_off[2]); dev.lm_out = (float *) (d + g->dev_off[3]);
    dev.dit_q = (const float *) (d + g->dev_off[4]); dev.dit_k = (const float *) (d + g->dev_off[5]);
    dev.dit_v = (const float *) (d + g->dev_off[6]); dev.dit_out = (float *) (d + g->dev_off[7]);

    // inputs: LM first, then each CFM timestep
    if (L > 0) {
        VOX_CUDA_TRY(cudaMemcpyAsync((void *) dev.lm_q, h->lm_q, lm_q_b, cudaMemcpyHostToDevice, g->st_copy));
        if (advance) {
            VOX_CUDA_TRY(cudaMemcpyAsync((void *) dev.lm_k_new, h->lm_k_new, lm_kv_b, cudaMemcpyHostToDevice, g->st_copy));
            VOX_CUDA_TRY(cudaMemcpyAsync((void *) dev.lm_v_new, h->lm_v_new, lm_kv_b, cudaMemcpyHostToDevice, g->st_copy));
        }
    }
    VOX_CUDA_TRY(cudaEventRecord(g->ev_lm_in, g->st_copy));
    const size_t T0 = c.cfm_zero_init_steps;  // timesteps that evaluate no network move no data either
    for (size_t t = T0; t < T; ++t) {
        VOX_CUDA_TRY(cudaMemcpyAsync((uint8_t *) dev.dit_q + t * dq_step, (const uint8_t *) h->dit_q + t * dq_step, dq_step, cudaMemcpyHostToDevice, g->st_copy));
        VOX_CUDA_TRY(cudaMemcpyAsync((uint8_t *) dev.dit_k + t * dkv_step, (const uint8_t *) h->dit_k + t * dkv_step, dkv_step, cudaMemcpyHostToDevice, g->st_copy));
        VOX_CUDA_TRY(cudaMemcpyAsync((uint8_t *) dev.dit_v + t * dkv_step, (const uint8_t *) h->dit_v + t * dkv_step, dkv_step, cudaMemcpyHostToDevice, g->st_copy));
        VOX_CUDA_TRY(cudaEventRecord(g->ev_dit_in[t], g->st_copy));
    }
    // compute: LM layers once their inputs are in, then each timestep as it lands
    vox_group_config lm_only = c; lm_only.cfm_steps = 0;
    vox_group_config saved = g->cfg;
    VOX_CUDA_TRY(cudaStreamWaitEvent(g->st_compute, g->ev_lm_in, 0));
    g->cfg = lm_only;
    int rc = vox_group_step(g, &dev, advance, g->st_compute);
    g->cfg = saved;
    if (rc != VOX_ATTN_OK) return rc;
    VOX_CUDA_TRY(cudaEventRecord(g->ev_lm_done, g->st_compute));
    const float scale = 1.0f / sqrtf((float) c.head_dim);
    for (size_t t = T0; t < T && c.locdit_layers > 0; ++t) {
        VOX_CUDA_TRY(cudaStreamWaitEvent(g->st_compute, g->ev_dit_in[t], 0));
        vox_locdit_args la;
        la.n_streams = c.n_streams; la.n_layers = c.locdit_layers; la.n_heads = c.n_heads; la.n_kv_heads = c.n_kv_heads;
        la.seq = c.locdit_seq; la.head_dim = c.head_dim; la.scale = scale;
        la.q = (const float *) ((const uint8_t *) dev.dit_q + t * dq_step);
        la.k = (const float *) ((const uint8_t *) dev.dit_k + t * dkv_step);
        la.v = (const float *) ((const uint8_t *) dev.dit_v + t * dkv_step);
        la.dst = (float *) ((uint8_t *) dev.dit_out + t * dq_step);
        rc = vox_attn_locdit_step(g->e, &la, g->st_compute);
        if (rc != VOX_ATTN_OK) return rc;
        VOX_CUDA_TRY(cudaEventRecord(g->ev_dit_done[t], g->st_compute));
    }
    // outputs go back on a stream of their own: PCIe is full duplex, so they overlap the inputs still arriving
    if (L > 0) {
        VOX_CUDA_TRY(cudaStreamWaitEvent(g->st_back, g->ev_lm_done, 0));
        VOX_CUDA_TRY(cudaMemcpyAsync(h->lm_out, dev.lm_out, lm_q_b, cudaMemcpyDeviceToHost, g->st_back));
    }
    for (size_t t = T0; t < T && c.locdit_layers > 0; ++t) {
        VOX_CUDA_TRY(cudaStreamWaitEvent(g->st_back, g->ev_dit_done[t], 0));
        VOX_CUDA_TRY(cudaMemcpyAsync((uint8_t *) h->dit_out + t * dq_step, (const uint8_t *) dev.dit_out + t * dq_step, dq_step, cudaMemcpyDeviceToHost, g->st_back));
    }
    VOX_CUDA_TRY(cudaStreamSynchronize(g->st_back));
    return vox_engine_sync_status(g->e, g->st_compute);
}

int vox_partition_streams(const int32_t * kv_len, int n_streams, int n_gpus, int32_t * owner) {
    VOX_REQUIRE(kv_len && owner && n_streams >= 0 && n_gpus > 0, VOX_ATTN_INVALID_ARGUMENT, "bad partition arguments");
    std::vector<int> order(n_streams);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return kv_len[a] > kv_len[b]; });
    std::vector<long long> load(n_gpus, 0);
    std::vector<int>       count(n_gpus, 0);
    for (int s : order) {
        int best = 0;
        for (int gidx = 1; gidx < n_gpus; ++gidx)
            if (load[gidx] < load[best] || (load[gidx] == load[best] && count[gidx] < count[best])) best = gidx;
        owner[s] = best;
        load[best] += std::max(kv_len[s], 0);
        count[best] += 1;
    }
    return VOX_ATTN_OK;
}

}  // extern "C"
