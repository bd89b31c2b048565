// KV cache: storage, in-place append (f32 -> f16 / q8_0), host import/export.
//
// Replaces MiniCPMKVCache (src/minicpm.cpp:144-271) and the cpy + concat pair that
// MiniCPMModel::attention_forward emits around every attention call
// (src/minicpm.cpp:684-701).  Rows are stored once, already in the type the decode kernel
// streams, so nothing is re-copied or re-converted per step.
#include "kv_cache.cuh"

#include <cstring>
#include <new>
#include <vector>

using namespace vox;

namespace {

// One warp per cache row (64 values): lane l holds elements 2l, 2l+1.
// f16: GGML_FP32_TO_FP16 rounding (round-to-nearest-even) == __float2half_rn.
// q8_0: the arithmetic of quantize_row_q8_0_ref (ggml-quants.c:199-222), one 32-value block
// per half-warp: d = amax/127, id = d ? 1/d : 0, q = roundf(x*id), scale stored as f16(d).
struct CacheView {
    uint8_t * k_data; uint8_t * v_data; uint8_t * k_scale; uint8_t * v_scale;
    size_t nb_pos, nb_head, nb_stream, nb_layer;
    size_t sb_pos, sb_head, sb_stream, sb_layer;
    int    n_kv_heads, max_len, type;
};

__device__ __forceinline__ void write_row(const CacheView & c, uint8_t * data, uint8_t * scale, int layer, int stream,
                                          int head, int pos, float x0, float x1, int lane) {
    const size_t pair = (size_t) layer * c.nb_layer + (size_t) stream * c.nb_stream + (size_t) head * c.nb_head;
    if (c.type == VOX_TYPE_F16) {
        *reinterpret_cast<__half2 *>(data + pair + (size_t) pos * c.nb_pos + lane * 4) = __floats2half2_rn(x0, x1);
    } else {
        char2 q;
        float d;
        q8_0_quantize_pair(x0, x1, q, d);
        const size_t tile = pair + q8_tile_off(pos);
        *reinterpret_cast<uchar2 *>(data + tile + q8_byte_off(pos, 2 * lane)) = q8_0_biased(q);
        if ((lane & 15) == 0) *reinterpret_cast<__half *>(scale + tile + q8_scale_off(pos, lane >> 4)) = __float2half_rn(d);
    }
}

__global__ void kv_append_kernel(CacheView c, int layer, int n_streams, int n_tok, const int32_t * positions, int pos0,
                                 const float * k, const float * v, size_t nb_head, size_t nb_tok, size_t nb_stream,
                                 int * status) {
    const int warps_per_block = blockDim.x >> 5;
    const int lane            = threadIdx.x & 31;
    pdl_wait();  // positions come from the kernel before; earlier readers of these cache rows are done
    pdl_launch_dependents();
    const long long n_rows    = (long long) n_streams * n_tok * c.n_kv_heads;
    for (long long row = (long long) blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < n_rows;
         row += (long long) gridDim.x * warps_per_block) {
        const int head   = (int) (row % c.n_kv_heads);
        const int tok    = (int) ((row / c.n_kv_heads) % n_tok);
        const int stream = (int) (row / ((long long) c.n_kv_heads * n_tok));
        const int pos    = (positions ? positions[stream] : pos0) + tok;
        if (pos < 0 || pos >= c.max_len) {  // never write outside the stream's rows
            if (lane == 0) atomicOr(status, kStatusBadState);
            continue;
        }
        const size_t src = (size_t) head * nb_head + (size_t) tok * nb_tok + (size_t) stream * nb_stream;
        const float2 kk  = *reinterpret_cast<const float2 *>(reinterpret_cast<const uint8_t *>(k) + src + lane * 8);
        const float2 vv  = *reinterpret_cast<const float2 *>(reinterpret_cast<const uint8_t *>(v) + src + lane * 8);
        write_row(c, c.k_data, c.k_scale, layer, stream, head, pos, kk.x, kk.y, lane);
        write_row(c, c.v_data, c.v_scale, layer, stream, head, pos, vv.x, vv.y, lane);
    }
}

// Synthetic state: rows [0, kv_len[s]) of every layer/head filled from the counter-based generator.
__global__ void kv_fill_kernel(CacheView c, int n_layers, int n_streams, const int32_t * kv_len, uint64_t seed) {
    const int warps_per_block = blockDim.x >> 5;
    const int lane            = threadIdx.x & 31;
    const long long rows_per_stream = (long long) c.max_len * c.n_kv_heads * n_layers;
    const long long n_rows          = rows_per_stream * n_streams;
    for (long long row = (long long) blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < n_rows;
         row += (long long) gridDim.x * warps_per_block) {
        const int pos    = (int) (row % c.max_len);
        const int head   = (int) ((row / c.max_len) % c.n_kv_heads);
        const int layer  = (int) ((row / ((long long) c.max_len * c.n_kv_heads)) % n_layers);
        const int stream = (int) (row / rows_per_stream);
        if (pos >= kv_len[stream]) continue;
        const uint64_t idx = ((uint64_t) row * 2) * 64 + lane * 2;
        write_row(c, c.k_data, c.k_scale, layer, stream, head, pos, synth_normal(seed, idx), synth_normal(seed, idx + 1),
                  lane);
        write_row(c, c.v_data, c.v_scale, layer, stream, head, pos, synth_normal(seed, idx + 64),
                  synth_normal(seed, idx + 65), lane);
    }
}

CacheView view_of(const vox_kv_cache * c) {
    CacheView v;
    v.k_data = c->k_data; v.v_data = c->v_data; v.k_scale = c->k_scale; v.v_scale = c->v_scale;
    v.nb_pos = c->nb_pos; v.nb_head = c->nb_head; v.nb_stream = c->nb_stream; v.nb_layer = c->nb_layer;
    v.sb_pos = c->sb_pos; v.sb_head = c->sb_head; v.sb_stream = c->sb_stream; v.sb_layer = c->sb_layer;
    v.n_kv_heads = c->cfg.n_kv_heads; v.max_len = c->cfg.max_len; v.type = c->cfg.type;
    return v;
}

}  // namespace

namespace vox {
// after a kernel gave up (status word raised) some of a pair's CTAs may have taken tickets that nobody reset
void reset_ticket_counters(vox_engine * e, cudaStream_t stream) {
    cudaMemsetAsync(e->counters_dev, 0, sizeof(int) * kCounterSlots, stream);
    for (vox_kv_cache * c : e->caches)
        cudaMemsetAsync(c->counters, 0, sizeof(int) * (size_t) c->cfg.n_layers * c->cfg.n_streams * c->cfg.n_kv_heads, stream);
    cudaStreamSynchronize(stream);
}

int kv_fill_synthetic(vox_kv_cache * c, const int32_t * kv_len_dev, uint64_t seed, cudaStream_t stream) {
    const long long rows = (long long) c->cfg.max_len * c->cfg.n_kv_heads * c->cfg.n_layers * c->cfg.n_streams;
    const int blocks     = (int) std::min<long long>((rows + 7) / 8, (long long) c->e->sm_count * 16);
    kv_fill_kernel<<<blocks, 256, 0, stream>>>(view_of(c), c->cfg.n_layers, c->cfg.n_streams, kv_len_dev, seed);
    return check_launch(c->e, "kv_fill_kernel");
}
}  // namespace vox

extern "C" {

int vox_kv_create(vox_engine * e, const vox_kv_config * cfg, vox_kv_cache ** out) {
    VOX_REQUIRE(e && cfg && out, VOX_ATTN_INVALID_ARGUMENT, "vox_kv_create: null argument");
    *out = nullptr;
    VOX_REQUIRE(cfg->head_dim == kHeadDim, VOX_ATTN_UNSUPPORTED, "head_dim %d not supported (64 only)", cfg->head_dim);
    VOX_REQUIRE(cfg->type == VOX_TYPE_F16 || cfg->type == VOX_TYPE_Q8_0, VOX_ATTN_UNSUPPORTED,
                "cache type %d not supported (f16 or q8_0)", cfg->type);
    VOX_REQUIRE(cfg->n_layers > 0 && cfg->n_streams > 0 && cfg->n_kv_heads > 0 && cfg->max_len > 0,
                VOX_ATTN_INVALID_ARGUMENT, "cache extents must be positive");
    VOX_REQUIRE(cfg->max_len % 8 == 0, VOX_ATTN_INVALID_ARGUMENT, "max_len must be a multiple of 8 (16-byte scale rows)");
    VOX_CUDA_TRY(cudaSetDevice(e->device));

    vox_kv_cache * c = new (std::nothrow) vox_kv_cache();
    VOX_REQUIRE(c != nullptr, VOX_ATTN_OUT_OF_MEMORY, "out of host memory");
    c->e   = e;
    c->cfg = *cfg;
    const bool q8 = cfg->type == VOX_TYPE_Q8_0;
    if (!q8) {
        c->nb_pos    = 128;
        c->nb_head   = c->nb_pos * cfg->max_len;
        c->nb_stream = c->nb_head * cfg->n_kv_heads;
        c->nb_layer  = c->nb_stream * cfg->n_streams;
        c->bytes     = 2 * c->nb_layer * cfg->n_layers;
    } else {
        const size_t tiles = ((size_t) cfg->max_len + kKvTile - 1) / kKvTile;
        c->nb_pos    = 0;
        c->nb_head   = tiles * kQ8TileBytes;
        c->nb_stream = c->nb_head * cfg->n_kv_heads;
        c->nb_layer  = c->nb_stream * cfg->n_streams;
        c->sb_pos = 0; c->sb_head = c->nb_head; c->sb_stream = c->nb_stream; c->sb_layer = c->nb_layer;
        c->bytes     = c->nb_layer * cfg->n_layers;
    }
    uint8_t * base = nullptr;
    cudaError_t err = cudaMalloc(reinterpret_cast<void **>(&base), c->bytes);
    if (err != cudaSuccess) {
        set_error("KV cache allocation of %zu bytes failed: %s", c->bytes, cudaGetErrorString(err));
        cudaGetLastError();
        delete c;
        return VOX_ATTN_OUT_OF_MEMORY;
    }
    c->k_data = base;
    if (!q8) {
        c->v_data = base + c->bytes / 2;
    } else {
        c->v_data  = base + kQ8VBytesOff;
        c->k_scale = base + kQ8KScaleOff;
        c->v_scale = base + kQ8VScaleOff;
    }
    // MiniCPMKVCache::init ends with clear(): every stored value is zero (a q8_0 byte holds q + 128)
    err = cudaMemset(base, 0, c->bytes);
    if (err == cudaSuccess && q8)  // the byte blocks of every tile
        err = cudaMemset2D(base, kQ8TileBytes, 0x80, kQ8KScaleOff, c->bytes / kQ8TileBytes);
    if (err == cudaSuccess) {
        const size_t n_ctr = (size_t) cfg->n_layers * cfg->n_streams * cfg->n_kv_heads;
        err = cudaMalloc(reinterpret_cast<void **>(&c->counters), sizeof(int) * n_ctr);
        if (err == cudaSuccess) err = cudaMemset(c->counters, 0, sizeof(int) * n_ctr);
    }
    int rc = err == cudaSuccess ? VOX_ATTN_OK : VOX_ATTN_CUDA_ERROR;
    if (rc == VOX_ATTN_OK && !q8) {
        const uint64_t dims[5]    = {64, (uint64_t) cfg->max_len, (uint64_t) cfg->n_kv_heads, (uint64_t) cfg->n_streams,
                                     (uint64_t) cfg->n_layers};
        const uint64_t strides[4] = {c->nb_pos, c->nb_head, c->nb_stream, c->nb_layer};
        const uint32_t box[5]     = {64, kKvTile, 1, 1, 1};
        rc = make_tensor_map(e, &c->map_k, c->k_data, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc == VOX_ATTN_OK)
            rc = make_tensor_map(e, &c->map_v, c->v_data, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    } else if (rc == VOX_ATTN_OK) {
        memset(&c->map_k, 0, sizeof(c->map_k));
        memset(&c->map_v, 0, sizeof(c->map_v));
    } else {
        set_error("clearing the KV cache or allocating its ticket counters failed: %s", cudaGetErrorString(err));
    }
    if (rc != VOX_ATTN_OK) {
        cudaFree(base);
        if (c->counters) cudaFree(c->counters);
        delete c;
        return rc;
    }
    e->caches.push_back(c);
    *out = c;
    return VOX_ATTN_OK;
}

void vox_kv_destroy(vox_kv_cache * c) {
    if (!c) return;
    cudaSetDevice(c->e->device);
    auto & list = c->e->caches;
    for (size_t i = 0; i < list.size(); ++i)
        if (list[i] == c) { list.erase(list.begin() + i); break; }
    if (c->k_data) cudaFree(c->k_data);
    if (c->counters) cudaFree(c->counters);
    delete c;
}

size_t vox_kv_bytes(const vox_kv_cache * c) { return c ? c->bytes : 0; }

int vox_kv_clear(vox_kv_cache * c, int stream_id, void * stream) {
    VOX_REQUIRE(c != nullptr, VOX_ATTN_INVALID_ARGUMENT, "cache is null");
    VOX_REQUIRE(stream_id >= -1 && stream_id < c->cfg.n_streams, VOX_ATTN_INVALID_ARGUMENT, "stream_id %d out of range",
                stream_id);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool q8 = c->cfg.type == VOX_TYPE_Q8_0;  // a q8_0 byte holds q + 128: zero is 0x80 there, and 0 in the scales
    if (stream_id < 0) {
        VOX_CUDA_TRY(cudaMemsetAsync(c->k_data, 0, c->bytes, st));
        if (q8) VOX_CUDA_TRY(cudaMemset2DAsync(c->k_data, kQ8TileBytes, 0x80, kQ8KScaleOff, c->bytes / kQ8TileBytes, st));
        return VOX_ATTN_OK;
    }
    for (int l = 0; l < c->cfg.n_layers; ++l) {
        const size_t off = (size_t) l * c->nb_layer + (size_t) stream_id * c->nb_stream;
        VOX_CUDA_TRY(cudaMemsetAsync(c->k_data + off, 0, c->nb_stream, st));
        if (q8) VOX_CUDA_TRY(cudaMemset2DAsync(c->k_data + off, kQ8TileBytes, 0x80, kQ8KScaleOff, c->nb_stream / kQ8TileBytes, st));
        else    VOX_CUDA_TRY(cudaMemsetAsync(c->v_data + off, 0, c->nb_stream, st));
    }
    return VOX_ATTN_OK;
}

int vox_kv_append(vox_kv_cache * c, int layer, int n_streams, int n_tok, const int32_t * positions, int pos0,
                  const float * k, const float * v, size_t nb_head, size_t nb_tok, size_t nb_stream, void * stream) {
    VOX_REQUIRE(c && k && v, VOX_ATTN_INVALID_ARGUMENT, "vox_kv_append: null argument");
    VOX_REQUIRE(layer >= 0 && layer < c->cfg.n_layers, VOX_ATTN_INVALID_ARGUMENT, "layer %d out of range", layer);
    VOX_REQUIRE(n_streams > 0 && n_streams <= c->cfg.n_streams, VOX_ATTN_INVALID_ARGUMENT, "n_streams %d out of range",
                n_streams);
    VOX_REQUIRE(n_tok > 0 && n_tok <= c->cfg.max_len, VOX_ATTN_INVALID_ARGUMENT, "n_tok %d out of range", n_tok);
    VOX_REQUIRE(positions != nullptr || (pos0 >= 0 && pos0 + n_tok <= c->cfg.max_len), VOX_ATTN_INVALID_ARGUMENT,
                "rows %d..%d exceed the cache capacity %d", pos0, pos0 + n_tok, c->cfg.max_len);
    VOX_REQUIRE(nb_head % 8 == 0 && nb_tok % 8 == 0 && nb_stream % 8 == 0 &&
                    (reinterpret_cast<uintptr_t>(k) & 7) == 0 && (reinterpret_cast<uintptr_t>(v) & 7) == 0,
                VOX_ATTN_INVALID_ARGUMENT, "new K/V rows must be 8-byte aligned");
    const long long rows = (long long) n_streams * n_tok * c->cfg.n_kv_heads;
    const int blocks     = (int) std::min<long long>((rows + 7) / 8, (long long) c->e->sm_count * 8);
    launch_pdl(kv_append_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), view_of(c), layer, n_streams, n_tok,
               positions, pos0, k, v, nb_head, nb_tok, nb_stream, c->e->status_dev);
    return check_launch(c->e, "kv_append_kernel");
}

int vox_kv_view(const vox_kv_cache * c, int layer, int stream_id, int seq_len, vox_tensor * k, vox_tensor * v) {
    VOX_REQUIRE(c && k && v, VOX_ATTN_INVALID_ARGUMENT, "vox_kv_view: null argument");
    VOX_REQUIRE(layer >= 0 && layer < c->cfg.n_layers && stream_id >= 0 && stream_id < c->cfg.n_streams,
                VOX_ATTN_INVALID_ARGUMENT, "layer/stream out of range");
    VOX_REQUIRE(seq_len >= 0 && seq_len <= c->cfg.max_len, VOX_ATTN_INVALID_ARGUMENT, "seq_len %d out of range", seq_len);
    VOX_REQUIRE(c->cfg.type == VOX_TYPE_F16, VOX_ATTN_UNSUPPORTED,
                "a q8_0 cache is stored as tiles of bytes and scales and has no ggml tensor view");
    const size_t off = (size_t) layer * c->nb_layer + (size_t) stream_id * c->nb_stream;
    vox_tensor * ts[2]   = {k, v};
    uint8_t *    base[2] = {c->k_data, c->v_data};
    for (int i = 0; i < 2; ++i) {
        ts[i]->type  = VOX_TYPE_F16;
        ts[i]->ne[0] = 64; ts[i]->ne[1] = seq_len; ts[i]->ne[2] = c->cfg.n_kv_heads; ts[i]->ne[3] = 1;
        ts[i]->nb[0] = 2; ts[i]->nb[1] = c->nb_pos; ts[i]->nb[2] = c->nb_head; ts[i]->nb[3] = c->nb_stream;
        ts[i]->data  = base[i] + off;
    }
    return VOX_ATTN_OK;
}

static int kv_transfer(const vox_kv_cache * c, int layer, int stream_id, int n_pos, void * k_host, void * v_host,
                       bool to_host) {
    VOX_REQUIRE(c && k_host && v_host, VOX_ATTN_INVALID_ARGUMENT, "null argument");
    VOX_REQUIRE(layer >= 0 && layer < c->cfg.n_layers && stream_id >= 0 && stream_id < c->cfg.n_streams,
                VOX_ATTN_INVALID_ARGUMENT, "layer/stream out of range");
    VOX_REQUIRE(n_pos >= 0 && n_pos <= c->cfg.max_len, VOX_ATTN_INVALID_ARGUMENT, "n_pos %d out of range", n_pos);
    VOX_CUDA_TRY(cudaSetDevice(c->e->device));
    const int  HK = c->cfg.n_kv_heads;
    const bool q8 = c->cfg.type == VOX_TYPE_Q8_0;
    uint8_t *  hosts[2]  = {static_cast<uint8_t *>(k_host), static_cast<uint8_t *>(v_host)};
    if (!q8) {
        uint8_t * datas[2] = {c->k_data, c->v_data};
        for (int t = 0; t < 2; ++t)
            for (int h = 0; h < HK; ++h) {
                uint8_t * dev = datas[t] + (size_t) layer * c->nb_layer + (size_t) stream_id * c->nb_stream + (size_t) h * c->nb_head;
                uint8_t * hp  = hosts[t] + (size_t) h * n_pos * 128;
                if (to_host) VOX_CUDA_TRY(cudaMemcpy(hp, dev, (size_t) n_pos * 128, cudaMemcpyDeviceToHost));
                else         VOX_CUDA_TRY(cudaMemcpy(dev, hp, (size_t) n_pos * 128, cudaMemcpyHostToDevice));
            }
        return VOX_ATTN_OK;
    }
    // q8_0: the tiles that hold rows [0, n_pos) of a pair come to the host as they are; rows are taken out of them, or
    // put into them and the tiles sent back (rows past n_pos in the last tile keep what they held).  Host side: two
    // block_q8_0 per row (34 bytes each: f16 scale, 32 signed bytes).
    const size_t         span = (size_t) ((n_pos + kKvTile - 1) / kKvTile) * kQ8TileBytes;
    std::vector<uint8_t> tiles(span);
    const uint32_t       byte_block[2] = {0, (uint32_t) kQ8VBytesOff}, scale_block[2] = {(uint32_t) kQ8KScaleOff, (uint32_t) kQ8VScaleOff};
    for (int h = 0; h < HK && span > 0; ++h) {
        uint8_t * dev = c->k_data + (size_t) layer * c->nb_layer + (size_t) stream_id * c->nb_stream + (size_t) h * c->nb_head;
        VOX_CUDA_TRY(cudaMemcpy(tiles.data(), dev, span, cudaMemcpyDeviceToHost));
        for (int t = 0; t < 2; ++t) {
            uint8_t * hp = hosts[t] + (size_t) h * n_pos * 68;
            for (int p = 0; p < n_pos; ++p) {
                uint8_t * tile = tiles.data() + q8_tile_off(p);
                for (int b = 0; b < 2; ++b) {
                    uint8_t * blk = hp + (size_t) p * 68 + b * 34;
                    uint8_t * sc  = tile + scale_block[t] + q8_scale_off(p, b);
                    if (to_host) memcpy(blk, sc, 2);
                    else         memcpy(sc, blk, 2);
                    for (int i = 0; i < 32; ++i) {
                        uint8_t * q = tile + byte_block[t] + q8_byte_off(p, 32 * b + i);
                        if (to_host) blk[2 + i] = (uint8_t) (*q ^ 0x80);  // the cache holds q + 128
                        else         *q = (uint8_t) (blk[2 + i] ^ 0x80);
                    }
                }
            }
        }
        if (!to_host) VOX_CUDA_TRY(cudaMemcpy(dev, tiles.data(), span, cudaMemcpyHostToDevice));
    }
    return VOX_ATTN_OK;
}

int vox_kv_export(const vox_kv_cache * c, int layer, int stream_id, int n_pos, void * k_host, void * v_host) {
    return kv_transfer(c, layer, stream_id, n_pos, k_host, v_host, true);
}

int vox_kv_import(vox_kv_cache * c, int layer, int stream_id, int n_pos, const void * k_host, const void * v_host) {
    return kv_transfer(c, layer, stream_id, n_pos, const_cast<void *>(k_host), const_cast<void *>(v_host), false);
}

int vox_kv_copy_from(vox_kv_cache * dst, const vox_kv_cache * src, void * stream) {
    VOX_REQUIRE(dst && src, VOX_ATTN_INVALID_ARGUMENT, "null cache");
    VOX_REQUIRE(memcmp(&dst->cfg, &src->cfg, sizeof(vox_kv_config)) == 0, VOX_ATTN_INVALID_ARGUMENT,
                "caches differ in shape or type");
    VOX_CUDA_TRY(cudaMemcpyAsync(dst->k_data, src->k_data, src->bytes, cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)));
    return VOX_ATTN_OK;
}

}  // extern "C"
