// KV cache object shared by the cache, decode and stream-group translation units.
#pragma once

#include "common.cuh"

constexpr int kKvTile = 64;  // cache rows moved per bulk copy

// A q8_0 cache keeps every 64-row tile of a (layer, stream, kv head) as ONE contiguous span, laid out exactly as the decode
// kernel wants it in shared memory, so that a tile is one bulk copy (cp.async.bulk) instead of four bulk-tensor copies:
//   [K bytes: 64 rows x 64, each byte q + 128][V bytes likewise][K scales: 64 rows x 2 halves][V scales]
// Inside a byte block the 16-byte pieces of row r sit at piece index (d / 16) ^ ((r / 2) % 4): the 64-byte swizzle the
// kernel's shared-memory reads are written for (what a bulk-tensor copy with CU_TENSOR_MAP_SWIZZLE_64B would produce).
constexpr int kQ8TileBytes = 2 * kKvTile * 64 + 2 * kKvTile * 4;  // 8704
constexpr int kQ8VBytesOff = kKvTile * 64, kQ8KScaleOff = 2 * kKvTile * 64, kQ8VScaleOff = 2 * kKvTile * 64 + kKvTile * 4;
// where row `pos` of a pair starts its tile, and where value d / scale b of that row lie inside the tile's byte / scale block
__host__ __device__ inline size_t   q8_tile_off(int pos) { return (size_t) (pos >> 6) * kQ8TileBytes; }
__host__ __device__ inline uint32_t q8_byte_off(int pos, int d) {
    const int r = pos & 63;
    return (uint32_t) (r * 64 + ((((d >> 4) ^ ((r >> 1) & 3)) << 4) | (d & 15)));
}
__host__ __device__ inline uint32_t q8_scale_off(int pos, int b) { return (uint32_t) ((pos & 63) * 4 + b * 2); }

struct vox_kv_cache {
    vox_engine *  e = nullptr;
    vox_kv_config cfg{};
    // f16: two planes of 128-byte rows, [layer][stream][kv_head][pos][64], nb_* the strides in bytes.
    // q8_0: one run of tiles (see kQ8TileBytes), [layer][stream][kv_head][tile]: k_data is its start, v_data / k_scale /
    // v_scale point at the V bytes / K scales / V scales of the first tile, nb_head / nb_stream / nb_layer (and sb_*,
    // the same) are the strides of a pair / stream / layer, nb_pos is unused: a row's bytes lie at
    // pair + q8_tile_off(pos) + q8_byte_off(pos, d), its scales at pair + q8_tile_off(pos) + q8_scale_off(pos, b).
    uint8_t * k_data = nullptr;
    uint8_t * v_data = nullptr;
    size_t    nb_pos = 0, nb_head = 0, nb_stream = 0, nb_layer = 0;
    uint8_t * k_scale = nullptr;
    uint8_t * v_scale = nullptr;
    size_t    sb_pos = 0, sb_head = 0, sb_stream = 0, sb_layer = 0;
    size_t    bytes  = 0;
    // split-KV arrival tickets of the decode launches on this cache: one int per (layer, stream, kv head), zero
    // between launches.  They belong to the cache so that launches on different caches (or layers) never share one.
    int *     counters = nullptr;
    // f16 only: bulk-tensor descriptors of the planes, 5-D (64, pos, head, stream, layer), box = kKvTile rows
    CUtensorMap map_k, map_v;
};

namespace vox {

// Deterministic N(0,1) value number `idx` of stream `seed`: counter-based, so that any kernel
// (cache fill, benchmarks) can regenerate the same synthetic state without storing it.
__host__ __device__ inline float synth_normal(uint64_t seed, uint64_t idx) {
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + idx * 0xD1B54A32D192ED03ull + 0x632BE59BD9B4E019ull;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    const uint32_t a = static_cast<uint32_t>(z), b = static_cast<uint32_t>(z >> 32);
    const float u1 = (static_cast<float>(a >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
    const float u2 = static_cast<float>(b >> 8) * (1.0f / 16777216.0f);           // [0, 1)
#ifdef __CUDA_ARCH__
    return sqrtf(-2.0f * __logf(u1)) * __cosf(6.2831853f * u2);
#else
    return sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2);
#endif
}

#ifdef __CUDACC__
// q8_0 of one 32-value block held by a half-warp, two values per lane: the arithmetic of
// quantize_row_q8_0_ref (third_party/ggml/src/ggml-quants.c:199-222): d = amax/127, id = d ? 1/d : 0,
// q = roundf(x*id).  All 32 lanes of the warp must call it (the two half-warps are two blocks).
__device__ __forceinline__ void q8_0_quantize_pair(float x0, float x1, char2 & q, float & d) {
    float amax = fmaxf(fabsf(x0), fabsf(x1));
#pragma unroll
    for (int m = 1; m < 16; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    d = amax / 127.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    q.x = (signed char) (int) roundf(x0 * id);
    q.y = (signed char) (int) roundf(x1 * id);
}
// The int8 plane of a q8_0 cache holds q + 128 as unsigned bytes (1..255): such a byte, placed in the low byte of a
// 16-bit word whose high byte is zero, IS the f16 number (q + 128) * 2^-24, so the decode kernel turns bytes into tensor-core
// operands with one byte permute and takes the 128 out of its accumulators once.  vox_kv_export / vox_kv_import
// convert to and from the reference's signed bytes.
__device__ __forceinline__ uchar2 q8_0_biased(char2 q) {
    return make_uchar2((unsigned char) ((int) q.x + 128), (unsigned char) ((int) q.y + 128));
}
#endif

}  // namespace vox
