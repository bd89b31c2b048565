/* TEST INFRASTRUCTURE — CPU restatement of the reference's attention operator.
 * See attn_oracle.h for scope and parity status.  Plain C11, scalar, single-threaded.
 *
 * Reference locations (paths inside the reference project):
 *   third_party/ggml/src/ggml-cpu/ops.cpp:8109-8345  row-at-a-time online softmax
 *   third_party/ggml/src/ggml-cpu/ops.cpp:8347-8633  64x64 tiled path
 *   third_party/ggml/src/ggml-cpu/ops.cpp:8637-8705  merge of split-KV partials
 *   third_party/ggml/src/ggml-cpu/ops.cpp:8707-8836  path selection
 *   third_party/ggml/src/ggml-quants.c:199-222,401-415  q8_0 quantise / dequantise
 *   src/minicpm.cpp:602-620, src/locdit.cpp:63-130     the two masks the callers build
 */
#include "attn_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define QK8_0 32
#define TILE_Q 64  /* third_party/ggml/src/ggml-cpu/common.h:9-10 */
#define TILE_KV 64

/* ---------------------------------------------------------------- fp16 <-> fp32 */

float voxo_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t) (h & 0x8000u) << 16;
    const uint32_t exp  = (h >> 10) & 0x1Fu;
    const uint32_t man  = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: value = man * 2^-24 */
            float f = (float) man * 5.9604644775390625e-8f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* round-to-nearest-even, as the F16C instruction and the reference's software path do */
uint16_t voxo_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t) ((x >> 16) & 0x8000u);
    const uint32_t ax   = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) { /* inf / nan */
        return (uint16_t) (sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0u));
    }
    if (ax >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t) (sign | 0x7C00u);
    }
    if (ax < 0x38800000u) { /* result is subnormal or zero: quantum 2^-24 */
        float a;
        memcpy(&a, &ax, 4);
        /* nearbyint rounds to even under the default rounding mode */
        const float r = nearbyintf(a * 16777216.0f);
        return (uint16_t) (sign | (uint16_t) r);
    }
    uint32_t man  = ax & 0x7FFFFFu;
    uint32_t e    = (ax >> 23) - 112u;
    uint32_t half = (e << 10) | (man >> 13);
    const uint32_t rest = man & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) {
        half += 1u; /* may carry into the exponent, which is the correct result */
    }
    return (uint16_t) (sign | half);
}

/* ---------------------------------------------------------------- q8_0 */

typedef struct {
    uint16_t d;
    int8_t   qs[QK8_0];
} blk_q8_0; /* 34 bytes, no padding */

void voxo_quantize_row_q8_0(const float * x, void * yv, int64_t n) {
    uint8_t * y = (uint8_t *) yv;
    const int64_t nblk = n / QK8_0;
    for (int64_t i = 0; i < nblk; ++i) {
        float amax = 0.0f;
        for (int j = 0; j < QK8_0; ++j) {
            const float a = fabsf(x[i * QK8_0 + j]);
            if (a > amax) amax = a;
        }
        const float d  = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        const uint16_t dh = voxo_fp32_to_fp16(d);
        memcpy(y + i * 34, &dh, 2);
        for (int j = 0; j < QK8_0; ++j) {
            const float s = x[i * QK8_0 + j] * id;
            y[i * 34 + 2 + j] = (uint8_t) (int8_t) roundf(s);
        }
    }
}

void voxo_dequantize_row_q8_0(const void * xv, float * y, int64_t n) {
    const uint8_t * x = (const uint8_t *) xv;
    const int64_t nblk = n / QK8_0;
    for (int64_t i = 0; i < nblk; ++i) {
        uint16_t dh;
        memcpy(&dh, x + i * 34, 2);
        const float d = voxo_fp16_to_fp32(dh);
        for (int j = 0; j < QK8_0; ++j) {
            y[i * QK8_0 + j] = (float) (int8_t) x[i * 34 + 2 + j] * d;
        }
    }
}

void voxo_kv_store(const float * x, int64_t n_rows, int64_t D, int type, void * dst) {
    if (type == VOXO_F16) {
        uint16_t * o = (uint16_t *) dst;
        for (int64_t i = 0; i < n_rows * D; ++i) o[i] = voxo_fp32_to_fp16(x[i]);
    } else if (type == VOXO_Q8_0) {
        voxo_quantize_row_q8_0(x, dst, n_rows * D);
    } else {
        memcpy(dst, x, (size_t) (n_rows * D) * sizeof(float));
    }
}

/* ---------------------------------------------------------------- masks */

void voxo_causal_mask(const int32_t * pos, int n_tok, int total_len, uint16_t * mask) {
    for (int r = 0; r < n_tok; ++r) {
        for (int c = 0; c < total_len; ++c) {
            /* step(key - query - 0.5) * -1e9, then cast to f16 */
            const float x    = (float) c - (float) pos[r] - 0.5f;
            const float step = x > 0.0f ? 1.0f : 0.0f;
            mask[(size_t) r * total_len + c] = voxo_fp32_to_fp16(step * -1.0e9f);
        }
    }
}

void voxo_cfg_pair_mask(int seq, uint16_t * mask) {
    const int n = 2 * seq;
    for (int r = 0; r < n; ++r) {
        for (int c = 0; c < n; ++c) {
            mask[(size_t) r * n + c] = voxo_fp32_to_fp16((r / seq) == (c / seq) ? 0.0f : -1.0e9f);
        }
    }
}

/* ---------------------------------------------------------------- helpers */

static size_t row_bytes(int type, int64_t D) {
    switch (type) {
        case VOXO_F32:  return (size_t) D * 4;
        case VOXO_F16:  return (size_t) D * 2;
        case VOXO_Q8_0: return (size_t) (D / QK8_0) * 34;
        default:        return 0;
    }
}

static void row_to_f32(int type, const void * src, float * dst, int64_t D) {
    if (type == VOXO_F32) {
        memcpy(dst, src, (size_t) D * 4);
    } else if (type == VOXO_F16) {
        const uint16_t * s = (const uint16_t *) src;
        for (int64_t d = 0; d < D; ++d) dst[d] = voxo_fp16_to_fp32(s[d]);
    } else {
        voxo_dequantize_row_q8_0(src, dst, D);
    }
}

static const char * kv_row(const voxo_tensor * t, int64_t i1, int64_t i2, int64_t i3) {
    return (const char *) t->data + i1 * t->nb[1] + i2 * t->nb[2] + i3 * t->nb[3];
}

static const uint16_t * mask_row(const voxo_tensor * m, int64_t iq1, int64_t iq2, int64_t iq3) {
    if (!m) return NULL;
    return (const uint16_t *) ((const char *) m->data + iq1 * m->nb[1] + (iq2 % m->ne[2]) * m->nb[2] +
                               (iq3 % m->ne[3]) * m->nb[3]);
}

/* K.Q the way the reference's type traits do it for each K type (ggml-cpu.c:208-261):
 * f32 K: f32 products; f16 K: Q rounded to f16 first; q8_0 K: Q quantised to q8_0 and an
 * integer dot per block scaled by both block scales. */
static float kq_dot_as_shipped(int ktype, const void * krow, const float * qrow, const void * q_conv,
                               int64_t D) {
    if (ktype == VOXO_F32) {
        const float * kf = (const float *) krow;
        float s = 0.0f;
        for (int64_t d = 0; d < D; ++d) s += kf[d] * qrow[d];
        return s;
    }
    if (ktype == VOXO_F16) {
        const uint16_t * kh = (const uint16_t *) krow;
        const uint16_t * qh = (const uint16_t *) q_conv;
        float s = 0.0f;
        for (int64_t d = 0; d < D; ++d) s += voxo_fp16_to_fp32(kh[d]) * voxo_fp16_to_fp32(qh[d]);
        return s;
    }
    const uint8_t * kb = (const uint8_t *) krow;
    const uint8_t * qb = (const uint8_t *) q_conv;
    float s = 0.0f;
    for (int64_t b = 0; b < D / QK8_0; ++b) {
        uint16_t dk, dq;
        memcpy(&dk, kb + b * 34, 2);
        memcpy(&dq, qb + b * 34, 2);
        int32_t acc = 0;
        for (int j = 0; j < QK8_0; ++j) acc += (int32_t) (int8_t) kb[b * 34 + 2 + j] * (int32_t) (int8_t) qb[b * 34 + 2 + j];
        s += (float) acc * (voxo_fp16_to_fp32(dk) * voxo_fp16_to_fp32(dq));
    }
    return s;
}

/* one Q row over KV positions [ic0, ic1): leaves running max M, sum S and the
 * un-normalised accumulator acc[D].  exact != 0 selects the f32-everything variant. */
static void row_online_softmax(const voxo_tensor * k, const voxo_tensor * v, const uint16_t * mp,
                               const float * qrow, int64_t ik2, int64_t ik3, int64_t iv2, int64_t iv3,
                               int64_t ic0, int64_t ic1, float scale, int exact, float * Mout, float * Sout,
                               float * acc) {
    const int64_t D = k->ne[0];
    float    S = 0.0f, M = -INFINITY;
    float    vtmp[256], ktmp[256];
    uint16_t acc16[256];
    uint8_t  qconv[256 * 4];
    const int v_f16_acc = (!exact && v->type == VOXO_F16);

    memset(acc, 0, (size_t) D * sizeof(float));
    memset(acc16, 0, sizeof(acc16));
    if (!exact) {
        if (k->type == VOXO_F16) {
            for (int64_t d = 0; d < D; ++d) ((uint16_t *) qconv)[d] = voxo_fp32_to_fp16(qrow[d]);
        } else if (k->type == VOXO_Q8_0) {
            voxo_quantize_row_q8_0(qrow, qconv, D);
        }
    }

    for (int64_t ic = ic0; ic < ic1; ++ic) {
        const float mv = mp ? voxo_fp16_to_fp32(mp[ic]) : 0.0f;
        if (mv == -INFINITY) continue;

        const void * krow = kv_row(k, ic, ik2, ik3);
        float s;
        if (exact) {
            row_to_f32(k->type, krow, ktmp, D);
            s = 0.0f;
            for (int64_t d = 0; d < D; ++d) s += ktmp[d] * qrow[d];
        } else {
            s = kq_dot_as_shipped(k->type, krow, qrow, qconv, D);
        }
        s = s * scale + mv;

        const float Mold = M;
        float ms = 1.0f, vs = 1.0f;
        if (s > M) {
            M  = s;
            ms = expf(Mold - M);
        } else {
            vs = expf(s - M);
        }
        const void * vrow = kv_row(v, ic, iv2, iv3);
        if (v_f16_acc) {
            const uint16_t * vh = (const uint16_t *) vrow;
            if (ms != 1.0f) {
                for (int64_t d = 0; d < D; ++d) acc16[d] = voxo_fp32_to_fp16(voxo_fp16_to_fp32(acc16[d]) * ms);
            }
            for (int64_t d = 0; d < D; ++d) {
                acc16[d] = voxo_fp32_to_fp16(fmaf(voxo_fp16_to_fp32(vh[d]), vs, voxo_fp16_to_fp32(acc16[d])));
            }
        } else {
            row_to_f32(v->type, vrow, vtmp, D);
            if (ms != 1.0f) {
                for (int64_t d = 0; d < D; ++d) acc[d] *= ms;
            }
            for (int64_t d = 0; d < D; ++d) acc[d] += vtmp[d] * vs;
        }
        S = S * ms + vs;
    }
    if (v_f16_acc) {
        for (int64_t d = 0; d < D; ++d) acc[d] = voxo_fp16_to_fp32(acc16[d]);
    }
    *Mout = M;
    *Sout = S;
}

static float * dst_row(float * dst, int64_t D, int64_t H, int64_t n_q, int64_t iq1, int64_t iq2, int64_t iq3) {
    /* result [D, H, n_q, B]: row index (i3*n_q*H + i2 + i1*H), ops.cpp:8342 */
    return dst + (size_t) (iq3 * n_q * H + iq2 + iq1 * H) * D;
}

/* ---------------------------------------------------------------- paths */

static void path_rows(const voxo_tensor * q, const voxo_tensor * k, const voxo_tensor * v, const voxo_tensor * mask,
                      float scale, int exact, int n_chunks, float * dst) {
    const int64_t D = q->ne[0], n_q = q->ne[1], H = q->ne[2], B = q->ne[3];
    const int64_t n_kv = k->ne[1];
    const int64_t rk2 = H / k->ne[2], rk3 = B / k->ne[3], rv2 = H / v->ne[2], rv3 = B / v->ne[3];
    float acc[256], part[256];

    for (int64_t iq3 = 0; iq3 < B; ++iq3)
    for (int64_t iq2 = 0; iq2 < H; ++iq2)
    for (int64_t iq1 = 0; iq1 < n_q; ++iq1) {
        const float * qrow = (const float *) ((const char *) q->data + iq1 * q->nb[1] + iq2 * q->nb[2] + iq3 * q->nb[3]);
        const uint16_t * mp = mask_row(mask, iq1, iq2, iq3);
        float * out = dst_row(dst, D, H, n_q, iq1, iq2, iq3);
        float M, S;
        if (n_chunks <= 1) {
            row_online_softmax(k, v, mp, qrow, iq2 / rk2, iq3 / rk3, iq2 / rv2, iq3 / rv3, 0, n_kv, scale, exact, &M, &S, acc);
        } else {
            /* split-KV: equal chunks, partial (M,S,acc) per chunk, merged in chunk order */
            const int64_t chunk = (n_kv + n_chunks - 1) / n_chunks;
            float Mf = -INFINITY, Sf = 0.0f;
            memset(acc, 0, sizeof(acc));
            for (int c = 0; c < n_chunks; ++c) {
                const int64_t ic0 = c * chunk;
                if (ic0 >= n_kv) continue;
                const int64_t ic1 = ic0 + chunk < n_kv ? ic0 + chunk : n_kv;
                float Mc, Sc;
                row_online_softmax(k, v, mp, qrow, iq2 / rk2, iq3 / rk3, iq2 / rv2, iq3 / rv3, ic0, ic1, scale, exact, &Mc, &Sc, part);
                if (Sc == 0.0f) continue;
                const float Mn = fmaxf(Mf, Mc);
                const float so = expf(Mf - Mn), sn = expf(Mc - Mn);
                for (int64_t d = 0; d < D; ++d) acc[d] = acc[d] * so + part[d] * sn;
                Sf = Sf * so + Sc * sn;
                Mf = Mn;
            }
            S = Sf;
        }
        const float S_inv = S == 0.0f ? 0.0f : 1.0f / S; /* fully masked row -> zeros */
        for (int64_t d = 0; d < D; ++d) out[d] = acc[d] * S_inv;
    }
}

static void path_tiled(const voxo_tensor * q, const voxo_tensor * k, const voxo_tensor * v, const voxo_tensor * mask,
                       float scale, float * dst) {
    const int64_t D = q->ne[0], n_q = q->ne[1], H = q->ne[2], B = q->ne[3];
    const int64_t n_kv = k->ne[1];
    const int64_t rk2 = H / k->ne[2], rk3 = B / k->ne[3], rv2 = H / v->ne[2], rv3 = B / v->ne[3];

    float * Qt  = (float *) malloc(sizeof(float) * TILE_Q * D);
    float * Kt  = (float *) malloc(sizeof(float) * TILE_KV * D);
    float * Vt  = (float *) malloc(sizeof(float) * TILE_KV * D);
    float * KQ  = (float *) malloc(sizeof(float) * TILE_Q * TILE_KV);
    float * Mk  = (float *) malloc(sizeof(float) * TILE_Q * TILE_KV);
    float * Acc = (float *) malloc(sizeof(float) * TILE_Q * D);

    for (int64_t iq3 = 0; iq3 < B; ++iq3)
    for (int64_t iq2 = 0; iq2 < H; ++iq2)
    for (int64_t iq1 = 0; iq1 < n_q; iq1 += TILE_Q) {
        const int rows = (int) (n_q - iq1 < TILE_Q ? n_q - iq1 : TILE_Q);
        float S[TILE_Q], M[TILE_Q];
        for (int i = 0; i < TILE_Q; ++i) { S[i] = 0.0f; M[i] = -INFINITY; }
        memset(Acc, 0, sizeof(float) * TILE_Q * D);
        for (int t = 0; t < rows; ++t) {
            memcpy(Qt + t * D, (const char *) q->data + (iq1 + t) * q->nb[1] + iq2 * q->nb[2] + iq3 * q->nb[3], sizeof(float) * D);
        }

        for (int64_t ic = 0; ic < n_kv; ic += TILE_KV) {
            const int cols = (int) (n_kv - ic < TILE_KV ? n_kv - ic : TILE_KV);
            int can_skip = mask != NULL;
            if (mask) {
                for (int t = 0; t < rows; ++t) {
                    const uint16_t * mp = mask_row(mask, iq1 + t, iq2, iq3);
                    for (int c = 0; c < cols; ++c) {
                        const float mvv = voxo_fp16_to_fp32(mp[ic + c]);
                        Mk[t * TILE_KV + c] = mvv;
                        if (mvv != -INFINITY) can_skip = 0;
                    }
                }
                if (can_skip) continue; /* whole tile masked, ops.cpp:8493-8512 */
            }
            for (int c = 0; c < cols; ++c) {
                row_to_f32(k->type, kv_row(k, ic + c, iq2 / rk2, iq3 / rk3), Kt + c * D, D);
                row_to_f32(v->type, kv_row(v, ic + c, iq2 / rv2, iq3 / rv3), Vt + c * D, D);
            }
            for (int t = 0; t < rows; ++t) {
                float * row = KQ + t * TILE_KV;
                float tmax = -INFINITY;
                for (int c = 0; c < cols; ++c) {
                    float s = 0.0f;
                    for (int64_t d = 0; d < D; ++d) s += Qt[t * D + d] * Kt[c * D + d];
                    s *= scale;
                    if (mask) s += Mk[t * TILE_KV + c];
                    row[c] = s;
                    if (s > tmax) tmax = s;
                }
                if (tmax == -INFINITY) continue; /* nothing visible in this tile for this row */
                const float Mold = M[t];
                const float Mnew = fmaxf(Mold, tmax);
                if (Mnew > Mold) {
                    const float ms = expf(Mold - Mnew);
                    for (int64_t d = 0; d < D; ++d) Acc[t * D + d] *= ms;
                    S[t] *= ms;
                }
                M[t] = Mnew;
                float sum = 0.0f;
                for (int c = 0; c < cols; ++c) {
                    row[c] = expf(row[c] - Mnew);
                    sum += row[c];
                }
                S[t] += sum;
                for (int c = 0; c < cols; ++c) {
                    const float p = row[c];
                    for (int64_t d = 0; d < D; ++d) Acc[t * D + d] += p * Vt[c * D + d];
                }
            }
        }
        for (int t = 0; t < rows; ++t) {
            const float S_inv = S[t] == 0.0f ? 0.0f : 1.0f / S[t];
            float * out = dst_row(dst, D, H, n_q, iq1 + t, iq2, iq3);
            for (int64_t d = 0; d < D; ++d) out[d] = Acc[t * D + d] * S_inv;
        }
    }
    free(Qt); free(Kt); free(Vt); free(KQ); free(Mk); free(Acc);
}

static void path_f64(const voxo_tensor * q, const voxo_tensor * k, const voxo_tensor * v, const voxo_tensor * mask,
                     float scale, float * dst) {
    const int64_t D = q->ne[0], n_q = q->ne[1], H = q->ne[2], B = q->ne[3];
    const int64_t n_kv = k->ne[1];
    const int64_t rk2 = H / k->ne[2], rk3 = B / k->ne[3], rv2 = H / v->ne[2], rv3 = B / v->ne[3];
    double * s = (double *) malloc(sizeof(double) * (size_t) n_kv);
    float tmp[256];

    for (int64_t iq3 = 0; iq3 < B; ++iq3)
    for (int64_t iq2 = 0; iq2 < H; ++iq2)
    for (int64_t iq1 = 0; iq1 < n_q; ++iq1) {
        const float * qrow = (const float *) ((const char *) q->data + iq1 * q->nb[1] + iq2 * q->nb[2] + iq3 * q->nb[3]);
        const uint16_t * mp = mask_row(mask, iq1, iq2, iq3);
        double mx = -INFINITY;
        for (int64_t ic = 0; ic < n_kv; ++ic) {
            row_to_f32(k->type, kv_row(k, ic, iq2 / rk2, iq3 / rk3), tmp, D);
            double a = 0.0;
            for (int64_t d = 0; d < D; ++d) a += (double) tmp[d] * (double) qrow[d];
            a = a * (double) scale + (mp ? (double) voxo_fp16_to_fp32(mp[ic]) : 0.0);
            s[ic] = a;
            if (a > mx) mx = a;
        }
        double acc[256] = {0}, sum = 0.0;
        if (mx != -INFINITY) {
            for (int64_t ic = 0; ic < n_kv; ++ic) {
                if (s[ic] == -INFINITY) continue;
                const double p = exp(s[ic] - mx);
                sum += p;
                row_to_f32(v->type, kv_row(v, ic, iq2 / rv2, iq3 / rv3), tmp, D);
                for (int64_t d = 0; d < D; ++d) acc[d] += p * (double) tmp[d];
            }
        }
        float * out = dst_row(dst, D, H, n_q, iq1, iq2, iq3);
        for (int64_t d = 0; d < D; ++d) out[d] = sum == 0.0 ? 0.0f : (float) (acc[d] / sum);
    }
    free(s);
}

/* ---------------------------------------------------------------- entry */

int voxo_flash_attn_ext(const voxo_tensor * q, const voxo_tensor * k, const voxo_tensor * v,
                        const voxo_tensor * mask, float scale, int path, int n_chunks, float * dst) {
    if (!q || !k || !v || !dst) return 1;
    if (q->type != VOXO_F32) return 2;
    if (row_bytes(k->type, k->ne[0]) == 0 || row_bytes(v->type, v->ne[0]) == 0) return 2;
    const int64_t D = q->ne[0];
    if (D > 256 || D % QK8_0 != 0) return 3;
    if (k->ne[0] != D || v->ne[0] != D || k->ne[1] != v->ne[1]) return 3;
    if (k->ne[2] == 0 || q->ne[2] % k->ne[2] != 0 || q->ne[2] % v->ne[2] != 0) return 3; /* GQA broadcast */
    if (q->ne[3] != k->ne[3] || q->ne[3] != v->ne[3]) return 3;                          /* ggml.c:5292-5293 */
    if (q->nb[0] != 4 || k->nb[0] != (k->type == VOXO_F32 ? 4u : k->type == VOXO_F16 ? 2u : 34u)) return 4;
    if (mask) {
        if (mask->type != VOXO_F16 || mask->ne[0] < k->ne[1] || mask->ne[1] < q->ne[1]) return 5;
        if (q->ne[2] % mask->ne[2] != 0 || q->ne[3] % mask->ne[3] != 0) return 5;
    }

    if (path == VOXO_PATH_AUTO) {
        const int kv_plain = (k->type == VOXO_F32 || k->type == VOXO_F16) && k->type == v->type;
        if (q->ne[1] == 1 && q->ne[3] == 1 && kv_plain && k->ne[1] >= 512) path = VOXO_PATH_SPLIT_KV;
        else if (kv_plain && q->ne[1] >= TILE_Q) path = VOXO_PATH_TILED;
        else path = VOXO_PATH_ROW;
    }
    switch (path) {
        case VOXO_PATH_ROW:      path_rows(q, k, v, mask, scale, 0, 1, dst); break;
        case VOXO_PATH_ROW_F32:  path_rows(q, k, v, mask, scale, 1, 1, dst); break;
        case VOXO_PATH_SPLIT_KV: path_rows(q, k, v, mask, scale, 0, n_chunks > 0 ? n_chunks : 1, dst); break;
        case VOXO_PATH_TILED:    path_tiled(q, k, v, mask, scale, dst); break;
        case VOXO_PATH_F64:      path_f64(q, k, v, mask, scale, dst); break;
        default: return 6;
    }
    return 0;
}

/* ------------------------------------------------------------------ rotary embedding */

void voxo_rope_table(const int32_t * pos, int64_t n_pos, int n_dims, float freq_base, float attn_factor,
                     const float * freq_factors, float * table) {
    const float theta_scale = powf(freq_base, -2.0f / n_dims); /* ops.cpp:5778 */
    for (int64_t p = 0; p < n_pos; ++p) {
        float theta = (float) pos[p]; /* theta_base = position (ops.cpp: cache init per token) */
        for (int i0 = 0; i0 < n_dims; i0 += 2) {
            const float ff = freq_factors ? freq_factors[i0 / 2] : 1.0f;
            const float th = 1.0f * (theta / ff); /* rope_yarn with freq_scale 1 and ext_factor 0 */
            table[(p * (n_dims / 2) + i0 / 2) * 2 + 0] = cosf(th) * attn_factor;
            table[(p * (n_dims / 2) + i0 / 2) * 2 + 1] = sinf(th) * attn_factor;
            theta *= theta_scale;
        }
    }
}

void voxo_rope_neox(float * x, int64_t n_rows, int n_dims, const float * table, const int32_t * pos_index) {
    const int half = n_dims / 2;
    for (int64_t r = 0; r < n_rows; ++r) {
        const float * tb  = table + (int64_t) pos_index[r] * half * 2;
        float *       row = x + r * n_dims;
        for (int i = 0; i < half; ++i) {
            const float c = tb[2 * i], s = tb[2 * i + 1];
            const float x0 = row[i], x1 = row[i + half];
            row[i]        = x0 * c - x1 * s;
            row[i + half] = x0 * s + x1 * c;
        }
    }
}

/* ------------------------------------------------------------------ Q/K/V projection */

/* ggml_mul_mat with f16 weights as the CPU backend computes it (ggml_compute_forward_mul_mat, vec_dot_type F16:
 * third_party/ggml/src/ggml-cpu/ggml-cpu.c:217; ggml_vec_dot_f16, ggml-cpu/vec.cpp:264): the activations are rounded to
 * f16 (from_float of the vec_dot_type), every product of two f16 values is exact in f32, and the sum is kept in f32
 * (the reference sums in SIMD lanes, so the order differs from this loop; the result agrees to f32 rounding).
 *   x [n_tok][k] f32, w [n_out][k] f16 bits, out [n_tok][n_out] f32 */
void voxo_mul_mat_f16(const float * x, const uint16_t * w, int64_t n_tok, int64_t k, int64_t n_out, float * out) {
    for (int64_t t = 0; t < n_tok; ++t) {
        for (int64_t o = 0; o < n_out; ++o) {
            float acc = 0.0f;
            for (int64_t i = 0; i < k; ++i)
                acc += voxo_fp16_to_fp32(voxo_fp32_to_fp16(x[t * k + i])) * voxo_fp16_to_fp32(w[o * k + i]);
            out[t * n_out + o] = acc;
        }
    }
}

/* MiniCPMModel::rms_norm (src/minicpm.cpp:572-580): ggml_rms_norm (ggml_compute_forward_rms_norm_f32,
 * third_party/ggml/src/ggml-cpu/ops.cpp:3725-3755: the sum of squares in double, mean and scale in float, y = x * scale),
 * then ggml_mul with the weight.   x, out [n_tok][k] f32, w [k] f32 */
void voxo_rms_norm_mul(const float * x, const float * w, float eps, int64_t n_tok, int64_t k, float * out) {
    for (int64_t t = 0; t < n_tok; ++t) {
        double sum = 0.0;
        for (int64_t i = 0; i < k; ++i) sum += (double) (x[t * k + i] * x[t * k + i]);
        const float mean  = (float) (sum / (double) k);
        const float scale = 1.0f / sqrtf(mean + eps);
        for (int64_t i = 0; i < k; ++i) {
            const float y = x[t * k + i] * scale;
            out[t * k + i] = y * w[i];
        }
    }
}

/* ggml_swiglu_split(gate, up) as MiniCPMModel::mlp_forward issues it (src/minicpm.cpp:738-741): silu(gate) * up with
 * silu(x) = x / (1 + expf(-x)) (ggml_silu_f32, third_party/ggml/src/ggml-cpu/vec.h:1061; ggml_vec_swiglu_f32,
 * ggml-cpu/vec.cpp:433-469, whose SIMD paths use a polynomial expf that agrees to a few units in the last place). */
void voxo_swiglu(const float * gate, const float * up, int64_t n, float * out) {
    for (int64_t i = 0; i < n; ++i) out[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
}
