"""Seeded operand sets shared by the golden-fixture generator and the parity tests.

Each case names shapes in the reference's terms (n_q query rows, n_kv cache rows, H query heads,
HK key/value heads, batch B) plus the K/V storage type and the mask the reference's callers
would build.  ``make_inputs`` regenerates the operands from the seed, so fixtures store outputs
only (and a digest of the inputs, to detect generator drift).
"""
from __future__ import annotations

import hashlib

import numpy as np

D = 64

CASES = {
    # config 1: backbone single-token decode, f16 cache (one layer per seed)
    "decode_kv256_f16_l0": dict(B=1, n_q=1, n_kv=256, H=16, HK=2, kv="f16", mask=None, seed=0),
    "decode_kv256_f16_l1": dict(B=1, n_q=1, n_kv=256, H=16, HK=2, kv="f16", mask=None, seed=1),
    # config 4: long-form decode, both cache types, ragged lengths that are no tile multiple
    "decode_kv1024_f16": dict(B=1, n_q=1, n_kv=1024, H=16, HK=2, kv="f16", mask=None, seed=2),
    "decode_kv2048_b2_f16": dict(B=2, n_q=1, n_kv=2048, H=16, HK=2, kv="f16", mask=None, seed=3),
    "decode_kv777_f16": dict(B=1, n_q=1, n_kv=777, H=16, HK=2, kv="f16", mask=None, seed=4),
    "decode_kv256_q8": dict(B=1, n_q=1, n_kv=256, H=16, HK=2, kv="q8_0", mask=None, seed=5),
    "decode_kv1000_q8": dict(B=1, n_q=1, n_kv=1000, H=16, HK=2, kv="q8_0", mask=None, seed=6),
    "decode_kv1_f16": dict(B=1, n_q=1, n_kv=1, H=16, HK=2, kv="f16", mask=None, seed=7),
    # config 2: causal prefill (reference mask from create_causal_mask)
    "prefill72_causal_f16": dict(B=1, n_q=72, n_kv=72, H=16, HK=2, kv="f16", mask="causal", seed=8, q_f16=True),
    "prefill128_gqa4_causal_f16": dict(B=2, n_q=128, n_kv=128, H=4, HK=1, kv="f16", mask="causal", seed=9, q_f16=True),
    # config 3: LocDiT, batch form and the reference's packed 18-token form with block-diagonal mask
    "locdit_2x9_f32": dict(B=2, n_q=9, n_kv=9, H=16, HK=2, kv="f32", mask=None, seed=10),
    "locdit_packed18_f32": dict(B=1, n_q=18, n_kv=18, H=16, HK=2, kv="f32", mask="cfg_pair", seed=10),
    # LocEnc patch: 5 tokens, no mask
    "locenc_5_f32": dict(B=1, n_q=5, n_kv=5, H=16, HK=2, kv="f32", mask=None, seed=11),
    # contract edges exercised by ggml's own op test grid (odd sizes, random block mask, q8_0 with n_q > 1)
    "odd_nq3_kv113_f16_mask": dict(B=1, n_q=3, n_kv=113, H=16, HK=2, kv="f16", mask="random", seed=12),
    "odd_nq33_kv75_q8_mask": dict(B=2, n_q=33, n_kv=75, H=8, HK=2, kv="q8_0", mask="random", seed=13),
    "masked_row_f32": dict(B=1, n_q=4, n_kv=40, H=4, HK=4, kv="f32", mask="row_masked", seed=14),
    # the configured full sizes that the reference's CPU code finishes in seconds: prefill of a 512-token prompt
    # (fixture keeps a sample of the query rows, see golden_rows) and long-form decode at 4096 / 8192 rows
    "prefill512_causal_f16": dict(B=1, n_q=512, n_kv=512, H=16, HK=2, kv="f16", mask="causal", seed=15, q_f16=True, sample_rows=True),
    "decode_kv4096_f16": dict(B=1, n_q=1, n_kv=4096, H=16, HK=2, kv="f16", mask=None, seed=16),
    "decode_kv8192_f16": dict(B=1, n_q=1, n_kv=8192, H=16, HK=2, kv="f16", mask=None, seed=17),
    "decode_kv4096_q8": dict(B=1, n_q=1, n_kv=4096, H=16, HK=2, kv="q8_0", mask=None, seed=18),
    "decode_kv8192_q8": dict(B=1, n_q=1, n_kv=8192, H=16, HK=2, kv="q8_0", mask=None, seed=19),
}


def golden_rows(case):
    """Query rows of the output a fixture keeps: all of them, or for the large prefill case the first and last eight and
    every 13th in between (every 128-row tile, its first and last rows and the diagonal tiles are all represented)."""
    n_q = case["n_q"]
    if not case.get("sample_rows"):
        return np.arange(n_q)
    return np.unique(np.concatenate([np.arange(8), np.arange(8, n_q - 8, 13), np.arange(120, 136), np.arange(n_q - 8, n_q)]))


def pick_rows(out, case):
    """The rows of an operator result [B, n_q, H, D] that the case's fixture holds."""
    return np.asarray(out)[:, golden_rows(case)]


def make_mask(case, oracle):
    kind, n_q, n_kv = case["mask"], case["n_q"], case["n_kv"]
    if kind is None:
        return None
    if kind == "causal":
        return oracle.causal_mask(np.arange(n_kv - n_q, n_kv), n_kv)[None, None]
    if kind == "cfg_pair":
        return oracle.cfg_pair_mask(n_q // 2)[None, None]
    rng = np.random.default_rng(1000 + case["seed"])
    m = np.where(rng.random((1, 1, n_q, n_kv)) < 0.3, -np.inf, 0.0).astype(np.float16)
    m[..., 0] = 0.0  # keep at least one key visible per row
    if kind == "row_masked":
        m[0, 0, 1, :] = -np.inf  # one query row sees nothing: the reference returns zeros for it
    return m


def make_inputs(case, oracle):
    """Returns q [B,H,n_q,64] f32, k/v in the case's storage type, mask or None, and f32 views of
    exactly the K/V values the stored type holds."""
    rng = np.random.default_rng(case["seed"])
    B, n_q, n_kv, H, HK = case["B"], case["n_q"], case["n_kv"], case["H"], case["HK"]
    q = rng.standard_normal((B, H, n_q, D)).astype(np.float32)
    k = rng.standard_normal((B, HK, n_kv, D)).astype(np.float32)
    v = rng.standard_normal((B, HK, n_kv, D)).astype(np.float32)
    if case.get("q_f16"):
        q = q.astype(np.float16).astype(np.float32)
    if case["kv"] == "f16":
        ks, vs = k.astype(np.float16), v.astype(np.float16)
        kf, vf = ks.astype(np.float32), vs.astype(np.float32)
    elif case["kv"] == "q8_0":
        ks, vs = oracle.quantize_q8_0(k), oracle.quantize_q8_0(v)
        kf, vf = oracle.dequantize_q8_0(ks), oracle.dequantize_q8_0(vs)
    else:
        ks, vs, kf, vf = k, v, k, v
    return dict(q=q, k=ks, v=vs, kf=kf, vf=vf, mask=make_mask(case, oracle))


# Rotary embedding: (tokens, heads) of 64-wide rows at the listed positions; "long" uses per-frequency factors
# and the magnitude factor apply_rope derives for sequences beyond the original context.
ROPE_CASES = {
    "rope_plain": dict(seed=30, n_heads=16, freq_base=10000.0, attn_factor=1.0, factors=False, n_ctx_orig=32768,
                       positions=[0, 1, 2, 63, 64, 255, 1000, 4095]),
    "rope_long": dict(seed=31, n_heads=2, freq_base=1000000.0, attn_factor=1.1893, factors=True, n_ctx_orig=4096,
                      positions=[0, 7, 511, 4096, 8191, 20000, 32767]),
}


# Q/K/V projection of a decode step (src/minicpm.cpp:644-689): tokens at the listed positions, hidden 1024 -> 16 Q, 2 K, 2 V
# heads of 64, f16 weights in ggml's layout [features][hidden], rotary embedding on q and k.
QKV_CASE = dict(seed=40, hidden=1024, n_heads=16, n_kv_heads=2, positions=[0, 3, 100, 2047, 4095], freq_base=10000.0, attn_factor=1.0)


def qkv_inputs(args=QKV_CASE, n_tok=None):
    rng = np.random.default_rng(args["seed"])
    pos = np.array(args["positions"], np.int32) if n_tok is None else rng.integers(0, 4096, n_tok).astype(np.int32)
    n_out = (args["n_heads"] + 2 * args["n_kv_heads"]) * D
    w = (rng.standard_normal((n_out, args["hidden"])) / np.sqrt(args["hidden"])).astype(np.float16)
    x = rng.standard_normal((len(pos), args["hidden"])).astype(np.float32)
    return x, w, pos


def split_qkv(y, args=QKV_CASE):
    """[n_tok, (H + 2 HK) * 64] -> q [n_tok, H, 64], k, v [n_tok, HK, 64] (the views attention_forward takes of qkv)."""
    n, H, HK = y.shape[0], args["n_heads"], args["n_kv_heads"]
    return (y[:, :H * D].reshape(n, H, D), y[:, H * D:(H + HK) * D].reshape(n, HK, D), y[:, (H + HK) * D:].reshape(n, HK, D))


# The rest of a decoder layer for single-token steps (src/minicpm.cpp:715, 718-747, 762-776): output projection with the
# scaled residual add, RMS norm, gate_up projection, SwiGLU, down projection with the scaled residual add.  f16 weights in
# ggml's layout [features][inputs]; scale = scale_depth / sqrt(num_layers) of the 24-layer model.
LAYER_CASE = dict(seed=41, hidden=1024, inter=4096, n_tok=5, eps=1e-5, scale=1.4 / np.sqrt(24.0))


def layer_inputs(args=LAYER_CASE, n_tok=None):
    rng = np.random.default_rng(args["seed"])
    n, hid, inter = args["n_tok"] if n_tok is None else n_tok, args["hidden"], args["inter"]
    return dict(attn=rng.standard_normal((n, hid)).astype(np.float32),
                hidden=rng.standard_normal((n, hid)).astype(np.float32),
                w_o=(rng.standard_normal((hid, hid)) / np.sqrt(hid)).astype(np.float16),
                norm_w=(1.0 + 0.1 * rng.standard_normal(hid)).astype(np.float32),
                w_gate_up=(rng.standard_normal((2 * inter, hid)) / np.sqrt(hid)).astype(np.float16),
                w_down=(rng.standard_normal((hid, inter)) / np.sqrt(inter)).astype(np.float16))


def layer_tail(ops, inp, args=LAYER_CASE, given=None):
    """The chain above with `ops` providing mul_mat_f16, rms_norm_mul and swiglu (the oracle, or the reference build).
    Returns every stage: h1 (hidden state after attention), normed, gate_up, fused (the SwiGLU output), h2 (the layer's
    output).  With `given` (a mapping stage -> array, e.g. the reference's fixture) each stage is computed from the GIVEN
    output of the stage before instead of from its own: a rounding that falls the other way in one stage (the
    activations are rounded to f16 in front of every product) is then not carried into the next."""
    scale, inter = np.float32(args["scale"]), args["inter"]
    prev = (lambda name, own: own) if given is None else (lambda name, own: np.asarray(given[name]))
    h1 = inp["hidden"] + ops.mul_mat_f16(inp["attn"], inp["w_o"]) * scale
    normed = ops.rms_norm_mul(prev("h1", h1), inp["norm_w"], args["eps"])
    gate_up = ops.mul_mat_f16(prev("normed", normed), inp["w_gate_up"])
    gu = prev("gate_up", gate_up)
    fused = ops.swiglu(np.ascontiguousarray(gu[:, :inter]), np.ascontiguousarray(gu[:, inter:]))
    h2 = prev("h1", h1) + ops.mul_mat_f16(prev("fused", fused), inp["w_down"]) * scale
    return dict(h1=h1, normed=normed, gate_up=gate_up, fused=fused, h2=h2)


def rope_inputs(args):
    rng = np.random.default_rng(args["seed"])
    pos = np.array(args["positions"], np.int32)
    x = rng.standard_normal((len(pos), args["n_heads"], D)).astype(np.float32)
    ff = (1.0 + 3.0 * rng.random(D // 2)).astype(np.float32) if args["factors"] else None
    return x, pos, ff


def digest(inp) -> str:
    h = hashlib.sha256()
    for name in ("q", "k", "v"):
        h.update(np.ascontiguousarray(inp[name]).tobytes())
    if inp["mask"] is not None:
        h.update(np.ascontiguousarray(inp["mask"]).tobytes())
    return h.hexdigest()[:16]


KV_TYPE = {"f32": 0, "f16": 1, "q8_0": 8}


def rel_err(a, b) -> float:
    """max-abs deviation over the RMS of the expected output: the parity metric."""
    b64 = np.asarray(b, np.float64)
    return float(np.abs(np.asarray(a, np.float64) - b64).max() / max(np.sqrt((b64 ** 2).mean()), 1e-30))
