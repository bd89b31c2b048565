"""CPU tests that pin the oracle: the C restatement against fixtures generated from the
reference's own ggml CPU backend, and against that backend itself where it is present."""
import numpy as np
import pytest

from cases import (CASES, KV_TYPE, QKV_CASE, ROPE_CASES, digest, layer_inputs, layer_tail, make_inputs, pick_rows, qkv_inputs, rel_err,
                   rope_inputs, split_qkv)

# tolerance of the restatement against the reference's accurate path (both f32; they differ by
# summation order and libm vs vectorised expf only)
GATE_TOL = 2e-5
# the as-shipped row path keeps an fp16 accumulator for f16 V: the order of the fp16 roundings
# differs between the scalar restatement and the reference's SIMD code
SHIPPED_TOL = {"f16": 5e-3, "q8_0": 2e-5, "f32": 2e-5}


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_golden_gate(name, oracle, vo, golden):
    case = CASES[name]
    inp = make_inputs(case, oracle)
    assert digest(inp) == bytes(golden[name + "/digest"]).decode(), "input generator drifted from the fixtures"
    gate = golden[name + "/gate"]
    kt = KV_TYPE[case["kv"]]
    exact = oracle.attn(inp["q"], inp["k"], inp["v"], inp["mask"], kv_type=kt, path=vo.PATH_ROW_F32)
    assert rel_err(pick_rows(exact, case), gate) < GATE_TOL
    tiled = oracle.attn(inp["q"], inp["k"], inp["v"], inp["mask"], kv_type=kt, path=vo.PATH_TILED)
    assert rel_err(pick_rows(tiled, case), gate) < GATE_TOL
    f64 = oracle.attn(inp["q"], inp["k"], inp["v"], inp["mask"], kv_type=kt, path=vo.PATH_F64)
    assert rel_err(pick_rows(f64, case), gate) < GATE_TOL


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_golden_as_shipped(name, oracle, vo, golden):
    case = CASES[name]
    inp = make_inputs(case, oracle)
    key = name + "/shipped"
    shipped = golden[key] if key in golden.files else golden[name + "/gate"]
    kt = KV_TYPE[case["kv"]]
    # one thread in the fixture => no split-KV: the shipped path is the row loop (or the tiled one)
    path = vo.PATH_TILED if (case["n_q"] >= 64 and case["kv"] != "q8_0") else vo.PATH_ROW
    mine = oracle.attn(inp["q"], inp["k"], inp["v"], inp["mask"], kv_type=kt, path=path)
    assert rel_err(pick_rows(mine, case), shipped) < SHIPPED_TOL[case["kv"]]


@pytest.mark.parametrize("name", sorted(ROPE_CASES))
def test_rope_restatement_matches_the_reference_fixture(name, oracle, golden):
    """cos/sin table + NEOX rotation against ggml_rope_ext as apply_rope calls it.  Both are f32; the reference build
    may fuse x0*cos - x1*sin into an FMA, the restatement does not: one unit in the last place."""
    args = ROPE_CASES[name]
    x, pos, ff = rope_inputs(args)
    table = oracle.rope_table(pos, freq_base=args["freq_base"], attn_factor=args["attn_factor"], freq_factors=ff)
    got = oracle.rope(x, table)
    want = golden[name + "/out"]
    assert np.abs(got - want).max() <= 1e-6 * max(1.0, float(np.abs(want).max()))
    # a rotation scaled by attn_factor: row norms are preserved up to that factor
    assert np.allclose(np.linalg.norm(got, axis=-1), np.linalg.norm(x, axis=-1) * args["attn_factor"], rtol=1e-5)
    # position 0 is the identity (times the factor)
    assert np.allclose(got[0], x[0] * np.float32(args["attn_factor"]), rtol=1e-6, atol=1e-7)


def test_projection_restatement_matches_the_reference_fixture(oracle, golden):
    """ggml_mul_mat with f16 weights + ggml_rope_ext on q and k, as attention_forward issues them (src/minicpm.cpp:660-689):
    the restatement (activations rounded to f16, f32 accumulation; rotation from the cos/sin table) against the
    reference's output.  They differ by the order of the f32 sums only."""
    x, w, pos = qkv_inputs()
    q, k, v = split_qkv(oracle.mul_mat_f16(x, w))
    table = oracle.rope_table(pos, freq_base=QKV_CASE["freq_base"], attn_factor=QKV_CASE["attn_factor"])
    assert rel_err(oracle.rope(q, table), golden["qkv/q"]) < GATE_TOL
    assert rel_err(oracle.rope(k, table), golden["qkv/k"]) < GATE_TOL
    assert rel_err(v, golden["qkv/v"]) < GATE_TOL


def test_layer_tail_restatement_matches_the_reference_fixture(oracle, golden):
    """The rest of a decoder layer after attention (src/minicpm.cpp:715, 718-747, 762-776): ggml_mul_mat(o_proj) with the
    scaled residual add, rms_norm, ggml_mul_mat(gate_up_proj), ggml_swiglu_split, ggml_mul_mat(down_proj) with the scaled
    residual add; the restatement against the reference's own output of the same chain."""
    given = {stage: golden["layer/" + stage] for stage in ("h1", "normed", "gate_up", "fused", "h2")}
    # stage by stage, each from the reference's output of the stage before: sums in another order, nothing else
    staged = layer_tail(oracle, layer_inputs(), given=given)
    assert np.array_equal(staged["normed"], given["normed"])
    for stage in ("h1", "gate_up", "fused", "h2"):
        assert rel_err(staged[stage], given[stage]) < GATE_TOL, stage
    # the whole chain on its own: an f16 rounding of an activation that falls the other way moves an output by about 1e-5
    chain = layer_tail(oracle, layer_inputs())
    assert rel_err(chain["h2"], given["h2"]) < 2e-4


def test_storage_formats_bit_exact(oracle, golden):
    x = golden["storage/x"]
    assert np.array_equal(oracle.quantize_q8_0(x), golden["storage/q8_0"])
    mine = np.array([oracle.lib.voxo_fp32_to_fp16(float(t)) for t in x.ravel()], np.uint16).reshape(x.shape)
    assert np.array_equal(mine, golden["storage/f16"])
    assert np.array_equal(oracle.kv_store(x, 1).view(np.uint16), golden["storage/f16"])
    assert np.array_equal(oracle.kv_store(x, 8), golden["storage/q8_0"])
    # dequantise(quantise(x)) stays within half a quantisation step of x, plus the f16 rounding of
    # the block scale (relative 2^-11) carried by the largest quant (127)
    back = oracle.dequantize_q8_0(golden["storage/q8_0"])
    step = np.abs(x).reshape(64, 2, 32).max(-1, keepdims=True) / 127.0
    bound = step * (0.5 + 127.0 * 2.0 ** -11) * 1.001 + 1e-12
    normal = step >= 2.0 ** -14  # below that the f16 scale itself is subnormal and coarser
    ok = (np.abs(back.reshape(64, 2, 32) - x.reshape(64, 2, 32)) <= bound) | ~normal
    assert bool(ok.all())
    assert int(normal.sum()) > 60


def test_fp16_special_values(oracle):
    cv = oracle.lib.voxo_fp32_to_fp16
    assert cv(0.0) == 0 and cv(-0.0) == 0x8000
    assert cv(65504.0) == 0x7BFF and cv(65519.0) == 0x7BFF and cv(65520.0) == 0x7C00
    assert cv(float("inf")) == 0x7C00 and cv(float("-inf")) == 0xFC00
    assert cv(-1.0e9) == 0xFC00  # the callers' -1e9 mask value becomes -inf in f16
    assert cv(5.960464477539063e-08) == 1 and cv(2.9e-08) == 0  # subnormal edge, ties to even
    for h in (0, 1, 0x3FF, 0x400, 0x3C00, 0x7BFF, 0x8001, 0xFBFF):
        assert cv(oracle.lib.voxo_fp16_to_fp32(h)) == h


def test_masks(oracle):
    m = oracle.causal_mask(np.arange(4, 8), 8)  # 4 new tokens after 4 cached ones
    assert m.shape == (4, 8)
    for r in range(4):
        assert np.all(m[r, : r + 5] == 0) and np.all(np.isneginf(m[r, r + 5:]))
    assert np.signbit(m[0, 0])  # step(..)*-1e9 leaves -0 where visible, as the reference's graph does
    c = oracle.cfg_pair_mask(9)
    assert c.shape == (18, 18)
    assert np.all(c[:9, :9] == 0) and np.all(c[9:, 9:] == 0) and np.all(np.isneginf(c[:9, 9:])) and np.all(np.isneginf(c[9:, :9]))


def test_fully_masked_row_is_zero(oracle, vo):
    case = CASES["masked_row_f32"]
    inp = make_inputs(case, oracle)
    for path in (vo.PATH_ROW, vo.PATH_ROW_F32, vo.PATH_TILED, vo.PATH_F64):
        out = oracle.attn(inp["q"], inp["k"], inp["v"], inp["mask"], kv_type=0, path=path)
        assert np.all(out[0, 1] == 0.0)
        assert np.all(np.isfinite(out))


def test_packed_cfg_pair_equals_batch_form(oracle, vo):
    """The reference packs cond/uncond as 18 tokens with a block-diagonal mask; the engine treats the
    branches as a batch of two 9-token sequences.  The two forms are the same arithmetic."""
    a = make_inputs(CASES["locdit_2x9_f32"], oracle)
    packed_q = np.concatenate([a["q"][0], a["q"][1]], axis=1)[None]
    packed_k = np.concatenate([a["k"][0], a["k"][1]], axis=1)[None]
    packed_v = np.concatenate([a["v"][0], a["v"][1]], axis=1)[None]
    mask = oracle.cfg_pair_mask(9)[None, None]
    batch = oracle.attn(a["q"], a["k"], a["v"], None, kv_type=0, path=vo.PATH_ROW)
    packed = oracle.attn(packed_q, packed_k, packed_v, mask, kv_type=0, path=vo.PATH_ROW)
    assert np.array_equal(packed[0, :9], batch[0]) and np.array_equal(packed[0, 9:], batch[1])


def test_split_kv_merge_matches_single_pass(oracle, vo):
    inp = make_inputs(CASES["decode_kv1024_f16"], oracle)
    one = oracle.attn(inp["q"], inp["kf"], inp["vf"], None, kv_type=0, path=vo.PATH_ROW)
    for n_chunks in (2, 7, 8, 64):
        split = oracle.attn(inp["q"], inp["kf"], inp["vf"], None, kv_type=0, path=vo.PATH_SPLIT_KV, n_chunks=n_chunks)
        assert rel_err(split, one) < 1e-5


def test_oracle_rejects_what_the_reference_rejects(oracle):
    q = np.zeros((1, 3, 1, 64), np.float32)
    k = np.zeros((1, 2, 8, 64), np.float32)
    with pytest.raises(ValueError):  # 3 query heads cannot broadcast over 2 kv heads
        oracle.attn(q, k, k, kv_type=0)


# ------------------------------------------------------------------ live comparison with the reference build

@pytest.mark.parametrize("name", ["decode_kv256_f16_l0", "decode_kv1000_q8", "prefill72_causal_f16", "locdit_2x9_f32",
                                  "odd_nq33_kv75_q8_mask", "prefill512_causal_f16", "decode_kv8192_f16"])
def test_reference_build_reproduces_fixtures(name, ref, oracle, golden):
    case = CASES[name]
    inp = make_inputs(case, oracle)
    gate = ref.attn(inp["q"], inp["kf"], inp["vf"], inp["mask"], kv_type=0, n_threads=1)
    # same library, possibly another ISA variant than the one that wrote the fixture
    assert rel_err(pick_rows(gate, case), golden[name + "/gate"]) < 1e-5


def test_reference_tiled_path_agrees_with_f32_typed_path(ref, oracle):
    """Gate A of the parity plan: f16 K/V with Q replicated to 64 rows runs the reference's tiled f32
    path; its row 0 agrees with the F32-typed run (gate B') far inside the parity tolerance."""
    inp = make_inputs(CASES["decode_kv1024_f16"], oracle)
    q64 = np.repeat(inp["q"], 64, axis=2)
    tiled = ref.attn(q64, inp["k"], inp["v"], None, kv_type=1, n_threads=2)[:, :1]
    typed = ref.attn(inp["q"], inp["kf"], inp["vf"], None, kv_type=0, n_threads=1)
    assert rel_err(tiled, typed) < 2e-5


def test_reference_rope_matches_oracle(ref, oracle):
    rng = np.random.default_rng(6)
    pos = np.array([0, 3, 100, 2047, 4096, 30000], np.int32)
    x = rng.standard_normal((len(pos), 2, 64)).astype(np.float32)
    ff = (1.0 + rng.random(32)).astype(np.float32)
    want = ref.rope(x, pos, freq_base=500000.0, attn_factor=1.1, freq_factors=ff, n_ctx_orig=4096, n_threads=2)
    got = oracle.rope(x, oracle.rope_table(pos, freq_base=500000.0, attn_factor=1.1, freq_factors=ff))
    assert np.abs(got - want).max() <= 1e-6 * float(np.abs(want).max())


def test_reference_quantiser_matches_oracle(ref, oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((257, 64)).astype(np.float32) * 3.0
    assert np.array_equal(ref.quantize_q8_0(x), oracle.quantize_q8_0(x))
    assert np.array_equal(ref.fp32_to_fp16(x).view(np.uint16), oracle.kv_store(x, 1).view(np.uint16))
    blocks = oracle.quantize_q8_0(x)
    assert np.array_equal(ref.dequantize_q8_0(blocks), oracle.dequantize_q8_0(blocks))
