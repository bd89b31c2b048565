"""The batched Q/K/V projection (vox_qkv_project) against the oracle and the reference's fixture: ggml_mul_mat with f16
weights, ggml_rope_ext on q and k, and the store of the new rows into the cache, for all streams of a group in one launch
(src/minicpm.cpp:644-701).  Tolerance: the tensor core sums the same exact f16 x f16 products in f32 in another order than
the reference's SIMD lanes, so results agree to a few f32 roundings of a 1024-term sum: 1e-4 of the output RMS is asserted
(measured: about 1e-6)."""
import numpy as np
import pytest

from cases import KV_TYPE, QKV_CASE, qkv_inputs, rel_err, split_qkv

pytestmark = pytest.mark.gpu

H, HK, D = 16, 2, 64
TOL = 1e-4


def dev(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def test_projection_matches_the_reference_fixture(engine, oracle, golden):
    x, w, pos = qkv_inputs()
    table = oracle.rope_table(pos, freq_base=QKV_CASE["freq_base"], attn_factor=QKV_CASE["attn_factor"])
    q, k, v = engine.qkv_project(dev(x), dev(w), H, HK, rope_table=dev(table))
    engine.sync_status()
    assert rel_err(q.cpu().numpy(), golden["qkv/q"]) < TOL
    assert rel_err(k.cpu().numpy(), golden["qkv/k"]) < TOL
    assert rel_err(v.cpu().numpy(), golden["qkv/v"]) < TOL


@pytest.mark.parametrize("n_tok", [1, 127, 128, 129, 256, 300])
@pytest.mark.parametrize("rope", [False, True])
def test_projection_for_any_number_of_streams(n_tok, rope, engine, oracle):
    x, w, pos = qkv_inputs(n_tok=n_tok)
    table = oracle.rope_table(pos, freq_base=1000000.0, attn_factor=1.1) if rope else None
    launches = engine.launches
    q, k, v = engine.qkv_project(dev(x), dev(w), H, HK, rope_table=dev(table) if rope else None)
    engine.sync_status()
    assert engine.launches - launches == 2  # the f16 copy of the activations, the projection
    qr, kr, vr = split_qkv(oracle.mul_mat_f16(x, w))
    if rope:
        qr, kr = oracle.rope(qr, table), oracle.rope(kr, table)
    assert rel_err(q.cpu().numpy(), qr) < TOL and rel_err(k.cpu().numpy(), kr) < TOL and rel_err(v.cpu().numpy(), vr) < TOL


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_projection_stores_the_rows_and_decode_attends_to_them(kv, engine, pkg, oracle, vo):
    """The whole front of a decode step on the device: projection with the rotary embedding, K/V rows written straight into
    the cache at each stream's position, then decode attention with kv_len = position + 1 and nothing to append.  The
    stored rows are what storing the oracle's projection would give (up to the storage type's rounding of values that
    differ in their last f32 bits), and the attention output matches the oracle's over exactly the stored rows."""
    import torch
    lens = [1, 64, 65, 700, 1500, 2048]  # rows after this step
    S, cap = len(lens), 2048
    rng = np.random.default_rng(12)
    cache = pkg.KVCache(engine, 2, S, HK, cap, KV_TYPE[kv])
    for s, n in enumerate(lens):
        if n > 1:
            past_k = rng.standard_normal((HK, n - 1, D)).astype(np.float32)
            past_v = rng.standard_normal((HK, n - 1, D)).astype(np.float32)
            cache.import_(1, s, oracle.kv_store(past_k, KV_TYPE[kv]), oracle.kv_store(past_v, KV_TYPE[kv]))
    x, w, _ = qkv_inputs(n_tok=S)
    pos = np.array(lens, np.int32) - 1
    table = oracle.rope_table(pos, freq_base=10000.0, attn_factor=1.0)
    q, k_none, v_none = engine.qkv_project(dev(x), dev(w), H, HK, rope_table=dev(table), cache=cache, layer=1, positions=dev(pos))
    assert k_none is None and v_none is None
    out = cache.decode(1, q, dev(np.array(lens, np.int32)), max(lens))
    engine.sync_status()
    qr, kr, vr = split_qkv(oracle.mul_mat_f16(x, w))
    qr, kr = oracle.rope(qr, table), oracle.rope(kr, table)
    assert rel_err(q.cpu().numpy(), qr) < TOL
    out = out.cpu().numpy()
    step = {"f16": 2.0 ** -10, "q8_0": 1.0 / 100}[kv]  # one unit of the storage type against the row's largest value
    for s, n in enumerate(lens):
        ke, ve = cache.export(1, s, n)
        for got, want in ((ke, kr[s]), (ve, vr[s])):
            stored = oracle.dequantize_q8_0(got[:, n - 1]) if kv == "q8_0" else got[:, n - 1].astype(np.float32)
            assert np.abs(stored - want).max() <= step * np.abs(want).max() + 1e-6
        ref = oracle.attn(qr[s][None, :, None, :], ke[None], ve[None], kv_type=KV_TYPE[kv], path=vo.PATH_ROW_F32)[0, 0]
        assert rel_err(out[s], ref) < {"f16": 2e-3, "q8_0": 1e-2}[kv], f"stream {s}"
    assert not cache.export(0, 0, cap)[0].view(np.uint8).any()  # the other layer was not touched


def test_projection_refuses_bad_arguments(engine, pkg):
    import torch
    x = torch.zeros((4, 1024), device="cuda")
    w = torch.zeros((1280, 1024), device="cuda", dtype=torch.float16)
    with pytest.raises(pkg.VoxError) as e:
        engine.qkv_project(x[:, :1000], w[:, :1000], H, HK)  # hidden not a multiple of 64
    assert e.value.status_name in ("UNSUPPORTED", "INVALID_ARGUMENT")
    cache = pkg.KVCache(engine, 1, 2, HK, 64, pkg.F16)
    with pytest.raises(pkg.VoxError) as e:  # more streams than the cache holds
        engine.qkv_project(x, w, H, HK, cache=cache, layer=0, positions=torch.zeros(4, dtype=torch.int32, device="cuda"))
    assert e.value.status_name == "INVALID_ARGUMENT"
    # a position beyond the rows is reported, nothing is written for it
    q, _, _ = engine.qkv_project(x[:2], w, H, HK, cache=cache, layer=0, positions=torch.tensor([64, 3], dtype=torch.int32, device="cuda"))
    with pytest.raises(pkg.VoxError) as e:
        engine.sync_status()
    assert e.value.status_name == "DEVICE_STATE"


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_group_step_from_hidden_states(kv, engine, pkg, oracle, vo):
    """vox_group_step with projection weights set: every layer is projection (rotary embedding included) + decode
    attention, from the hidden states alone.  Checked against the same step fed with the oracle's projections."""
    import torch
    lens = np.array([5, 300, 64, 1023], np.int32)
    S, L, hidden = len(lens), 3, 1024
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((L, (H + 2 * HK) * D, hidden)) / np.sqrt(hidden)).astype(np.float16)
    x = rng.standard_normal((L, S, hidden)).astype(np.float32)
    ff = np.linspace(1.0, 2.0, 32, dtype=np.float32)
    outs = []
    for mode in ("hidden", "projected"):
        g = pkg.Group(engine, n_streams=S, max_len=1088, kv_type=KV_TYPE[kv], base_layers=2, res_layers=1, locdit_layers=0, cfm_steps=0)
        g.set_kv_len(lens)
        g.fill_synthetic(seed=3)
        g.set_rope(freq_base=10000.0, attn_factor=1.0, freq_factors=ff)
        shapes = g.buffer_shapes()
        bufs = {"lm_out": torch.full(shapes["lm_out"], float("nan"), device="cuda")}
        if mode == "hidden":
            wd = dev(w)
            g.set_qkv_weights(wd)
            bufs["lm_hidden"] = dev(x)
        else:  # the oracle's projection, not rotated: the step rotates it
            q, k, v = zip(*(split_qkv(oracle.mul_mat_f16(x[l], w[l])) for l in range(L)))
            bufs.update(lm_q=dev(np.stack(q)), lm_k_new=dev(np.stack(k)), lm_v_new=dev(np.stack(v)))
        g.step(bufs, advance=True)
        engine.sync_status()
        outs.append((bufs["lm_out"].cpu().numpy(), [[g.cache(st).export(l, s, int(lens[s]) + 1) for s in range(S)] for st, l in ((0, 0), (0, 1), (1, 0))]))
        assert list(g.kv_len()) == list(lens + 1)
        g.close()
    (a, rows_a), (b, rows_b) = outs
    assert np.all(np.isfinite(a))
    assert rel_err(a, b) < {"f16": 2e-3, "q8_0": 1e-2}[kv]
    for la, lb in zip(rows_a, rows_b):  # the stored rows: equal up to a unit of the storage type where the projections differ in their last bits
        for (ka, va), (kb, vb) in zip(la, lb):
            fa = oracle.dequantize_q8_0(ka) if kv == "q8_0" else ka.astype(np.float32)
            fb = oracle.dequantize_q8_0(kb) if kv == "q8_0" else kb.astype(np.float32)
            assert np.abs(fa - fb).max() <= ({"f16": 2.0 ** -10, "q8_0": 1.0 / 100}[kv]) * np.abs(fb).max()
