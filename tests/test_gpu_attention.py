"""GPU parity tests: every entry point of the C ABI against the oracle and the golden fixtures.

Tolerances are the ones the engine is specified to: max-abs deviation relative to the RMS of the
expected output of 2e-3 with f16 (or f32) K/V and 1e-2 with q8_0 K/V.  The expected output is the
reference's accurate path (fixtures) or the oracle's f32 restatement of it on the same stored values.
"""
import ctypes as C

import numpy as np
import pytest

from cases import CASES, KV_TYPE, make_inputs, pick_rows, rel_err

pytestmark = pytest.mark.gpu

TOL = {"f32": 2e-3, "f16": 2e-3, "q8_0": 1e-2}
H, HK, D = 16, 2, 64


def dev(x):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


# ------------------------------------------------------------------ generic operator

@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_matches_reference_fixture(name, engine, oracle, golden):
    case = CASES[name]
    inp = make_inputs(case, oracle)
    out = engine.forward(dev(inp["q"]), dev(inp["k"]), dev(inp["v"]), dev(inp["mask"]) if inp["mask"] is not None else None)
    engine.sync_status()
    out = out.cpu().numpy()
    assert np.all(np.isfinite(out))
    assert rel_err(pick_rows(out, case), golden[name + "/gate"]) < TOL[case["kv"]]
    if case["mask"] == "row_masked":
        assert np.all(out[0, 1] == 0.0)  # a row that sees nothing is zeros, not NaN


@pytest.mark.parametrize("name", ["decode_kv256_f16_l0", "prefill72_causal_f16", "odd_nq33_kv75_q8_mask"])
def test_forward_host_buffers(name, engine, oracle, golden):
    import torch
    case = CASES[name]
    inp = make_inputs(case, oracle)
    t = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in inp.items() if v is not None and k in ("q", "k", "v", "mask")}
    out = engine.forward_host(t["q"], t["k"], t["v"], t.get("mask")).numpy()
    assert rel_err(out, golden[name + "/gate"]) < TOL[case["kv"]]


def test_forward_with_strided_views(engine, oracle, vo):
    """K/V handed over as views of a larger cache tensor (row stride > row size, permuted head axis),
    the way get_k/get_v views of the reference's cache are."""
    import torch
    rng = np.random.default_rng(21)
    n_kv, cap = 200, 256
    q = rng.standard_normal((1, H, 1, D)).astype(np.float32)
    k = rng.standard_normal((1, HK, n_kv, D)).astype(np.float16)
    v = rng.standard_normal((1, HK, n_kv, D)).astype(np.float16)
    kc = torch.zeros((1, HK, cap, D), dtype=torch.float16, device="cuda")
    vc = torch.zeros((1, HK, cap, D), dtype=torch.float16, device="cuda")
    kc[:, :, :n_kv] = dev(k)
    vc[:, :, :n_kv] = dev(v)
    qbig = torch.zeros((1, 1, H, 2 * D), dtype=torch.float32, device="cuda")  # [n_q][H][D] projection layout, padded
    qbig[0, 0, :, :D] = dev(q[0, :, 0])
    qv = qbig[:, :, :, :D].permute(0, 2, 1, 3)
    out = engine.forward(qv, kc[:, :, :n_kv], vc[:, :, :n_kv])
    engine.sync_status()
    ref = oracle.attn(q, k, v, kv_type=vo.F16, path=vo.PATH_ROW_F32)
    assert rel_err(out.cpu().numpy(), ref) < TOL["f16"]


def _ggml_grid():
    """The head-size-64 slice of the reference's own operator test (test_flash_attn_ext,
    third_party/ggml/tests/test-backend-ops.cpp:8286-8329): 4 KV heads, GQA ratio nr2, batch nr3, kv, n_q = nb,
    with and without mask, every K/V type this engine stores."""
    for mask in (True, False):
        for nr3 in (1, 3):
            for nr2 in (1, 4):
                for kv in (113, 512, 1024):
                    if nr2 != 1 and kv != 512:
                        continue
                    for nb in (1, 3, 32, 75):
                        for kv_type in ("f32", "f16", "q8_0"):
                            yield pytest.param(mask, nr3, nr2, kv, nb, kv_type, id=f"mask{int(mask)}-nr3_{nr3}-nr2_{nr2}-kv{kv}-nb{nb}-{kv_type}")


def _kq_mask(rng, n_kv, n_q, ne3):
    """init_tensor_kq_mask of the same file (:152-193): uniform values, and 20 % of the 128x64 blocks set to
    -inf or 0 at random places."""
    m = rng.uniform(-1.0, 1.0, (ne3, 1, n_q, n_kv)).astype(np.float32)
    for _ in range(int(0.2 * m.size / (128 * 64))):
        p3, p1, p0 = rng.integers(ne3), rng.integers(n_q), rng.integers(n_kv)
        m[p3, 0, p1:p1 + 64, p0:p0 + 128] = -np.inf if rng.integers(2) else 0.0
    return m.astype(np.float16)


@pytest.mark.parametrize("mask, nr3, nr2, kv, nb, kv_type", list(_ggml_grid()))
def test_forward_on_the_reference_test_grid(mask, nr3, nr2, kv, nb, kv_type, engine, oracle, vo):
    """Same shapes, value ranges, mask construction and K/V-as-cache-view layout as the reference's backend test, which
    accepts a backend at NMSE <= 5e-4 against its CPU op; here both that metric and this engine's own tolerance apply,
    against the accurate path of the CPU algorithm."""
    import torch
    import zlib
    rng = np.random.default_rng(zlib.crc32(f"{mask}-{nr3}-{nr2}-{kv}-{nb}-{kv_type}".encode()))
    HKg, Hg = 4, 4 * nr2
    q = rng.uniform(-1, 1, (nr3, Hg, nb, D)).astype(np.float32)
    k = rng.uniform(-1, 1, (nr3, HKg, kv, D)).astype(np.float32)
    v = rng.uniform(-1, 1, (nr3, HKg, kv, D)).astype(np.float32)
    if kv_type == "f16":
        ks, vs = k.astype(np.float16), v.astype(np.float16)
    elif kv_type == "q8_0":
        ks, vs = oracle.quantize_q8_0(k), oracle.quantize_q8_0(v)
    else:
        ks, vs = k, v
    m = _kq_mask(rng, kv, nb, nr3) if mask else None
    # K and V are views of tensors twice as long, as in the reference test ("usually a view of the cache")
    def as_view(x):
        t = dev(x)
        big = torch.zeros((t.shape[0], t.shape[1], 2 * t.shape[2], t.shape[3]), dtype=t.dtype, device="cuda")
        big[:, :, :t.shape[2]] = t
        return big[:, :, :t.shape[2]]
    out = engine.forward(dev(q), as_view(ks), as_view(vs), dev(m) if m is not None else None)
    engine.sync_status()
    out = out.cpu().numpy()
    ref = oracle.attn(q, ks, vs, m, kv_type=KV_TYPE[kv_type], path=vo.PATH_ROW_F32)
    assert np.all(np.isfinite(out))
    nmse = float(((out.astype(np.float64) - ref) ** 2).sum() / max((ref.astype(np.float64) ** 2).sum(), 1e-30))
    assert nmse <= 5e-4
    assert rel_err(out, ref) < TOL[kv_type]


def test_forward_refuses_bad_operands(engine, pkg):
    import torch
    q = torch.zeros((1, H, 1, D), device="cuda")
    k = torch.zeros((1, HK, 64, D), dtype=torch.float16, device="cuda")
    with pytest.raises(pkg.VoxError) as e:
        engine.forward(q, k, k[:, :, :32])
    assert e.value.status_name == "INVALID_ARGUMENT"
    with pytest.raises(pkg.VoxError) as e:
        engine.forward(q[:, :15], k, k)
    assert e.value.status_name == "INVALID_ARGUMENT"
    k128 = torch.zeros((1, HK, 64, 128), dtype=torch.float16, device="cuda")
    q128 = torch.zeros((1, H, 1, 128), device="cuda")
    with pytest.raises(pkg.VoxError) as e:
        engine.forward(q128, k128, k128)
    assert e.value.status_name == "UNSUPPORTED"


def test_a_wait_that_runs_out_is_reported_and_the_engine_keeps_working(engine, pkg, oracle, vo):
    """Failure detection without a fault: a kernel waits (about a millisecond) on a barrier nothing arrives at, gives
    up the way every bounded wait of the engine does, and the host reads that as a status; the context is intact."""
    engine.sync_status()
    engine.selftest_wait(limit_cycles=2_000_000)
    with pytest.raises(pkg.VoxError) as e:
        engine.sync_status()
    assert e.value.status_name == "TIMEOUT" and "bounded wait" in str(e.value)
    engine.sync_status()  # the word was cleared by the report
    rng = np.random.default_rng(2)
    q = rng.standard_normal((1, H, 1, D)).astype(np.float32)
    k = rng.standard_normal((1, HK, 300, D)).astype(np.float16)
    v = rng.standard_normal((1, HK, 300, D)).astype(np.float16)
    out = engine.forward(dev(q), dev(k), dev(v))
    engine.sync_status()
    assert rel_err(out.cpu().numpy(), oracle.attn(q, k, v, kv_type=vo.F16, path=vo.PATH_ROW_F32)) < TOL["f16"]
    with pytest.raises(pkg.VoxError):
        engine.selftest_wait(limit_cycles=10 ** 12)  # limits above a second are refused


# ------------------------------------------------------------------ KV cache

@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_append_stores_exactly_what_the_reference_stores(kv, engine, pkg, oracle):
    import torch
    rng = np.random.default_rng(3)
    S, T, L = 3, 37, 2
    cache = pkg.KVCache(engine, n_layers=L, n_streams=S, n_kv_heads=HK, max_len=128, type_=KV_TYPE[kv])
    k = (rng.standard_normal((S, T, HK, D)) * 3).astype(np.float32)
    v = (rng.standard_normal((S, T, HK, D)) * 3).astype(np.float32)
    k[0, 0, 0, :32] = 0.0  # an all-zero block: scale 0, quants 0
    pos = np.array([0, 5, 91], np.int32)
    cache.append(1, dev(k), dev(v), positions=dev(pos))
    engine.sync_status()
    for s in range(S):
        ke, ve = cache.export(1, s, 128)
        want_k = oracle.kv_store(k[s].transpose(1, 0, 2), KV_TYPE[kv])
        want_v = oracle.kv_store(v[s].transpose(1, 0, 2), KV_TYPE[kv])
        got_k = ke[:, pos[s]:pos[s] + T]
        got_v = ve[:, pos[s]:pos[s] + T]
        assert np.array_equal(got_k.view(np.uint8), want_k.view(np.uint8))
        assert np.array_equal(got_v.view(np.uint8), want_v.view(np.uint8))
        untouched = np.delete(ke.view(np.uint8), np.s_[pos[s]:pos[s] + T], axis=1)
        assert not untouched.any()  # nothing outside the appended rows was written
    ke0, _ = cache.export(0, 0, 128)
    assert not ke0.view(np.uint8).any()  # other layers untouched


def test_append_refuses_rows_beyond_capacity(engine, pkg):
    import torch
    cache = pkg.KVCache(engine, 1, 1, HK, 64, pkg.F16)
    k = torch.zeros((1, 8, HK, D), device="cuda")
    with pytest.raises(pkg.VoxError) as e:
        cache.append(0, k, k, pos0=60)
    assert e.value.status_name == "INVALID_ARGUMENT"
    with pytest.raises(pkg.VoxError) as e:
        cache.append(3, k, k, pos0=0)
    assert e.value.status_name == "INVALID_ARGUMENT"


def test_cache_import_export_clear_copy(engine, pkg, oracle):
    rng = np.random.default_rng(8)
    for kv in ("f16", "q8_0"):
        a = pkg.KVCache(engine, 2, 2, HK, 64, KV_TYPE[kv])
        b = pkg.KVCache(engine, 2, 2, HK, 64, KV_TYPE[kv])
        x = rng.standard_normal((HK, 40, D)).astype(np.float32)
        stored = oracle.kv_store(x, KV_TYPE[kv])
        a.import_(1, 1, stored, stored)
        ke, ve = a.export(1, 1, 40)
        assert np.array_equal(ke.view(np.uint8), stored.view(np.uint8)) and np.array_equal(ve.view(np.uint8), stored.view(np.uint8))
        b.copy_from(a)
        engine.sync_status()
        kb, _ = b.export(1, 1, 40)
        assert np.array_equal(kb.view(np.uint8), stored.view(np.uint8))
        a.clear(1)
        engine.sync_status()
        assert not a.export(1, 1, 64)[0].view(np.uint8).any()
        assert a.nbytes > 0


def test_f16_cache_view_feeds_the_generic_operator(engine, pkg, oracle, vo):
    import torch
    rng = np.random.default_rng(9)
    cache = pkg.KVCache(engine, 1, 2, HK, 512, pkg.F16)
    n = 300
    k = rng.standard_normal((HK, n, D)).astype(np.float32)
    v = rng.standard_normal((HK, n, D)).astype(np.float32)
    cache.import_(0, 1, oracle.kv_store(k, vo.F16), oracle.kv_store(v, vo.F16))
    kt, vt = cache.view(0, 1, n)
    q = rng.standard_normal((1, H, 1, D)).astype(np.float32)
    qd = dev(q)
    dst = torch.empty((1, 1, H, D), device="cuda")
    a = pkg.AttnArgs()
    a.q, a.k, a.v, a.mask, a.dst, a.scale = pkg.Tensor.from_torch(qd), kt, vt, pkg.Tensor.none(), pkg.Tensor.from_torch(dst), 0.125
    L = pkg.lib()
    ws = engine.workspace(L.vox_attn_workspace_bytes(C.byref(a)))
    rc = L.vox_attn_forward(engine.h, C.byref(a), C.c_void_p(ws.data_ptr()), ws.numel(), None)
    assert rc == 0, L.vox_attn_last_error_string()
    engine.sync_status()
    ref = oracle.attn(q, oracle.kv_store(k, vo.F16)[None], oracle.kv_store(v, vo.F16)[None], kv_type=vo.F16, path=vo.PATH_ROW_F32)
    assert rel_err(dst.cpu().numpy(), ref) < TOL["f16"]


# ------------------------------------------------------------------ batched decode on the cache

def _fill(cache, oracle, rng, lens, kv, layer=0):
    ks, vs = [], []
    for s, n in enumerate(lens):
        k = rng.standard_normal((HK, n, D)).astype(np.float32)
        v = rng.standard_normal((HK, n, D)).astype(np.float32)
        sk, sv = oracle.kv_store(k, KV_TYPE[kv]), oracle.kv_store(v, KV_TYPE[kv])
        if n:
            cache.import_(layer, s, sk, sv)
        ks.append(sk)
        vs.append(sv)
    return ks, vs


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
@pytest.mark.parametrize("lens", [[256], [1, 2, 63, 64, 65, 127, 128, 129, 130], [1024, 17, 2048, 700], [8192], [0, 5]])
def test_decode_ragged_batch(kv, lens, engine, pkg, oracle, vo):
    rng = np.random.default_rng(len(lens) * 1000 + lens[0])
    S, cap = len(lens), max(64, -(-max(lens) // 64) * 64)
    cache = pkg.KVCache(engine, 2, S, HK, cap, KV_TYPE[kv])
    ks, vs = _fill(cache, oracle, rng, lens, kv, layer=1)
    q = rng.standard_normal((S, H, D)).astype(np.float32)
    out = cache.decode(1, dev(q), dev(np.array(lens, np.int32)), max(lens))
    engine.sync_status()
    out = out.cpu().numpy()
    assert np.all(np.isfinite(out))
    for s, n in enumerate(lens):
        if n == 0:
            assert np.all(out[s] == 0.0)
            continue
        ref = oracle.attn(q[s][None, :, None, :], ks[s][None], vs[s][None], kv_type=KV_TYPE[kv], path=vo.PATH_ROW_F32)[0, 0]
        assert rel_err(out[s], ref) < TOL[kv], f"stream {s} (kv_len {n})"


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
@pytest.mark.parametrize("n_kv", list(range(1, 131, 7)) + [130])
def test_decode_every_tail_length(n_kv, kv, engine, pkg, oracle, vo):
    """kv lengths 1..130 walk through every position of the 16-row warp slices and 64-row tiles."""
    rng = np.random.default_rng(n_kv)
    cache = pkg.KVCache(engine, 1, 1, HK, 192, KV_TYPE[kv])
    ks, vs = _fill(cache, oracle, rng, [n_kv], kv)
    q = rng.standard_normal((1, H, D)).astype(np.float32)
    out = cache.decode(0, dev(q), dev(np.array([n_kv], np.int32)), n_kv).cpu().numpy()
    engine.sync_status()
    ref = oracle.attn(q[0][None, :, None, :], ks[0][None], vs[0][None], kv_type=KV_TYPE[kv], path=vo.PATH_ROW_F32)[0, 0]
    assert rel_err(out[0], ref) < TOL[kv]


@pytest.mark.parametrize("name", ["decode_kv256_f16_l0", "decode_kv1024_f16", "decode_kv2048_b2_f16", "decode_kv777_f16",
                                  "decode_kv256_q8", "decode_kv1000_q8", "decode_kv1_f16", "decode_kv4096_f16", "decode_kv8192_f16",
                                  "decode_kv4096_q8", "decode_kv8192_q8"])
def test_cache_decode_matches_reference_fixture(name, engine, pkg, oracle, golden):
    """The reference's stored K/V (f16 rows / block_q8_0 rows) imported into the cache, decoded by the
    split-KV kernel, against the reference's accurate-path output."""
    case = CASES[name]
    inp = make_inputs(case, oracle)
    B, n_kv = case["B"], case["n_kv"]
    cache = pkg.KVCache(engine, 1, B, case["HK"], -(-n_kv // 64) * 64, KV_TYPE[case["kv"]])
    for b in range(B):
        cache.import_(0, b, inp["k"][b], inp["v"][b])
    q = np.ascontiguousarray(inp["q"][:, :, 0, :])
    out = cache.decode(0, dev(q), dev(np.full(B, n_kv, np.int32)), n_kv).cpu().numpy()
    engine.sync_status()
    assert rel_err(out, golden[name + "/gate"][:, 0]) < TOL[case["kv"]]


def test_decode_ignores_stale_rows_beyond_kv_len(engine, pkg, oracle, vo):
    """Rows past a stream's length (left by an earlier, longer use of the slot) must not leak in."""
    rng = np.random.default_rng(77)
    cache = pkg.KVCache(engine, 1, 1, HK, 256, pkg.F16)
    ks, vs = _fill(cache, oracle, rng, [256], "f16")
    q = rng.standard_normal((1, H, D)).astype(np.float32)
    out = cache.decode(0, dev(q), dev(np.array([100], np.int32)), 256).cpu().numpy()
    engine.sync_status()
    ref = oracle.attn(q[0][None, :, None, :], ks[0][None, :, :100], vs[0][None, :, :100], kv_type=vo.F16, path=vo.PATH_ROW_F32)[0, 0]
    assert rel_err(out[0], ref) < TOL["f16"]


def test_decode_gqa_ratios_and_large_logits(engine, pkg, oracle, vo):
    rng = np.random.default_rng(31)
    for heads, kvh in ((8, 8), (8, 2), (4, 1), (16, 2)):
        cache = pkg.KVCache(engine, 1, 2, kvh, 320, pkg.F16)
        lens = [320, 129]
        q = (rng.standard_normal((2, heads, D)) * 6).astype(np.float32)  # scores up to ~ +-40: max-subtraction matters
        outs = []
        for s, n in enumerate(lens):
            k = rng.standard_normal((kvh, n, D)).astype(np.float32)
            v = rng.standard_normal((kvh, n, D)).astype(np.float32)
            cache.import_(0, s, oracle.kv_store(k, vo.F16), oracle.kv_store(v, vo.F16))
            outs.append(oracle.attn(q[s][None, :, None, :], oracle.kv_store(k, vo.F16)[None], oracle.kv_store(v, vo.F16)[None],
                                    kv_type=vo.F16, path=vo.PATH_ROW_F32)[0, 0])
        out = cache.decode(0, dev(q), dev(np.array(lens, np.int32)), 320).cpu().numpy()
        engine.sync_status()
        for s in range(2):
            assert rel_err(out[s], outs[s]) < TOL["f16"], (heads, kvh, s)


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_decode_stores_the_arriving_row_itself(kv, engine, pkg, oracle, vo):
    """k_new / v_new given to the decode call: same cache bytes and same output bits as append followed by
    decode, with the arriving row on every kind of boundary (first row, tile edges, a chunk of its own)."""
    lens = [1, 2, 16, 17, 64, 65, 128, 512, 513, 1024, 1025, 1537, 2047, 2048, 700]  # lengths including the new row
    rng = np.random.default_rng(77)
    S, cap = len(lens), 2048
    two = [pkg.KVCache(engine, 2, S, HK, cap, KV_TYPE[kv]) for _ in range(2)]
    past = []
    for s, n in enumerate(lens):
        k = rng.standard_normal((HK, n - 1, D)).astype(np.float32)
        v = rng.standard_normal((HK, n - 1, D)).astype(np.float32)
        sk, sv = oracle.kv_store(k, KV_TYPE[kv]), oracle.kv_store(v, KV_TYPE[kv])
        past.append((sk, sv))
        if n > 1:
            for c in two:
                c.import_(1, s, sk, sv)
    q = rng.standard_normal((S, H, D)).astype(np.float32)
    k_new = (rng.standard_normal((S, HK, D)) * 2).astype(np.float32)
    v_new = (rng.standard_normal((S, HK, D)) * 2).astype(np.float32)
    k_new[3, 0, 32:] = 0.0  # an all-zero q8_0 block
    kv_len = dev(np.array(lens, np.int32))
    # separately: append at position len-1, then attend
    two[0].append(1, dev(k_new[:, None]), dev(v_new[:, None]), positions=dev(np.array(lens, np.int32) - 1))
    want = two[0].decode(1, dev(q), kv_len, max(lens))
    # in one launch
    before = engine.launches
    got = two[1].decode(1, dev(q), kv_len, max(lens), k_new=dev(k_new), v_new=dev(v_new))
    engine.sync_status()
    assert engine.launches - before == 1
    import torch
    assert torch.equal(got, want)
    # the same call with the promise that lengths and cache are older than the previous kernel (tiles are then
    # requested before the dependency wait): same row stored again, same bits out
    again = two[1].decode(1, dev(q), kv_len, max(lens), k_new=dev(k_new), v_new=dev(v_new), cache_stable=True)
    engine.sync_status()
    assert torch.equal(again, want)
    # ... and with the streams listed longest first instead of in index order: the work list is then cut at other
    # places, so the partial sums are folded in another order (the same values up to f32 rounding)
    order = np.argsort(-np.array(lens), kind="stable").astype(np.int32)
    again = two[1].decode(1, dev(q), kv_len, max(lens), k_new=dev(k_new), v_new=dev(v_new), cache_stable=True, stream_order=dev(order))
    engine.sync_status()
    assert rel_err(again.cpu().numpy(), want.cpu().numpy()) < TOL[kv] / 50
    out = got.cpu().numpy()
    for s, n in enumerate(lens):
        a, b = two[0].export(1, s, cap), two[1].export(1, s, cap)
        assert np.array_equal(a[0].view(np.uint8), b[0].view(np.uint8)) and np.array_equal(a[1].view(np.uint8), b[1].view(np.uint8))
        assert np.array_equal(b[0][:, n - 1].view(np.uint8), oracle.kv_store(k_new[s][:, None], KV_TYPE[kv])[:, 0].view(np.uint8))
        ref = oracle.attn(q[s][None, :, None, :], b[0][None, :, :n], b[1][None, :, :n], kv_type=KV_TYPE[kv], path=vo.PATH_ROW_F32)[0, 0]
        assert rel_err(out[s], ref) < TOL[kv], f"stream {s} (kv_len {n})"
    # the other layer was not touched
    assert not two[1].export(0, 0, cap)[0].view(np.uint8).any()


def test_decode_with_arriving_row_reports_a_stream_beyond_capacity(engine, pkg):
    import torch
    cache = pkg.KVCache(engine, 1, 2, HK, 64, pkg.F16)
    q = torch.zeros((2, H, D), device="cuda")
    rows = torch.ones((2, HK, D), device="cuda")
    cache.decode(0, q, dev(np.array([65, 3], np.int32)), 64, k_new=rows, v_new=rows)  # stream 0 claims 65 rows of 64
    with pytest.raises(pkg.VoxError) as e:
        engine.sync_status()
    assert e.value.status_name == "DEVICE_STATE" and "longer than its cache rows" in str(e.value)
    k0, _ = cache.export(0, 0, 64)
    assert not k0.view(np.uint8).any()  # nothing was written for the stream that does not fit
    k1, _ = cache.export(0, 1, 64)
    assert np.all(k1[:, 2].astype(np.float32) == 1.0)
    with pytest.raises(pkg.VoxError):
        cache.decode(0, q, dev(np.array([1, 1], np.int32)), 1, k_new=rows)  # v_new missing


def test_rope_table_matches_the_reference_angles(engine, oracle):
    pos = np.array([0, 1, 2, 63, 255, 1000, 4095, 8191, 32767], np.int32)
    rng = np.random.default_rng(4)
    ff = (1.0 + 3.0 * rng.random(32)).astype(np.float32)
    for args in (dict(freq_base=10000.0, attn_factor=1.0, freq_factors=None),
                 dict(freq_base=1000000.0, attn_factor=1.1893, freq_factors=ff)):
        got = engine.rope_table(dev(pos + 1), pos_offset=-1, freq_base=args["freq_base"], attn_factor=args["attn_factor"],
                                freq_factors=dev(ff) if args["freq_factors"] is not None else None)
        engine.sync_status()
        want = oracle.rope_table(pos, **args)
        # same f32 angle (built by the same chain of multiplications); cosf/sinf of the device and of the host's libm
        # may differ in the last place
        assert np.abs(got.cpu().numpy() - want).max() <= 4e-7 * args["attn_factor"]


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_decode_rotates_q_and_the_arriving_row(kv, engine, pkg, oracle, vo):
    """q and k_new handed over BEFORE the rotary embedding, with the step's cos/sin table: the cache must hold the
    rotated K row (bit for bit what the reference's rope + cpy store, given the same table) and the output must be the
    attention of the rotated query."""
    lens = [1, 17, 64, 65, 300, 512, 513, 1025, 2048]
    rng = np.random.default_rng(91)
    S, cap = len(lens), 2048
    cache = pkg.KVCache(engine, 1, S, HK, cap, KV_TYPE[kv])
    for s, n in enumerate(lens):
        if n > 1:
            k = rng.standard_normal((HK, n - 1, D)).astype(np.float32)
            v = rng.standard_normal((HK, n - 1, D)).astype(np.float32)
            cache.import_(0, s, oracle.kv_store(k, KV_TYPE[kv]), oracle.kv_store(v, KV_TYPE[kv]))
    q = rng.standard_normal((S, H, D)).astype(np.float32)
    k_new = rng.standard_normal((S, HK, D)).astype(np.float32)
    v_new = rng.standard_normal((S, HK, D)).astype(np.float32)
    ff = (1.0 + rng.random(32)).astype(np.float32)
    pos = np.array(lens, np.int32) - 1
    table = oracle.rope_table(pos, freq_base=1000000.0, attn_factor=1.05, freq_factors=ff)
    out = cache.decode(0, dev(q), dev(np.array(lens, np.int32)), max(lens), k_new=dev(k_new), v_new=dev(v_new), rope_table=dev(table))
    engine.sync_status()
    out = out.cpu().numpy()
    q_rot, k_rot = oracle.rope(q, table), oracle.rope(k_new, table)
    for s, n in enumerate(lens):
        ke, ve = cache.export(0, s, n)
        assert np.array_equal(ke[:, n - 1].view(np.uint8), oracle.kv_store(k_rot[s][:, None], KV_TYPE[kv])[:, 0].view(np.uint8))
        assert np.array_equal(ve[:, n - 1].view(np.uint8), oracle.kv_store(v_new[s][:, None], KV_TYPE[kv])[:, 0].view(np.uint8))
        ref = oracle.attn(q_rot[s][None, :, None, :], ke[None], ve[None], kv_type=KV_TYPE[kv], path=vo.PATH_ROW_F32)[0, 0]
        assert rel_err(out[s], ref) < TOL[kv], f"stream {s} (kv_len {n})"
    # the device-built table gives the same result within the tolerance (angles may differ in the last place)
    cache2 = pkg.KVCache(engine, 1, S, HK, cap, KV_TYPE[kv])
    cache2.copy_from(cache)
    t_dev = engine.rope_table(dev(np.array(lens, np.int32)), pos_offset=-1, freq_base=1000000.0, attn_factor=1.05, freq_factors=dev(ff))
    out2 = cache2.decode(0, dev(q), dev(np.array(lens, np.int32)), max(lens), k_new=dev(k_new), v_new=dev(v_new), rope_table=t_dev)
    engine.sync_status()
    assert rel_err(out2.cpu().numpy(), out) < TOL[kv] / 20  # q8_0: an angle off in the last place can move a stored byte


def test_decode_refuses_bad_arguments(engine, pkg):
    import torch
    cache = pkg.KVCache(engine, 1, 2, HK, 128, pkg.F16)
    q = torch.zeros((2, H, D), device="cuda")
    lens = torch.zeros(2, dtype=torch.int32, device="cuda")
    for kwargs, status in (({"layer": 1}, "INVALID_ARGUMENT"), ({"kv_bound": 129}, "INVALID_ARGUMENT")):
        with pytest.raises(pkg.VoxError) as e:
            cache.decode(kwargs.get("layer", 0), q, lens, kwargs.get("kv_bound", 128))
        assert e.value.status_name == status
    with pytest.raises(pkg.VoxError) as e:
        cache.decode(0, torch.zeros((3, H, D), device="cuda"), lens, 128)  # more streams than the cache holds
    assert e.value.status_name == "INVALID_ARGUMENT"
    with pytest.raises(pkg.VoxError) as e:
        cache.decode(0, torch.zeros((2, 15, D), device="cuda"), lens, 128)  # 15 heads over 2 kv heads
    assert e.value.status_name == "INVALID_ARGUMENT"


# ------------------------------------------------------------------ LocDiT and prefill

@pytest.mark.parametrize("S, L, seq", [(1, 8, 9), (3, 2, 9), (2, 1, 5), (1, 1, 16), (1, 1, 1)])
def test_locdit_step(S, L, seq, engine, oracle, vo):
    rng = np.random.default_rng(S * 100 + L * 10 + seq)
    q = rng.standard_normal((S, L, 2, H, seq, D)).astype(np.float32)
    k = rng.standard_normal((S, L, 2, HK, seq, D)).astype(np.float32)
    v = rng.standard_normal((S, L, 2, HK, seq, D)).astype(np.float32)
    before = engine.launches
    out = engine.locdit_step(dev(q), dev(k), dev(v))
    engine.sync_status()
    assert engine.launches - before == 1  # all layers, both branches, all heads: one launch
    out = out.cpu().numpy()
    for s in range(S):
        for l in range(L):
            ref = oracle.attn(q[s, l], k[s, l], v[s, l], kv_type=vo.F32, path=vo.PATH_ROW_F32)
            assert rel_err(out[s, l], ref) < TOL["f32"]


def test_locdit_matches_reference_fixture(engine, oracle, golden):
    inp = make_inputs(CASES["locdit_2x9_f32"], oracle)
    out = engine.locdit_step(dev(inp["q"][None, None]), dev(inp["k"][None, None]), dev(inp["v"][None, None]))
    engine.sync_status()
    got = out.cpu().numpy()[0, 0]
    assert rel_err(got, golden["locdit_2x9_f32/gate"]) < TOL["f32"]
    # and it equals the packed 18-token form with the block-diagonal mask that the reference builds
    packed = [np.concatenate([inp[n][0], inp[n][1]], axis=1)[None] for n in ("q", "k", "v")]
    mask = oracle.cfg_pair_mask(9)[None, None]
    via_mask = engine.forward(dev(packed[0]), dev(packed[1]), dev(packed[2]), dev(mask)).cpu().numpy()
    assert rel_err(got[0], via_mask[0, :9]) < 1e-5 and rel_err(got[1], via_mask[0, 9:]) < 1e-5


@pytest.mark.parametrize("name", ["prefill72_causal_f16", "prefill128_gqa4_causal_f16", "prefill512_causal_f16"])
def test_prefill_matches_reference_fixture(name, engine, oracle, golden):
    inp = make_inputs(CASES[name], oracle)
    out = engine.prefill(dev(inp["q"]), dev(inp["k"]), dev(inp["v"]))
    engine.sync_status()
    assert rel_err(pick_rows(out.cpu().numpy(), CASES[name]), golden[name + "/gate"]) < TOL["f16"]


@pytest.mark.parametrize("B, L", [(1, 512), (2, 200), (1, 130)])
def test_prefill_causal(B, L, engine, oracle, vo):
    rng = np.random.default_rng(B * 1000 + L)
    q = rng.standard_normal((B, H, L, D)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((B, HK, L, D)).astype(np.float16)
    v = rng.standard_normal((B, HK, L, D)).astype(np.float16)
    out = engine.prefill(dev(q), dev(k), dev(v))
    engine.sync_status()
    mask = oracle.causal_mask(np.arange(L), L)[None, None]
    ref = oracle.attn(q, k, v, mask, kv_type=vo.F16, path=vo.PATH_TILED)
    assert rel_err(out.cpu().numpy(), ref) < TOL["f16"]


def test_prefill_rising_logits_move_the_reference_maximum(engine, oracle, vo):
    """Scores that keep growing along the key axis (by far more than 2^8 per tile): the running reference of
    the kernel has to be raised inside tiles, in every block position, and the accumulated output rescaled."""
    rng = np.random.default_rng(11)
    B, L = 1, 300
    ramp = (np.arange(L, dtype=np.float32) / L * 15.0)[None, None, :, None]
    q = np.full((B, H, L, D), 0.5, np.float32) + rng.standard_normal((B, H, L, D)).astype(np.float16).astype(np.float32) * 0.05
    q = q.astype(np.float16).astype(np.float32)
    k = (ramp * np.ones((B, HK, L, D), np.float32) + rng.standard_normal((B, HK, L, D)).astype(np.float32) * 0.1).astype(np.float16)
    v = rng.standard_normal((B, HK, L, D)).astype(np.float16)
    out = engine.prefill(dev(q), dev(k), dev(v))
    engine.sync_status()
    mask = oracle.causal_mask(np.arange(L), L)[None, None]
    ref = oracle.attn(q, k, v, mask, kv_type=vo.F16, path=vo.PATH_TILED)
    assert np.all(np.isfinite(out.cpu().numpy()))
    assert rel_err(out.cpu().numpy(), ref) < TOL["f16"]


@pytest.mark.parametrize("n_q, n_kv", [(200, 328), (130, 207), (64, 512), (1, 300), (300, 503), (600, 640)])
def test_prefill_with_past(n_q, n_kv, engine, oracle, vo):
    """A chunk of n_q new tokens attending over n_kv - n_q cached ones and, causally, itself.  Offsets that are no
    multiple of 16 put the 16 tokens of a work item on both sides of a 128-key boundary: the causal cut then reaches
    into the item's last two key tiles, and the second 64-key half of the last one is walked or left out row block by
    row block."""
    rng = np.random.default_rng(n_q * 7 + n_kv)
    B = 2
    q = rng.standard_normal((B, H, n_q, D)).astype(np.float16).astype(np.float32)
    k = rng.standard_normal((B, HK, n_kv, D)).astype(np.float16)
    v = rng.standard_normal((B, HK, n_kv, D)).astype(np.float16)
    out = engine.prefill(dev(q), dev(k), dev(v))
    engine.sync_status()
    mask = oracle.causal_mask(np.arange(n_kv - n_q, n_kv), n_kv)[None, None]
    ref = oracle.attn(q, k, v, mask, kv_type=vo.F16, path=vo.PATH_TILED)
    assert rel_err(out.cpu().numpy(), ref) < TOL["f16"]


# ------------------------------------------------------------------ stream groups

@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_group_step_appends_then_attends(kv, engine, pkg, oracle, vo):
    import torch
    rng = np.random.default_rng(5)
    S = 5
    g = pkg.Group(engine, n_streams=S, max_len=256, kv_type=KV_TYPE[kv], base_layers=2, res_layers=1, cfm_steps=2, locdit_layers=2)
    lens = np.array([10, 64, 127, 200, 1], np.int32)
    g.set_kv_len(lens)
    g.fill_synthetic(seed=1)
    shapes = g.buffer_shapes()
    host = {n: rng.standard_normal(s).astype(np.float32) for n, s in shapes.items() if not n.endswith("out")}
    t = {n: dev(x) for n, x in host.items()}
    t["lm_out"] = torch.zeros(shapes["lm_out"], device="cuda")
    t["dit_out"] = torch.zeros(shapes["dit_out"], device="cuda")
    before = engine.launches
    g.step(t, advance=True)
    engine.sync_status()
    # per LM layer one decode launch that also stores the new row (no merge at these lengths); one length
    # bump; one launch per CFM timestep
    assert engine.launches - before == 3 + 1 + 2
    assert np.array_equal(g.kv_len(), lens + 1)
    lm_out = t["lm_out"].cpu().numpy()
    for l in range(3):
        cache = g.cache(0 if l < 2 else 1)
        layer = l if l < 2 else 0
        for s in range(S):
            ke, ve = cache.export(layer, s, int(lens[s]) + 1)
            # the row appended by this step is the reference's storage of the new K/V row
            assert np.array_equal(ke[:, -1].view(np.uint8), oracle.kv_store(host["lm_k_new"][l, s], KV_TYPE[kv]).view(np.uint8))
            ref = oracle.attn(host["lm_q"][l, s][None, :, None, :], ke[None], ve[None], kv_type=KV_TYPE[kv], path=vo.PATH_ROW_F32)[0, 0]
            assert rel_err(lm_out[l, s], ref) < TOL[kv]
    dit = t["dit_out"].cpu().numpy()
    for step in range(2):
        for s in (0, S - 1):
            for l in range(2):
                ref = oracle.attn(host["dit_q"][step, s, l], host["dit_k"][step, s, l], host["dit_v"][step, s, l], kv_type=vo.F32,
                                  path=vo.PATH_ROW_F32)
                assert rel_err(dit[step, s, l], ref) < TOL["f32"]
    # a second step without advance re-reads the same rows and reproduces the outputs
    t2 = dict(t)
    t2["lm_out"] = torch.zeros(shapes["lm_out"], device="cuda")
    g.step(t2, advance=False)
    engine.sync_status()
    assert np.array_equal(g.kv_len(), lens + 1)


def test_group_step_with_rotary_embedding(engine, pkg, oracle, vo):
    rng = np.random.default_rng(15)
    S = 4
    g = pkg.Group(engine, n_streams=S, max_len=1024, kv_type=pkg.F16, base_layers=2, res_layers=1, cfm_steps=0, locdit_layers=0)
    lens = np.array([5, 64, 700, 1000], np.int32)
    g.set_kv_len(lens)
    g.fill_synthetic(seed=3)
    ff = (1.0 + rng.random(32)).astype(np.float32)
    g.set_rope(freq_base=10000.0, attn_factor=1.0, freq_factors=ff)
    shapes = g.buffer_shapes()
    host = {n: rng.standard_normal(s).astype(np.float32) for n, s in shapes.items() if n.startswith("lm_") and not n.endswith("out")}
    import torch
    t = {n: dev(x) for n, x in host.items()}
    t["lm_out"] = torch.zeros(shapes["lm_out"], device="cuda")
    before = engine.launches
    g.step(t, advance=True)
    engine.sync_status()
    assert engine.launches - before == 3 + 1 + 1  # decode per layer, length update, one rotary table for the step
    table = oracle.rope_table(lens, freq_base=10000.0, attn_factor=1.0, freq_factors=ff)  # positions = old lengths
    lm_out = t["lm_out"].cpu().numpy()
    for l in range(3):
        cache = g.cache(0 if l < 2 else 1)
        layer = l if l < 2 else 0
        q_rot, k_rot = oracle.rope(host["lm_q"][l], table), oracle.rope(host["lm_k_new"][l], table)
        for s in range(S):
            ke, ve = cache.export(layer, s, int(lens[s]) + 1)
            assert np.abs(ke[:, -1].astype(np.float32) - k_rot[s]).max() < 4e-3  # f16 storage of the rotated row
            ref = oracle.attn(q_rot[s][None, :, None, :], ke[None], ve[None], kv_type=vo.F16, path=vo.PATH_ROW_F32)[0, 0]
            assert rel_err(lm_out[l, s], ref) < TOL["f16"]


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_captured_step_replays_for_every_position(kv, engine, pkg):
    """One CUDA graph of an advancing step, replayed: same outputs, same cache rows and same lengths as issuing the step
    anew at every position."""
    import torch
    S, steps = 3, 5
    lens = np.array([60, 250, 1000], np.int32)
    gen = torch.Generator(device="cuda").manual_seed(8)
    groups = []
    for _ in range(2):
        g = pkg.Group(engine, n_streams=S, max_len=1024 + 64, kv_type=KV_TYPE[kv], base_layers=2, res_layers=1, cfm_steps=2, locdit_layers=2)
        g.set_kv_len(lens)
        g.fill_synthetic(seed=9)
        g.set_rope(freq_base=10000.0)
        g.set_bound(1024 + 64)  # both runs size their grids for the capacity, so both split the KV range alike
        groups.append(g)
    shapes = groups[0].buffer_shapes()
    inputs = [{n: torch.randn(s, device="cuda", generator=gen) for n, s in shapes.items() if not n.endswith("out")} for _ in range(steps)]
    # reference run: a fresh launch sequence per position
    want = []
    for i in range(steps):
        t = dict(inputs[i], lm_out=torch.zeros(shapes["lm_out"], device="cuda"), dit_out=torch.zeros(shapes["dit_out"], device="cuda"))
        groups[0].step(t, advance=True)
        want.append((t["lm_out"].clone(), t["dit_out"].clone()))
    engine.sync_status()
    # captured run: static buffers, one graph, bound = capacity
    g = groups[1]
    static = {n: torch.zeros(s, device="cuda") for n, s in shapes.items()}
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            g.step(static, advance=True, stream=side)
    assert np.array_equal(g.kv_len(), lens)  # capturing moved nothing
    for i in range(steps):
        for n, x in inputs[i].items():
            static[n].copy_(x)
        graph.replay()
        g.advance(1)
        torch.cuda.synchronize()
        assert torch.equal(static["lm_out"], want[i][0]) and torch.equal(static["dit_out"], want[i][1]), f"position {i}"
    engine.sync_status()
    assert np.array_equal(g.kv_len(), lens + steps) and np.array_equal(groups[0].kv_len(), lens + steps)
    for stack in (0, 1):
        a, b = groups[0].cache(stack).export(0, 2, 1010), g.cache(stack).export(0, 2, 1010)
        assert np.array_equal(a[0].view(np.uint8), b[0].view(np.uint8)) and np.array_equal(a[1].view(np.uint8), b[1].view(np.uint8))
    with pytest.raises(pkg.VoxError):
        g.set_bound(10)  # below the longest stream


def test_group_step_host_equals_device_step(engine, pkg):
    import torch
    rng = np.random.default_rng(6)
    S = 4
    lens = np.array([33, 100, 255, 7], np.int32)
    outs = []
    for mode in ("device", "host"):
        g = pkg.Group(engine, n_streams=S, max_len=512, kv_type=pkg.F16, base_layers=2, res_layers=1, cfm_steps=3, locdit_layers=2)
        g.set_kv_len(lens)
        g.fill_synthetic(seed=4)
        shapes = g.buffer_shapes()
        r = np.random.default_rng(6)
        host = {n: torch.from_numpy(r.standard_normal(s).astype(np.float32)).pin_memory() for n, s in shapes.items()}
        if mode == "device":
            t = {n: x.cuda() for n, x in host.items()}
            g.step(t, advance=True)
            engine.sync_status()
            outs.append((t["lm_out"].cpu().numpy(), t["dit_out"].cpu().numpy()))
        else:
            g.step_host(host, advance=True)
            outs.append((host["lm_out"].numpy().copy(), host["dit_out"].numpy().copy()))
        g.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])


def test_group_refuses_to_outgrow_capacity(engine, pkg):
    import torch
    g = pkg.Group(engine, n_streams=2, max_len=64, base_layers=1, res_layers=0, cfm_steps=0, locdit_layers=0)
    g.set_kv_len(np.array([64, 3], np.int32))
    shapes = g.buffer_shapes()
    t = {n: torch.zeros(s, device="cuda") for n, s in shapes.items()}
    with pytest.raises(pkg.VoxError) as e:
        g.step(t, advance=True)
    assert e.value.status_name == "INVALID_ARGUMENT"
    with pytest.raises(pkg.VoxError):
        g.set_kv_len(np.array([65, 3], np.int32))


# Distance of the engine's f16 / q8_0 cache from the reference's F32 cache (src/minicpm.cpp:182-183 stores F32 rows
# and attends over them unrounded), max-abs over the RMS of the output, on N(0,1) rows.  f16 storage stays inside
# the 2e-3 parity bound; q8_0 storage cannot (the reference's own q8_0 K/V type is as far from its F32 cache): what
# is asserted for it is the bound that the storage format itself implies, and the measured figure is printed.
STORAGE_BOUND = {"f16": 2e-3, "q8_0": 8e-2}


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
@pytest.mark.parametrize("n_kv", [1024, 4096])
def test_cache_storage_against_the_reference_f32_cache(kv, n_kv, engine, pkg, oracle, vo, capsys):
    """f32 K/V rows go in through vox_kv_append (all but the last) and through the decode launch's own store (the last,
    k_new / v_new); the result is compared with the reference's attention over the ORIGINAL f32 rows, i.e. with what
    MiniCPMKVCache's F32 storage would have given."""
    import torch
    rng = np.random.default_rng(n_kv + len(kv))
    k = rng.standard_normal((1, n_kv, HK, D)).astype(np.float32)
    v = rng.standard_normal((1, n_kv, HK, D)).astype(np.float32)
    q = rng.standard_normal((1, H, D)).astype(np.float32)
    cache = pkg.KVCache(engine, 1, 1, HK, n_kv, KV_TYPE[kv])
    cache.append(0, dev(k[:, :-1]), dev(v[:, :-1]), pos0=0)
    out = cache.decode(0, dev(q), dev(np.array([n_kv], np.int32)), n_kv, k_new=dev(k[:, -1]), v_new=dev(v[:, -1]))
    engine.sync_status()
    kf, vf = k[0].transpose(1, 0, 2)[None], v[0].transpose(1, 0, 2)[None]  # [1, HK, n_kv, D]
    ref = oracle.attn(q[0][None, :, None, :], np.ascontiguousarray(kf), np.ascontiguousarray(vf), kv_type=vo.F32, path=vo.PATH_ROW_F32)[0, 0]
    err = rel_err(out.cpu().numpy()[0], ref)
    with capsys.disabled():
        print(f"\n[storage deviation] {kv} cache, {n_kv} rows, against the reference's F32 cache: {err:.2e} of the output RMS")
    assert err < STORAGE_BOUND[kv]


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_two_caches_decode_on_two_streams_at_once(kv, engine, pkg):
    """Two caches of one engine (backbone and residual stacks, say) decoding on two CUDA streams with their own
    workspaces: the split-KV tickets belong to each cache's layer, so the launches may overlap on the GPU and give the
    same bits as when they run one after the other."""
    import torch
    lens = [4096, 300, 2048, 1500, 64, 3000]
    S = len(lens)
    gen = torch.Generator(device="cuda").manual_seed(3)
    caches, qs = [], []
    for i in range(2):
        c = pkg.KVCache(engine, 1, S, HK, 4096, KV_TYPE[kv])
        c.append(0, torch.randn((S, 4096, HK, D), device="cuda", generator=gen), torch.randn((S, 4096, HK, D), device="cuda", generator=gen), pos0=0)
        caches.append(c)
        qs.append(torch.randn((S, H, D), device="cuda", generator=gen))
    kv_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
    need = pkg.lib().vox_attn_decode_workspace_bytes(S, H, HK, 4096)
    ws = [torch.empty(need, dtype=torch.uint8, device="cuda") for _ in range(2)]
    serial = [torch.empty((S, H, D), device="cuda") for _ in range(2)]
    both = [torch.empty((S, H, D), device="cuda") for _ in range(2)]

    def call(i, dst, stream):
        a = caches[i]._decode_args(0, qs[i], kv_len, 4096, dst, 0.125, None, None, False, None, None)
        rc = pkg.lib().vox_attn_decode(engine.h, C.byref(a), C.c_void_p(ws[i].data_ptr()), need, C.c_void_p(stream.cuda_stream))
        assert rc == 0

    main = torch.cuda.current_stream()
    for i in range(2):
        call(i, serial[i], main)
        torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for rep in range(20):  # many pairs of launches: some of them overlap
        for i in range(2):
            streams[i].wait_stream(main)
            call(i, both[i], streams[i])
    for s in streams:
        s.synchronize()
    engine.sync_status()
    for i in range(2):
        assert torch.equal(both[i], serial[i])


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
@pytest.mark.parametrize("n_kv, planes", [(700, 1), (2049, 16), (64, 2)])
def test_single_token_forward_with_a_mask(kv, n_kv, planes, engine, oracle, vo):
    """n_q == 1 with an additive mask (third_party/ggml/src/ggml-cpu/ops.cpp:8233-8237): the split-KV decode kernel adds
    the mask row of each head's plane to its scores.  Random finite biases, 30 % of the keys hidden, one (batch, plane)
    that sees nothing at all (zeros), an odd number of keys."""
    B = 3
    rng = np.random.default_rng(n_kv + planes)
    q = rng.standard_normal((B, H, 1, D)).astype(np.float32)
    k = rng.standard_normal((B, HK, n_kv, D)).astype(np.float32)
    v = rng.standard_normal((B, HK, n_kv, D)).astype(np.float32)
    if kv == "q8_0":
        ks, vs = oracle.quantize_q8_0(k), oracle.quantize_q8_0(v)
    else:
        ks, vs = k.astype(np.float16), v.astype(np.float16)
    mask = np.where(rng.random((B, planes, 1, n_kv)) < 0.3, -np.inf, rng.integers(-8, 1, (B, planes, 1, n_kv)) / 4.0).astype(np.float16)
    mask[..., 0] = 0.0
    mask[1, planes - 1, 0, :] = -np.inf
    launches = engine.launches
    out = engine.forward(dev(q), dev(ks), dev(vs), dev(mask))
    engine.sync_status()
    assert engine.launches - launches == (2 if kv == "q8_0" else 1)  # decode kernel (after the block repack for q8_0), not the general one
    out = out.cpu().numpy()
    ref = oracle.attn(q, ks, vs, mask, kv_type=KV_TYPE[kv], path=vo.PATH_ROW_F32)
    assert rel_err(out, ref) < TOL[kv]
    heads_of_last_plane = [h for h in range(H) if h % planes == planes - 1]
    assert np.all(out[1, 0, heads_of_last_plane] == 0.0)


def test_replay_past_the_capacity_is_reported(engine, pkg):
    """A captured step replayed once more than the cache has rows for: the host check of vox_group_advance comes after
    the replay, so it is the decode launch that notices (the stream's length is beyond its rows), stores nothing for it
    and raises the status word; the engine reports DEVICE_STATE and keeps working."""
    import torch
    g = pkg.Group(engine, n_streams=2, max_len=128, kv_type=pkg.F16, base_layers=1, res_layers=0, locdit_layers=0, cfm_steps=0)
    g.set_kv_len(np.array([126, 5], np.int32))
    g.set_bound(128)
    bufs = {n: torch.randn(s, device="cuda") for n, s in g.buffer_shapes().items() if n.startswith("lm_")}
    side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    g.step(bufs, advance=False)  # attributes and descriptors outside the capture
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            g.step(bufs, advance=True, stream=side)
    for _ in range(2):  # rows 127 and 128: both fit
        graph.replay()
        g.advance(1)
    engine.sync_status()
    graph.replay()     # row 129 of 128
    with pytest.raises(pkg.VoxError) as e:
        engine.sync_status()
    assert e.value.status_name == "DEVICE_STATE"
    with pytest.raises(pkg.VoxError):
        g.advance(1)   # and the host bookkeeping refuses to follow
    engine.sync_status()
    g.close()


def test_cluster_mode_against_the_ticket_modes(engine, pkg, oracle, vo, monkeypatch):
    """Launches of few pairs give every (stream, kv head) a thread-block cluster whose CTAs hand their partial results to
    the first one through distributed shared memory; larger launches (and VOX_DECODE_CLUSTER=0) fold through the
    workspace with tickets.  The same streams through both: ragged lengths with an empty stream, a one-tile stream and
    streams that split seven ways, the arriving row stored by the launch, rotary embedding, decode repeated to catch a
    barrier that is not reusable.  Both agree with the oracle, and with each other to f32 rounding of the folds."""
    import torch
    lens = [4096, 1, 64, 0, 700, 2049, 4095, 257, 1024, 3000]
    S, cap = len(lens), 4096
    rng = np.random.default_rng(21)
    k = rng.standard_normal((S, HK, cap, D)).astype(np.float32)
    v = rng.standard_normal((S, HK, cap, D)).astype(np.float32)
    q = rng.standard_normal((S, H, D)).astype(np.float32)
    k_new = rng.standard_normal((S, HK, D)).astype(np.float32)
    v_new = rng.standard_normal((S, HK, D)).astype(np.float32)
    pos = np.maximum(np.array(lens, np.int32) - 1, 0)
    table = oracle.rope_table(pos, freq_base=10000.0, attn_factor=1.0)
    outs = []
    for cluster in ("1", "0"):
        monkeypatch.setenv("VOX_DECODE_CLUSTER", cluster)
        eng = pkg.Engine(0)
        cache = pkg.KVCache(eng, 1, S, HK, cap, pkg.F16)
        for s, n in enumerate(lens):
            if n > 1:
                cache.import_(0, s, oracle.kv_store(k[s, :, :n - 1], vo.F16), oracle.kv_store(v[s, :, :n - 1], vo.F16))
        kv_len = torch.tensor(lens, dtype=torch.int32, device="cuda")
        qd, kd, vd = (torch.from_numpy(x).cuda() for x in (q, k_new, v_new))
        for rep in range(3):  # the row is stored again at the same position: same bytes
            out = cache.decode(0, qd, kv_len, cap, k_new=kd, v_new=vd, rope_table=torch.from_numpy(table).cuda())
        eng.sync_status()
        outs.append(out.cpu().numpy())
        cache.close()
        eng.close()
    qr = oracle.rope(q, table)
    kr = oracle.rope(k_new, table)
    for s, n in enumerate(lens):
        if n == 0:
            assert not outs[0][s].any() and not outs[1][s].any()  # nothing visible: zeros (ops.cpp:8333)
            continue
        ks = np.concatenate([k[s, :, :n - 1], kr[s][:, None, :]], axis=1)
        vs = np.concatenate([v[s, :, :n - 1], v_new[s][:, None, :]], axis=1)
        ref = oracle.attn(qr[s][None, :, None, :], oracle.kv_store(ks, vo.F16)[None], oracle.kv_store(vs, vo.F16)[None],
                          kv_type=vo.F16, path=vo.PATH_ROW_F32)[0, 0]
        for o in outs:
            assert rel_err(o[s], ref) < TOL["f16"], (s, n)
    assert rel_err(outs[0], outs[1]) < 1e-5

