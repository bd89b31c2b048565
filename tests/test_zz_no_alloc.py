"""vox_attn_decode_static: decode attention for callers that cannot allocate device memory.

A real-time audio thread, a host that owns all device memory through its own arena, or a plugin
that only receives its input and output buffers has no workspace to hand to vox_attn_decode.  The
static variant keeps the split-KV partials in a 4 MiB array inside the library instead.  These
tests call it through the C ABI, twice in a row on the same array (the second call finds the first
call's partials still there and must not be disturbed by them), compare with vox_attn_decode and
with the CPU oracle, and check that the device's free memory does not move across a call.

The file sorts last on purpose: a run that stops at the first failure has then already exercised
every other test.  It also passes when run alone in a fresh process, where its first call is the
one that resolves the array's device address.
"""
import ctypes as C

import numpy as np
import pytest

from cases import KV_TYPE, rel_err

pytestmark = pytest.mark.gpu

H, HK, D = 16, 2, 64
SCRATCH = 4 << 20


def _setup(pkg, engine, lens, seed, kv="f16"):
    import torch
    S = len(lens)
    cap = -(-max(lens) // 64) * 64
    cache = pkg.KVCache(engine, 1, S, HK, cap, KV_TYPE[kv])
    group_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(seed)
    # rows through the engine's own append path: [streams, tokens, kv heads, 64]
    k = torch.randn((S, cap, HK, D), device="cuda", generator=gen)
    v = torch.randn((S, cap, HK, D), device="cuda", generator=gen)
    cache.append(0, k, v, pos0=0)
    q = torch.randn((S, H, D), device="cuda", generator=gen)
    return cache, q, group_lens, k, v


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_static_scratch_decode_matches_workspace_decode_twice(kv, engine, pkg):
    import torch
    # two different problems back to back: the second runs over whatever the first left in the array.  Both cut
    # pairs across CTAs (partials in the scratch), the second one 16 ways.
    problems = [([4096, 700, 2048, 129, 3000, 64, 1, 4000], 1), ([8192], 2)]
    for lens, seed in problems:
        cache, q, kv_len, _, _ = _setup(pkg, engine, lens, seed, kv)
        bound = max(lens)
        assert 0 < pkg.lib().vox_attn_decode_workspace_bytes(len(lens), H, HK, bound) <= SCRATCH
        want = cache.decode(0, q, kv_len, bound)
        engine.sync_status()
        for call in range(2):
            got = torch.full_like(want, float("nan"))
            free_before = torch.cuda.mem_get_info()[0]
            cache.decode_static(0, q, kv_len, bound, got)
            engine.sync_status()
            assert torch.cuda.mem_get_info()[0] == free_before  # the call allocated nothing on the device
            # same kernel, same cut of the work, same fold order: identical bits
            assert torch.equal(got, want), f"problem {lens[:2]}..., call {call}: max diff {(got - want).abs().max().item():.3e}"


def test_static_scratch_decode_matches_the_oracle(engine, pkg, oracle, vo):
    """One static call checked against the CPU restatement of the reference, not only against the other entry point."""
    lens = [3000, 129, 1024]
    cache, q, kv_len, k, v = _setup(pkg, engine, lens, 5)
    import torch
    got = torch.full((len(lens), H, D), float("nan"), device="cuda")
    cache.decode_static(0, q, kv_len, max(lens), got)
    engine.sync_status()
    got, qh = got.cpu().numpy(), q.cpu().numpy()
    for s, n in enumerate(lens):
        ks = oracle.kv_store(k[s, :n].permute(1, 0, 2).contiguous().cpu().numpy(), vo.F16)
        vs = oracle.kv_store(v[s, :n].permute(1, 0, 2).contiguous().cpu().numpy(), vo.F16)
        ref = oracle.attn(qh[s][None, :, None, :], ks[None], vs[None], kv_type=vo.F16, path=vo.PATH_ROW_F32)[0, 0]
        assert rel_err(got[s], ref) < 2e-3, f"stream {s}"


@pytest.mark.parametrize("kv", ["f16", "q8_0"])
def test_static_scratch_decode_stores_the_arriving_row(kv, engine, pkg):
    """The fused append (k_new / v_new) through the static entry: same cache rows and same result as vox_attn_decode."""
    import torch
    lens = [2000, 65, 1300]
    gen = torch.Generator(device="cuda").manual_seed(9)
    k_new = torch.randn((len(lens), HK, D), device="cuda", generator=gen)
    v_new = torch.randn((len(lens), HK, D), device="cuda", generator=gen)
    outs, rows = [], []
    for static in (False, True):
        cache, q, kv_len, _, _ = _setup(pkg, engine, lens, 7, kv)
        out = torch.full((len(lens), H, D), float("nan"), device="cuda")
        if static:
            cache.decode_static(0, q, kv_len, max(lens), out, k_new=k_new, v_new=v_new)
        else:
            cache.decode(0, q, kv_len, max(lens), dst=out, k_new=k_new, v_new=v_new)
        engine.sync_status()
        outs.append(out)
        rows.append([cache.export(0, s, n) for s, n in enumerate(lens)])
    assert torch.equal(outs[0], outs[1])
    for a, b in zip(rows[0], rows[1]):
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_static_scratch_holds_the_largest_launch(engine, pkg):
    """The scratch a launch needs is two partial slots per CTA of a one-wave grid, so it is bounded by the device and
    not by the problem: the array holds the largest launch this device can get (a larger device would be refused
    with WORKSPACE_TOO_SMALL)."""
    import torch
    for S, cap in [(512, 8192), (4096, 65536), (1, 64)]:
        assert pkg.lib().vox_attn_decode_workspace_bytes(S, H, HK, cap) <= SCRATCH
    S, cap = 512, 1024
    cache = pkg.KVCache(engine, 1, S, HK, cap, pkg.F16)
    q = torch.randn((S, H, D), device="cuda")
    kv_len = torch.full((S,), cap, dtype=torch.int32, device="cuda")
    got = torch.full((S, H, D), float("nan"), device="cuda")
    cache.decode_static(0, q, kv_len, cap, got)
    engine.sync_status()
    assert torch.all(got == 0)  # a cleared cache: V is zero everywhere


def test_static_scratch_bad_arguments(engine, pkg):
    """Refused on the host with INVALID_ARGUMENT, before anything is derived from the arguments or launched."""
    import torch
    assert pkg.lib().vox_attn_decode_static(None, None, None) == 1
    cache = pkg.KVCache(engine, 1, 4, HK, 256, pkg.F16)
    q = torch.zeros((4, H, D), device="cuda")
    kv_len = torch.full((4,), 256, dtype=torch.int32, device="cuda")
    dst = torch.zeros((4, H, D), device="cuda")
    before = engine.launches
    for field, value in [("n_streams", 0), ("n_streams", -1), ("n_streams", 5), ("n_heads", 0), ("n_heads", 15), ("kv_bound", -1),
                         ("kv_bound", 257), ("layer", 1)]:
        a = cache._decode_args(0, q, kv_len, 256, dst, 0.125, None, None, False, None, None)
        setattr(a, field, value)
        assert pkg.lib().vox_attn_decode_static(engine.h, C.byref(a), None) == 1, field
        assert pkg.lib().vox_attn_decode(engine.h, C.byref(a), None, 0, None) == 1, field
    assert engine.launches == before
