"""vox_attn_decode_static: decode attention for callers that cannot allocate device memory.

A real-time audio thread, a host that owns all device memory through its own arena, or a plugin
that only receives its input and output buffers has no workspace to hand to vox_attn_decode.  The
static variant keeps the split-KV partials in a 16 MiB array inside the library instead.  These
tests call it through the C ABI, twice in a row on the same array (the second call finds the first
call's partials still there and must not be disturbed by them), and compare with vox_attn_decode.

The file sorts last on purpose: a run that stops at the first failure has then already exercised
every other test.  It also passes when run alone in a fresh process, where its first call is the
one that resolves the array's device address.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

H, HK, D = 16, 2, 64


def _setup(pkg, engine, lens, seed):
    import torch
    S = len(lens)
    cap = -(-max(lens) // 64) * 64
    cache = pkg.KVCache(engine, 1, S, HK, cap, pkg.F16)
    group_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(seed)
    # rows through the engine's own append path: [streams, tokens, kv heads, 64]
    k = torch.randn((S, cap, HK, D), device="cuda", generator=gen)
    v = torch.randn((S, cap, HK, D), device="cuda", generator=gen)
    cache.append(0, k, v, pos0=0)
    q = torch.randn((S, H, D), device="cuda", generator=gen)
    return cache, q, group_lens


def test_static_scratch_decode_matches_workspace_decode_twice(engine, pkg):
    import torch
    # two different problems back to back: the second runs over whatever the first left in the array
    problems = [([4096, 700, 2048, 129, 3000, 64, 1, 4000], 1), ([8192], 2)]
    for lens, seed in problems:
        cache, q, kv_len = _setup(pkg, engine, lens, seed)
        bound = max(lens)
        assert pkg.lib().vox_attn_decode_workspace_bytes(len(lens), H, HK, bound) > 0  # the split path, with partials
        want = cache.decode(0, q, kv_len, bound)
        engine.sync_status()
        for call in range(2):
            got = torch.full_like(want, float("nan"))
            cache.decode_static(0, q, kv_len, bound, got)
            engine.sync_status()
            # same kernels, same partial layout, same merge order: identical bits
            assert torch.equal(got, want), f"problem {lens[:2]}..., call {call}: max diff {(got - want).abs().max().item():.3e}"
            assert rel(got, want) < 2e-3


def rel(a, b):
    a, b = a.double().cpu().numpy(), b.double().cpu().numpy()
    return float(np.abs(a - b).max() / np.sqrt((b ** 2).mean()))


def test_static_scratch_refuses_oversized_calls(engine, pkg):
    import torch
    S, cap = 512, 8192  # 512 streams x 16 heads x 8 chunks x 264 B = 17.3 MB > 16 MiB
    need = pkg.lib().vox_attn_decode_workspace_bytes(S, H, HK, cap)
    assert need > (16 << 20)
    cache = pkg.KVCache(engine, 1, S, HK, cap, pkg.F16)
    q = torch.zeros((S, H, D), device="cuda")
    kv_len = torch.full((S,), cap, dtype=torch.int32, device="cuda")
    dst = torch.zeros((S, H, D), device="cuda")
    before = engine.launches
    with pytest.raises(pkg.VoxError) as e:
        cache.decode_static(0, q, kv_len, cap, dst)
    assert e.value.status_name == "WORKSPACE_TOO_SMALL"
    assert "built-in array" in str(e.value)
    assert engine.launches == before  # refused before anything was launched


def test_static_scratch_null_arguments(pkg):
    assert pkg.lib().vox_attn_decode_static(None, None, None) == 1
