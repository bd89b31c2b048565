"""The walk of the causal prefill kernel over its work, restated on the host from voxcpm.cpp_b200/csrc/prefill_attn.cu
(work_item, sub_tiles and the cut test of the softmax warps) and checked for what the kernel relies on: every key a row
may see lies in a 64-key score tile that is walked, no score tile is walked that no row of the item can see, a tile
that is not tested for the cut really is visible to every row in full, and the two softmax groups take alternate score
tiles of the CTA's whole sequence.  The GPU parity tests exercise the kernel itself; this file pins the arithmetic for
shapes they do not enumerate (offsets that are no multiple of 16, query counts that leave a partial item, key counts
that end inside a tile, every packing of heads)."""
import numpy as np
import pytest

TILE, KEYS, SUB = 128, 128, 64


def pack_of(n_heads, n_kv_heads):
    gqa = n_heads // n_kv_heads
    for pk in (8, 4, 2):
        if gqa % pk == 0:
            return pk
    return 1


def items_of(n_q, n_kv, n_heads, n_kv_heads, n_batch, causal_offset):
    """(qtile, head, batch, q0, n_tiles) in the order work_item numbers them (heaviest first)."""
    pack = pack_of(n_heads, n_kv_heads)
    tok = TILE // pack
    n_qtiles = -(-n_q // tok)
    n_hgroups = n_heads // pack
    out = []
    for idx in range(n_qtiles * n_hgroups * n_batch):
        per_tile = n_hgroups * n_batch
        rest = idx % per_tile
        qtile = n_qtiles - 1 - idx // per_tile
        q0 = qtile * tok
        last_tok = min(q0 + tok, n_q) - 1
        n_tiles = min(-(-n_kv // KEYS), (last_tok + causal_offset) // KEYS + 1)
        out.append((qtile, (rest % n_hgroups) * pack, rest // n_hgroups, q0, n_tiles))
    return out, pack, tok


def sub_tiles(q0, tok, n_q, n_kv, causal_offset, j):
    last_key = min(min(q0 + tok, n_q) - 1 + causal_offset, n_kv - 1)
    return 2 if last_key - j * KEYS >= SUB else 1


SHAPES = [
    # n_q, n_kv, heads, kv heads
    (512, 512, 16, 2), (200, 328, 16, 2), (130, 207, 16, 2), (1, 300, 16, 2), (300, 503, 16, 2), (600, 640, 16, 2),
    (77, 77, 16, 2), (129, 129, 8, 2), (64, 1000, 6, 2), (250, 250, 3, 1), (16, 4096, 16, 2), (333, 400, 4, 4),
]


@pytest.mark.parametrize("n_q, n_kv, n_heads, n_kv_heads", SHAPES)
def test_walk_covers_every_visible_key_and_nothing_else(n_q, n_kv, n_heads, n_kv_heads):
    off = n_kv - n_q
    items, pack, tok = items_of(n_q, n_kv, n_heads, n_kv_heads, 1, off)
    seen_rows = set()
    for qtile, head, batch, q0, n_tiles in items:
        uncut = min(q0 + off, n_kv - 1)
        cut_from = uncut // KEYS
        walked = []
        for j in range(n_tiles):
            for u in range(sub_tiles(q0, tok, n_q, n_kv, off, j)):
                walked.append(j * KEYS + SUB * u)
        assert walked == sorted(set(walked))
        last_tok = min(q0 + tok, n_q) - 1
        # no score tile beyond what the item's last row sees
        assert walked[-1] <= min(last_tok + off, n_kv - 1)
        for row in range(TILE):
            qpos = q0 + row // pack
            if qpos >= n_q:
                continue
            seen_rows.add((qpos, head + row % pack))
            limit = min(qpos + off, n_kv - 1)
            got = set()
            for k0 in walked:
                j = k0 // KEYS
                masked = j >= cut_from and k0 + SUB - 1 > uncut
                for i in range(SUB):
                    if masked:
                        if k0 + i <= limit:
                            got.add(k0 + i)
                    else:
                        assert k0 + i <= limit, "a tile that is not tested for the cut holds a key the row must not see"
                        got.add(k0 + i)
            assert got == set(range(limit + 1))
    assert len(seen_rows) == n_q * n_heads


def test_groups_take_alternate_score_tiles_of_a_cta():
    """Score tiles are numbered over all items of a CTA; group U % 2 takes tile U.  Both groups get within one tile of
    half of them, whatever the lengths of the items."""
    rng = np.random.default_rng(3)
    for _ in range(50):
        n_q = int(rng.integers(1, 700))
        n_kv = n_q + int(rng.integers(0, 300))
        items, pack, tok = items_of(n_q, n_kv, 16, 2, int(rng.integers(1, 4)), n_kv - n_q)
        grid = int(rng.integers(1, 149))
        for cta in range(min(grid, len(items))):
            U = 0
            mine = [0, 0]
            rnd = 0
            while True:
                idx = rnd * grid + (grid - 1 - cta if rnd & 1 else cta)
                if idx >= len(items):
                    break
                _, _, _, q0, n_tiles = items[idx]
                for j in range(n_tiles):
                    for _u in range(sub_tiles(q0, tok, n_q, n_kv, n_kv - n_q, j)):
                        mine[U & 1] += 1
                        U += 1
                rnd += 1
            assert abs(mine[0] - mine[1]) <= 1
