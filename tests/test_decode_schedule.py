"""The three ways a decode launch deals its 64-row tiles out to CTAs, restated on the host from
voxcpm.cpp_b200/csrc/decode_attn.cu (cut_work_list and the cluster mode of decode_kernel) and checked for the properties
the kernel relies on: every tile of every (stream, kv head) pair belongs to exactly one CTA, a CTA's tiles are
consecutive, no CTA index beyond the grid is used, a pair is cut into no more pieces than the fold can take, and the
count of pieces a pair's ticket waits for (last CTA - first CTA + 1) is the number of CTAs that hold a part of it.
The GPU parity tests exercise the kernel itself; this file pins the arithmetic of the cuts, for lengths the GPU tests do
not enumerate (ragged, empty streams, one-tile streams, lengths on tile boundaries)."""
import numpy as np
import pytest

TILE = 64


def tiles_of(length):
    return (length + TILE - 1) // TILE


def ceil_div_small(x, r):
    """The division-free ceil(x / r) of the kernel: floor(((x + r) - 0.5) / r) in f32."""
    return int(np.floor(np.float32(np.float32(x + r) - np.float32(0.5)) / np.float32(r)))


def flat_cut(tiles, n_kv_heads, grid, run_min):
    """tiles[i] per stream -> list over CTAs of [(stream, kv head, first tile, count), ...] (the segments of its run)."""
    pairs = [(s, h, t) for s, t in enumerate(tiles) for h in range(n_kv_heads) if t > 0]
    total = sum(t for _, _, t in pairs)
    run = max(run_min, -(-total // grid))
    flat = [(s, h, i) for s, h, t in pairs for i in range(t)]
    ctas = []
    for b in range(grid):
        seg, f0, f1 = [], b * run, min(total, (b + 1) * run)
        for f in range(f0, f1):
            s, h, i = flat[f]
            if seg and seg[-1][0] == s and seg[-1][1] == h:
                seg[-1][3] += 1
            else:
                seg.append([s, h, i, 1])
        ctas.append([tuple(x) for x in seg])
    return ctas, run


def aligned_cut(tiles, n_kv_heads, grid, run_min, slack):
    """Every pair split on its own into ceil(t / r) nearly equal parts, for the first r from the flat run up to a
    quarter (at most `slack` tiles) above it for which the parts fit the grid; None when there is none."""
    total = sum(tiles) * n_kv_heads
    run = max(run_min, -(-total // grid))
    if run > 64 or total >= 1 << 20:
        return None
    for r in range(run, run + max(1, min(slack, run >> 2)) + 1):
        parts = [ceil_div_small(t, r) for t in tiles]
        if sum(parts) * n_kv_heads > grid:
            continue
        ctas = []
        for s, (t, n) in enumerate(zip(tiles, parts)):
            for h in range(n_kv_heads):
                for j in range(n):
                    start, end = (j * t) // n, ((j + 1) * t) // n
                    ctas.append([(s, h, start, end - start)])
        return ctas, r
    return None


def cluster_parts(tiles, n_kv_heads, cluster):
    """One cluster of `cluster` CTAs per pair; its first min(cluster, t / 4) CTAs (at least one) take nearly equal parts."""
    ctas = []
    for s, t in enumerate(tiles):
        for h in range(n_kv_heads):
            parts = max(1, min(cluster, t >> 2))
            for rank in range(cluster):
                if rank < parts and t > 0:
                    start = (rank * t) // parts
                    ctas.append([(s, h, start, ((rank + 1) * t) // parts - start)])
                else:
                    ctas.append([])
    return ctas


def check_cover(ctas, tiles, n_kv_heads):
    seen = {}
    for b, segs in enumerate(ctas):
        for s, h, start, count in segs:
            assert count >= 1
            for i in range(start, start + count):
                assert (s, h, i) not in seen, "a tile is given to two CTAs"
                seen[(s, h, i)] = b
    assert len(seen) == sum(tiles) * n_kv_heads, "a tile is given to no CTA"
    holders = {}
    for (s, h, _), b in seen.items():
        holders.setdefault((s, h), set()).add(b)
    return holders


def length_sets():
    rng = np.random.default_rng(7)
    yield [4096] * 32
    yield [2048] * 32
    yield [1, 64, 65, 0, 4096, 63, 128]
    yield list(rng.integers(128, 4097, 256))
    yield list(rng.integers(128, 4097, 32))
    yield list(rng.integers(0, 300, 40))
    yield [8192]
    yield [0, 0, 5]
    for _ in range(20):
        yield list(rng.integers(0, 9000, int(rng.integers(1, 80))))


@pytest.mark.parametrize("slots", [444, 592])
def test_flat_and_aligned_cuts_cover_every_tile_once(slots):
    for lens in length_sets():
        tiles = [tiles_of(int(n)) for n in lens]
        bound = max(1, max(tiles))
        run_min = max(4, -(-bound // 16))
        grid = max(1, min(-(-len(lens) * 2 * bound // run_min), slots))
        ctas, run = flat_cut(tiles, 2, grid, run_min)
        holders = check_cover(ctas, tiles, 2)
        for (s, h), who in holders.items():
            assert max(who) - min(who) + 1 == len(who)  # consecutive CTAs: the ticket count is last - first + 1
            assert len(who) <= 17 + 1                    # what run_min promises the fold
        assert all(len([x for x in segs if x[3] < tiles[x[0]]]) <= 2 for segs in ctas)  # at most two cut pairs per run
        got = aligned_cut(tiles, 2, grid, run_min, 4 if slots == 444 else 3)
        if got is not None:
            actas, r = got
            assert len(actas) <= grid
            check_cover(actas, tiles, 2)
            assert all(seg[0][3] <= r for seg in actas)
            assert r <= run + max(1, min(4, run >> 2))


def test_cluster_parts_cover_every_tile_once():
    for lens in length_sets():
        tiles = [tiles_of(int(n)) for n in lens]
        for cluster in (5, 6, 7):
            ctas = cluster_parts(tiles, 2, cluster)
            assert len(ctas) == len(lens) * 2 * cluster
            holders = check_cover(ctas, tiles, 2)
            for (s, h), who in holders.items():
                base = (s * 2 + h) * cluster
                assert who == set(range(base, base + len(who)))  # the first CTAs of the pair's own cluster
                assert len(who) == max(1, min(cluster, tiles[s] >> 2))
            # a part of a split pair has four tiles or more
            assert all(seg[0][3] >= 4 or seg[0][3] == tiles[seg[0][0]] for seg in ctas if seg)


def test_division_free_ceiling_is_exact():
    for r in range(1, 90):
        for x in list(range(0, 600)) + [1 << 14, (1 << 14) + 1, (1 << 19) - 1]:
            assert ceil_div_small(x, r) == -(-x // r), (x, r)
