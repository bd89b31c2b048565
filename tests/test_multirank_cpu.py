"""The N > 1 path of the benchmark on CPU: two gloo ranks run the same stream assignment and the same
cross-rank plumbing (barrier, max and sum of scalars) that N GPUs run over NCCL.  Streams are the unit
of sharding; no rank ever needs another rank's data."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scaling, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import __graft_entry__ as entry
    import bench

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = entry.import_package()
    lens = bench.streams_of_rank(scaling, 256, rank, world, pkg.partition_streams)
    ranks = bench.Ranks(world, "cpu")
    ranks.barrier()
    total_streams = ranks.sum(float(len(lens)))
    total_rows = ranks.sum(float(lens.sum()))
    slowest = ranks.max(float(rank + 1) * 1.5)  # stands in for the per-rank elapsed time
    heaviest = ranks.max(float(lens.sum()))
    np.save(os.path.join(out_dir, f"lens_{scaling}_{rank}.npy"), lens)
    np.save(os.path.join(out_dir, f"agg_{scaling}_{rank}.npy"), np.array([total_streams, total_rows, slowest, heaviest]))
    dist.destroy_process_group()


@pytest.mark.parametrize("scaling", ["weak", "strong"])
def test_two_ranks_share_nothing_but_scalars(scaling, tmp_path):
    import torch.multiprocessing as mp

    sys.path.insert(0, ROOT)
    import bench

    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, scaling, str(tmp_path)), nprocs=world, join=True)
    lens = [np.load(tmp_path / f"lens_{scaling}_{r}.npy") for r in range(world)]
    agg = [np.load(tmp_path / f"agg_{scaling}_{r}.npy") for r in range(world)]
    assert np.array_equal(agg[0], agg[1])  # every rank sees the same reduced scalars
    total_streams, total_rows, slowest, heaviest = agg[0]
    assert slowest == 3.0  # max over ranks, not rank 0's own value
    assert total_rows == sum(x.sum() for x in lens) and heaviest == max(x.sum() for x in lens)
    if scaling == "weak":
        # every rank serves its own 256 streams: the same multiset of lengths (fixed work per GPU), its own order
        assert total_streams == 512 and all(len(x) == 256 for x in lens)
        assert not np.array_equal(lens[0], lens[1]) and np.array_equal(np.sort(lens[0]), np.sort(lens[1]))
        assert np.array_equal(np.sort(lens[0]), np.sort(bench.stream_lengths(256, 0)))
    else:
        # one population of 256 streams, split without loss or duplication and balanced by KV rows
        assert total_streams == 256
        everything = np.sort(np.concatenate(lens))
        assert np.array_equal(everything, np.sort(bench.stream_lengths(256, 0)))
        loads = np.array([x.sum() for x in lens], np.float64)
        assert loads.max() / loads.mean() < 1.01


def test_reference_arm_prints_one_contract_line(tmp_path):
    """`bench.py --impl reference` needs no GPU: one JSON line on stdout with the keys the benchmark contract names."""
    import json
    import subprocess

    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                        "--cpu-sample-streams", "2"], capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [x for x in r.stdout.splitlines() if x.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == "patches/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and "model" not in line["config"]
