#!/usr/bin/env python
"""Benchmark of the attention engine on the multi-stream serving workload.

One step = the attention of one decode step for every synthesis stream a GPU serves:
24 backbone + 6 residual-LM layers of single-token attention over each stream's own KV cache
(append of the new row included), followed by one LocDiT CFG patch (10 CFM timesteps x 8 layers,
2 branches x 9 tokens).  256 streams per GPU with KV lengths drawn uniformly from [128, 4096].
Metric: patches per second (one patch per stream per step), whole job.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--kv-type f16]

N > 1 is launched by torch.distributed.run, one rank per GPU; ranks share nothing on the data path
(every stream lives on one GPU), so the only cross-rank traffic is the barrier and the max-reduce of
the timings.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, HK, D = 16, 2, 64
BASE_LAYERS, RES_LAYERS = 24, 6
DIT_LAYERS, DIT_SEQ, CFM_STEPS = 8, 9, 10
KV_LO, KV_HI = 128, 4096
WORKLOAD = ("multi-stream serving: {s} streams/GPU, ragged KV U[128,4096], 24+6 LM layers single-token attention "
            "(append included) + 1 LocDiT CFG patch (10 CFM steps x 8 layers x 2 branches x 9 tokens)")


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="engine", choices=["engine", "reference"])
    p.add_argument("--streams", type=int, default=256, help="streams per GPU (weak) or in total (strong)")
    p.add_argument("--kv-type", default="f16", choices=["f16", "q8_0"])
    p.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    p.add_argument("--cpu-sample-streams", type=int, default=24)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--rope", action="store_true",
                   help="hand Q and the new K rows over before the rotary embedding: one cos/sin table per step, rotation inside the decode launches")
    p.add_argument("--prefill-shapes", default="512x1,512x8", help="LxB list for --workload prefill")
    p.add_argument("--prefill-kv", default="f16", choices=["f16", "q8_0"], help="K/V operand type for --workload prefill")
    p.add_argument("--prefill-mask", action="store_true",
                   help="--workload prefill through vox_attn_forward with the causal mask as a tensor, as the reference's call site passes it")
    p.add_argument("--workload", default="serving", choices=["serving", "prefill", "decode_sweep", "decode_c1"],
                   help="serving = the headline line; the others time one more configuration each on one GPU")
    return p.parse_args()


def stream_lengths(n, rank=0):
    return np.random.default_rng(12345 + rank).integers(KV_LO, KV_HI + 1, n).astype(np.int32)


def bind_to_gpu_numa_node(torch, device_index):
    """Keep this process (and the pinned host buffers it allocates afterwards) on the NUMA node of its GPU: with one
    process per GPU the host-buffer entry point otherwise sends half of its traffic across the socket link.  Returns
    the node, or None when the platform does not say (containers often hide it): then nothing is changed."""
    try:
        props = torch.cuda.get_device_properties(device_index)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        node = int(open(base + "/numa_node").read().strip())
        cpus = open(base + "/local_cpulist").read().strip()
        if node < 0 or not cpus:
            return None
        ids = set()
        for part in cpus.split(","):
            lo, _, hi = part.partition("-")
            ids.update(range(int(lo), int(hi or lo) + 1))
        allowed = ids & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def streams_of_rank(scaling, n_streams, rank, world, partition):
    """KV lengths of the streams one rank serves.  weak: every rank serves `n_streams` streams with the same
    multiset of ragged lengths (the per-GPU work is what is held fixed), in an order of its own; strong: one
    draw of `n_streams` is split over the ranks by `partition` (longest-processing-time on KV length).
    Streams never move between ranks and nothing is exchanged on the data path."""
    if scaling == "weak":
        return np.random.default_rng(777 + rank).permutation(stream_lengths(n_streams, 0))
    all_lens = stream_lengths(n_streams, 0)
    owner = partition(all_lens, world)
    return all_lens[owner == rank]


class Ranks:
    """The only cross-rank traffic of the benchmark: a barrier and max / sum of a scalar (timings, stream
    counts).  Works on any initialised process group (NCCL on GPUs, gloo in the CPU tests)."""

    def __init__(self, world, device):
        self.world, self.device = world, device

    def _reduce(self, x, op):
        if self.world == 1:
            return x
        import torch
        import torch.distributed as dist
        t = torch.tensor([x], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()

    def max(self, x):
        import torch.distributed as dist
        return self._reduce(x, dist.ReduceOp.MAX)

    def sum(self, x):
        import torch.distributed as dist
        return self._reduce(x, dist.ReduceOp.SUM)


def lm_bytes_per_layer(lens, kv_type):
    """Algorithmic bytes of one LM layer over all streams: K and V rows once, Q in, output out."""
    row = 512.0 if kv_type == "f16" else 272.0
    return float(np.sum(row * lens.astype(np.float64) + 8192.0))


# ------------------------------------------------------------------ clocks

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(s) > 2 + i and s[2 + i].lower() == "active" for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ------------------------------------------------------------------ reference arm / CPU baseline

def cpu_reference_throughput(n_streams, iters, kv_type):
    """patches/s of the reference's own ggml CPU attention (unmodified, as shipped: native K/V type,
    one graph of 30 single-token nodes per stream and one graph of 80 LocDiT nodes per patch, streams
    served one after another as the reference server does) on a sample of the workload."""
    from oracle import voxoracle as vo
    if vo.RefGgml.available():
        ref, kind = vo.RefGgml(), "reference"
    else:
        ref, kind = None, "port"
    oracle = vo.Oracle()
    cores = os.cpu_count() or 1
    lens = stream_lengths(max(n_streams, 1))[:n_streams]
    rng = np.random.default_rng(7)
    L = BASE_LAYERS + RES_LAYERS
    kvt = vo.F16 if kv_type == "f16" else vo.Q8_0
    work = []
    for n in lens:
        q = rng.standard_normal((L, 1, H, 1, D)).astype(np.float32)
        k = rng.standard_normal((L, 1, HK, int(n), D)).astype(np.float32)
        v = rng.standard_normal((L, 1, HK, int(n), D)).astype(np.float32)
        ks, vs = (k.astype(np.float16), v.astype(np.float16)) if kv_type == "f16" else (oracle.quantize_q8_0(k), oracle.quantize_q8_0(v))
        work.append((q, ks, vs))
    n_dit = CFM_STEPS * DIT_LAYERS
    dq = rng.standard_normal((n_dit, 2, H, DIT_SEQ, D)).astype(np.float32)
    dk = rng.standard_normal((n_dit, 2, HK, DIT_SEQ, D)).astype(np.float32)
    dv = rng.standard_normal((n_dit, 2, HK, DIT_SEQ, D)).astype(np.float32)

    def one_pass():
        t0 = time.perf_counter()
        for q, ks, vs in work:
            if ref is not None:
                ref.attn(q, ks, vs, None, kv_type=kvt, n_threads=cores, n_layers=L)
                ref.attn(dq, dk, dv, None, kv_type=vo.F32, n_threads=cores, n_layers=n_dit)
            else:
                for l in range(L):
                    oracle.attn(q[l], ks[l], vs[l], kv_type=kvt, path=vo.PATH_AUTO, n_chunks=cores)
                for l in range(n_dit):
                    oracle.attn(dq[l], dk[l], dv[l], kv_type=vo.F32, path=vo.PATH_ROW)
        return time.perf_counter() - t0

    one_pass()
    times = [one_pass() for _ in range(max(iters, 1))]
    med = statistics.median(times)
    return {"value": n_streams / med, "unit": "patches/s", "cores": cores if ref is not None else 1, "kind": kind,
            "sample": f"{n_streams} streams of the workload (KV lengths {int(lens.min())}..{int(lens.max())}), "
                      f"{L} decode layers + {n_dit} LocDiT calls each, median of {len(times)} passes, "
                      f"ggml CPU backend {'(' + ref.isa + ', OpenMP)' if ref is not None else 'restated in C'}",
            "ms_per_stream": med / n_streams * 1e3}


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    steps = max(args.steps, 1)
    r = cpu_reference_throughput(args.cpu_sample_streams, min(steps, 5), args.kv_type)
    line = {"impl": "reference", "metric": "patches/s", "value": r["value"], "unit": "patches/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_stream"] * args.cpu_sample_streams,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD.format(s=args.streams), "kv_type": args.kv_type,
                       "note": "host cores only; the reference serves streams one at a time"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "patches/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------ other configurations (one GPU)

def q8_0_blocks(x):
    """ggml q8_0 blocks of a device tensor whose last dimension is a multiple of 32: per block an f16 scale
    d = amax / 127 and 32 int8 values round(x / d), 34 bytes (synthetic benchmark input only)."""
    import torch
    blocks = x.reshape(*x.shape[:-1], x.shape[-1] // 32, 32)
    d = blocks.abs().amax(dim=-1, keepdim=True) / 127.0
    qv = torch.where(d > 0, blocks / torch.where(d > 0, d, torch.ones_like(d)), torch.zeros_like(blocks)).round().clamp(-127, 127).to(torch.int8)
    packed = torch.cat([d.half().view(torch.uint8), qv.view(torch.uint8)], dim=-1)
    return packed.reshape(*x.shape[:-1], x.shape[-1] // 32 * 34).contiguous()

def aux_workload(args, pkg, torch):
    """Times the other configurations: causal prefill (512 tokens, 24 layers, batch 1 and 8), the long-form decode
    sweep (KV 1k-8k, batch 1 and 32, f16 and q8_0, 24+6 layers) and single-stream decode at KV 256 (24 layers).
    Launch sequences are issued from C (stream groups) or replayed from a CUDA graph, so host launch cost is not
    what is measured.  L2 is scrubbed between repetitions for the "cold" figures."""
    eng = pkg.Engine(torch.cuda.current_device())
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    hbm, tens = float(peaks.get("hbm_gbs", 6650.0)), float(peaks.get("bf16_tflops", 1590.0))
    stream = torch.cuda.current_stream()
    scrub = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")  # > 126 MB L2

    def timed(fn, reps, cold):
        fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            if cold:
                scrub.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / reps  # ms

    out = {"workload": args.workload, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tens}, "results": []}
    gen = torch.Generator(device="cuda").manual_seed(0)
    if args.workload == "prefill":
        layers = BASE_LAYERS
        for L, B in [(int(x.split("x")[0]), int(x.split("x")[1])) for x in args.prefill_shapes.split(",")]:
            q = torch.randn((layers, B, H, L, D), device="cuda", generator=gen).half().float()
            k = torch.randn((layers, B, HK, L, D), device="cuda", generator=gen).half()
            v = torch.randn((layers, B, HK, L, D), device="cuda", generator=gen).half()
            if args.prefill_kv == "q8_0":
                k, v = q8_0_blocks(k.float()), q8_0_blocks(v.float())
            o = torch.empty((layers, B, L, H, D), device="cuda")
            if args.prefill_mask:
                hidden = torch.arange(L, device="cuda")[None, :] > torch.arange(L, device="cuda")[:, None]
                mask = torch.zeros((1, 1, L, L), device="cuda", dtype=torch.float16).masked_fill(hidden, float("-inf"))
                call = lambda l: eng.forward(q[l], k[l], v[l], mask, dst=o[l])
            else:
                call = lambda l: eng.prefill(q[l], k[l], v[l], dst=o[l])
            for l in range(layers):  # warm-up outside capture (attribute set-up, descriptors)
                call(l)
            eng.sync_status()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for l in range(layers):
                    call(l)
            ms = timed(graph.replay, 20, cold=False)
            flops = layers * B * 4.0 * H * D * L * (L + 1) / 2
            out["results"].append({"config": f"prefill L={L} B={B} x {layers} layers, {args.prefill_kv} K/V" + (", mask tensor" if args.prefill_mask else ""), "ms": ms, "us_per_layer": ms * 1e3 / layers,
                                   "tflops_causal_useful": flops / (ms * 1e-3) / 1e12,
                                   "frac_of_measured_bf16_peak": flops / (ms * 1e-3) / 1e12 / tens})
    else:
        combos = [(256, 1, "f16", 24, 0)] if args.workload == "decode_c1" else \
            [(L, B, t, BASE_LAYERS, RES_LAYERS) for t in ("f16", "q8_0") for B in (1, 32) for L in (1024, 2048, 4096, 8192)]
        for L, B, t, nb, nr in combos:
            g = pkg.Group(eng, n_streams=B, max_len=L, kv_type=pkg.F16 if t == "f16" else pkg.Q8_0, base_layers=nb, res_layers=nr,
                          n_heads=H, n_kv_heads=HK, locdit_layers=0, cfm_steps=0)
            lens = np.full(B, L, np.int32)
            g.set_kv_len(lens)
            g.fill_synthetic(seed=L + B)
            shapes = g.buffer_shapes()
            bufs = {n: torch.randn(s, device="cuda", generator=gen) for n, s in shapes.items() if n.startswith("lm_")}
            step = lambda: g.step(bufs, advance=False)
            nbytes = (nb + nr) * lm_bytes_per_layer(lens, t)
            warm, cold = timed(step, 20, cold=False), timed(step, 10, cold=True)
            eng.sync_status()
            # the same launch sequence captured once and replayed (vox_group_set_bound makes it position-independent):
            # for a single stream the host's launch rate, not the GPU, bounds a step issued call by call
            graph_us = None
            if B == 1:
                side = torch.cuda.Stream()
                graph = torch.cuda.CUDAGraph()
                g.set_bound(L)
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph, stream=side):
                        g.step(bufs, advance=False, stream=side)
                graph_us = timed(graph.replay, 20, cold=False) * 1e3 / (nb + nr)
                eng.sync_status()
            out["results"].append({"config": f"decode kv={L} B={B} {t} x {nb + nr} layers", "bytes": nbytes,
                                   "graph_replay_us_per_layer": graph_us,
                                   "warm_us_per_layer": warm * 1e3 / (nb + nr), "cold_us_per_layer": cold * 1e3 / (nb + nr),
                                   "warm_gb_s": nbytes / (warm * 1e-3) / 1e9, "cold_gb_s": nbytes / (cold * 1e-3) / 1e9,
                                   "cold_frac_of_measured_hbm": nbytes / (cold * 1e-3) / 1e9 / hbm,
                                   "cold_frac_of_8000": nbytes / (cold * 1e-3) / 1e9 / 8000.0})
            g.close()
    return out


# ------------------------------------------------------------------ engine arm

def main():
    args = parse()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.import_package()

    torch.cuda.set_device(local)
    numa_node = bind_to_gpu_numa_node(torch, local) if world > 1 else None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ranks = Ranks(world, "cuda")

    def barrier():
        ranks.barrier()
        torch.cuda.synchronize()

    max_over_ranks, sum_over_ranks = ranks.max, ranks.sum

    if args.workload != "serving":
        if rank == 0:
            print(json.dumps(aux_workload(args, pkg, torch)))
        return

    lens = streams_of_rank(args.scaling, args.streams, rank, world, pkg.partition_streams)
    S = len(lens)
    total_steps = args.warmup + args.steps
    max_len = ((KV_HI + 2 * (total_steps + 8) + 63) // 64) * 64
    kv_type = pkg.F16 if args.kv_type == "f16" else pkg.Q8_0

    eng = pkg.Engine(local)
    group = pkg.Group(eng, n_streams=S, max_len=max_len, kv_type=kv_type, base_layers=BASE_LAYERS, res_layers=RES_LAYERS,
                      n_heads=H, n_kv_heads=HK, locdit_layers=DIT_LAYERS, locdit_seq=DIT_SEQ, cfm_steps=CFM_STEPS)
    group.set_kv_len(lens)
    group.fill_synthetic(seed=rank)
    if args.rope:  # llama.rope.freq_base of the reference's GGUF defaults, per-frequency factors as LongRoPE ships them
        group.set_rope(freq_base=10000.0, attn_factor=1.0, freq_factors=np.linspace(1.0, 4.0, 32, dtype=np.float32))
    shapes = group.buffer_shapes()
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    dev_t = {n: (torch.empty(s, device="cuda") if n.endswith("out") else torch.randn(s, device="cuda", generator=gen))
             for n, s in shapes.items()}
    stream = torch.cuda.current_stream()

    # ---- device-resident throughput: K steps, CUDA events, barrier + sync on both sides
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()
    for _ in range(args.warmup):
        group.step(dev_t, advance=True)
    eng.sync_status()
    barrier()
    l0 = eng.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        group.step(dev_t, advance=True)
    e1.record(stream)
    barrier()
    eng.sync_status()
    launches = eng.launches - l0
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = ms_total / args.steps
    total_streams = sum_over_ranks(float(S))
    value = total_streams / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel (split-KV decode): mean duration of a launch by CUDA events on the
    #      launching stream over 150 back-to-back launches (gaps between launches included), lengths as they now stand
    cur = group.kv_len()
    lm_only = {n: x for n, x in dev_t.items() if n.startswith("lm_")}
    n_lm = BASE_LAYERS + RES_LAYERS
    reps = 5
    group.step(lm_only, advance=False)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(reps):
        group.step(lm_only, advance=False)  # 30 decode launches issued back to back from C, lengths fixed
    b.record(stream)
    torch.cuda.synchronize()
    dec_ms = a.elapsed_time(b) / (reps * n_lm)
    layer_bytes = lm_bytes_per_layer(cur, args.kv_type)
    achieved = layer_bytes / (dec_ms * 1e-3) / 1e9
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    roofline = {"bound": "hbm", "kernel": f"decode_kernel<{args.kv_type}> (split-KV, partials folded by the last CTA of each stream and kv head)",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                # DRAM bytes per launch: ncu captures of the 256-stream launch read 1.041x (f16) / 1.043x (q8_0) the
                # algorithmic bytes (the ncu summaries kept under profiles/); traffic grows with the streams' KV bytes
                "traffic": layer_bytes * (1.041 if args.kv_type == "f16" else 1.043),
                "traffic_source": "ncu capture of the 256-stream launch (DRAM bytes / algorithmic bytes), applied to this launch's algorithmic bytes",
                "peak_source": peak_src,
                "us_per_launch": dec_ms * 1e3, "algorithmic_bytes_per_launch": layer_bytes,
                "frac_of_nominal_8000": achieved / 8000.0}

    # ---- LocDiT: latency of one patch for one stream (10 launches), and launches per CFM timestep
    one = pkg.Group(eng, n_streams=1, max_len=64, kv_type=kv_type, base_layers=0, res_layers=0, n_heads=H, n_kv_heads=HK,
                    locdit_layers=DIT_LAYERS, locdit_seq=DIT_SEQ, cfm_steps=CFM_STEPS)
    one_t = {n: torch.randn(s, device="cuda", generator=gen) for n, s in one.buffer_shapes().items()}
    for _ in range(3):
        one.step(one_t, advance=False)
    torch.cuda.synchronize()
    lb = eng.launches
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    a.record(stream)
    for _ in range(reps):
        one.step(one_t, advance=False)  # the 10 CFM launches are issued back to back from C
    b.record(stream)
    torch.cuda.synchronize()
    issued_us = a.elapsed_time(b) * 1e3 / reps
    launches_per_step = (eng.launches - lb) / (reps * CFM_STEPS)
    # the same ten launches captured once and replayed: what a server that holds the step as a graph sees (issued
    # call by call, a single stream is bound by the host's launch rate, which differs from box to box)
    side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            one.step(one_t, advance=False, stream=side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    a.record(stream)
    for _ in range(reps):
        graph.replay()
    b.record(stream)
    torch.cuda.synchronize()
    replayed_us = a.elapsed_time(b) * 1e3 / reps
    one.close()
    locdit = {"us_per_patch_single_stream": issued_us, "us_per_patch_single_stream_graph_replay": replayed_us,
              "launches_per_cfm_step": launches_per_step}

    # ---- end to end through the host-buffer entry point: pinned host inputs, H2D + launches + D2H per step
    e2e = None
    if not args.no_e2e:
        host_t = {n: torch.empty(s, dtype=torch.float32).pin_memory() for n, s in shapes.items()}
        for n, x in host_t.items():
            if not n.endswith("out"):
                x.copy_(dev_t[n])
        # bytes copied per step by all ranks together (each rank feeds its own GPU over its own PCIe link)
        h2d = sum_over_ranks(float(group.step_bytes(0) + group.step_bytes(2)))
        d2h = sum_over_ranks(float(group.step_bytes(1) + group.step_bytes(3)))
        e2e_steps = max(2, min(args.steps, 5))
        group.step_host(host_t, advance=True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            group.step_host(host_t, advance=True)
        barrier()
        dt = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": total_streams * e2e_steps / dt, "unit": "patches/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": dt / e2e_steps * 1e3, "steps": e2e_steps}

    # clocks were sampled from the first warm-up step to the last end-to-end step (GPU under load throughout)
    clock_info = clocks.stop() if rank == 0 else None

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            r = cpu_reference_throughput(args.cpu_sample_streams, 3, args.kv_type)
            cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as ex:  # the baseline is a report, it must not take the bench line down
            cpu = {"value": None, "unit": "patches/s", "cores": 0, "kind": "unavailable", "sample": repr(ex)}

    if rank == 0:
        line = {"metric": "patches/s", "value": value, "unit": "patches/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD.format(s=args.streams), "streams_total": int(total_streams), "kv_type": args.kv_type,
                           "l2": "inputs larger than L2 (KV read per step >> 126 MB)", "append": "included",
                           "host_numa_node": numa_node,
                           "placement": "weak: every GPU serves the same multiset of ragged lengths" if args.scaling == "weak"
                           else "strong: one population split over the GPUs by KV rows (longest-processing-time)",
                           "rope": "rotary embedding of Q and the new K rows inside the decode launches" if args.rope else "applied by the caller",
                           "arithmetic": "f16 K/V (or q8_0), f32 Q and output, f16 tensor-core products with hi+lo split of Q and P, "
                                         "f32 accumulation; LocDiT f32 throughout"},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clock_info,
                "locdit": locdit,
                "decode": {"gb_per_s": achieved, "pct_of_measured_peak": 100 * achieved / peak, "pct_of_8000": 100 * achieved / 8000}}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
