#!/usr/bin/env python
"""Benchmark of the attention engine on the multi-stream serving workload.

One step = the attention of one decode step for every synthesis stream of the population:
24 backbone + 6 residual-LM layers of single-token attention over each stream's own KV cache
(append of the new row included), followed by one LocDiT CFG patch (10 CFM timesteps x 8 layers,
2 branches x 9 tokens).  The population is 256 streams with KV lengths drawn uniformly from
[128, 4096]; on N GPUs it is PARTITIONED (longest-processing-time on KV rows, vox_partition_streams),
every stream living on one GPU, nothing exchanged.  Metric: patches per second (one patch per stream
per step), whole job.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--kv-type f16]

N > 1 is launched by torch.distributed.run, one rank per GPU; the only cross-rank traffic is the barrier
and a few scalar reductions of timings.  Prints ONE JSON line on rank 0.  At N = 1 the line also carries
the other configured shapes (prefill, the q8_0 serving step, the long-form decode sweep, single-stream
decode), each beside the reference's ggml CPU attention timed on this machine's cores in the same run.
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
WORKLOAD = ("multi-stream serving: {s} streams in total, ragged KV U[128,4096], 24+6 LM layers single-token attention "
            "(append included) + 1 LocDiT CFG patch (10 CFM steps x 8 layers x 2 branches x 9 tokens), "
            "streams partitioned over the GPUs, no collective")


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=40)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="engine", choices=["engine", "reference"])
    p.add_argument("--streams", type=int, default=256, help="streams of the population (in total; per GPU for --scaling weak)")
    p.add_argument("--kv-type", default="f16", choices=["f16", "q8_0"])
    p.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                   help="strong: one population partitioned over the GPUs (the configured workload); weak: a population per GPU")
    p.add_argument("--cpu-sample-streams", type=int, default=24)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-extras", action="store_true", help="leave out the other configured shapes (N = 1 prints them by default)")
    p.add_argument("--rope", action="store_true",
                   help="hand Q and the new K rows over before the rotary embedding: one cos/sin table per step, rotation inside the decode launches")
    p.add_argument("--cfm-zero-init", type=int, default=0,
                   help="CFM timesteps at the start of a patch that evaluate no network (the reference's cfg-zero-star: 1 of 10)")
    p.add_argument("--prefill-shapes", default="512x1,512x8", help="LxB list for --workload prefill")
    p.add_argument("--prefill-kv", default="f16", choices=["f16", "q8_0"], help="K/V operand type for --workload prefill")
    p.add_argument("--prefill-mask", action="store_true",
                   help="--workload prefill through vox_attn_forward with the causal mask as a tensor, as the reference's call site passes it")
    p.add_argument("--workload", default="serving", choices=["serving", "prefill", "decode_sweep", "decode_c1", "decode_profile", "locdit_profile", "projection", "layer_linears"],
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
    """KV lengths of the streams one rank serves.  strong: one draw of `n_streams` is split over the ranks by
    `partition` (longest-processing-time on KV length); weak: every rank serves `n_streams` streams with the same
    multiset of ragged lengths (the per-GPU work is what is held fixed), in an order of its own.
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


def workload_config(args, streams_total):
    """The `config` of the line: what is measured, in the same words for the engine arm and the reference arm."""
    return {"workload": WORKLOAD.format(s=args.streams if args.scaling == "strong" else streams_total),
            "streams_total": int(streams_total), "kv_type": args.kv_type, "append": "included",
            "l2": "inputs larger than L2 (KV read per step >> 126 MB)",
            "cfm_evaluations_per_patch": CFM_STEPS - args.cfm_zero_init,
            "placement": "one population split over the GPUs by KV rows (longest-processing-time)" if args.scaling == "strong"
            else "weak: every GPU serves its own population with the same multiset of ragged lengths"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback"


def dram_traffic_ratio(kernel):
    """DRAM bytes per algorithmic byte of a kernel, from the ncu capture recorded in the package's data file
    (None when the file has no entry: the bench line then carries a null traffic)."""
    try:
        return float(json.load(open(os.path.join(ROOT, "voxcpm.cpp_b200", "dram_traffic.json")))[kernel]["dram_bytes_per_algorithmic_byte"])
    except Exception:
        return None


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


# ------------------------------------------------------------------ reference arm / CPU baselines

def cpu_checker():
    """The reference's own ggml CPU backend when it was built for this machine (kind "reference"), else the C
    restatement (kind "port").  Both are test infrastructure: they are timed here, never used by the engine."""
    from oracle import voxoracle as vo
    ref = vo.RefGgml() if vo.RefGgml.available() else None
    return vo, ref, vo.Oracle()


def sample_of_population(n_streams, population=256):
    """`n_streams` KV lengths of the population, every k-th of the sorted draw: the sample's mean length is the
    population's (the first draws of the generator happen to be long ones)."""
    lens = np.sort(stream_lengths(population))
    idx = ((np.arange(n_streams) + 0.5) * population / n_streams).astype(int)
    return lens[idx]


def cpu_reference_throughput(n_streams, passes, warmup, kv_type, cfm_evals=CFM_STEPS):
    """patches/s of the reference's own ggml CPU attention (unmodified, as shipped: native K/V type,
    one graph of 30 single-token nodes per stream and one graph of 80 LocDiT nodes per patch, streams
    served one after another as the reference server does) on a sample of the workload."""
    vo, ref, oracle = cpu_checker()
    kind = "reference" if ref is not None else "port"
    cores = os.cpu_count() or 1
    lens = sample_of_population(n_streams)
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
    n_dit = cfm_evals * DIT_LAYERS
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

    for _ in range(max(warmup, 1)):
        one_pass()
    times = [one_pass() for _ in range(max(passes, 1))]
    mean = sum(times) / len(times)
    return {"value": n_streams / mean, "unit": "patches/s", "cores": cores if ref is not None else 1, "kind": kind,
            "sample": f"{n_streams} streams of the population (every {256 // n_streams}th of the sorted KV lengths, mean {lens.mean():.0f} rows "
                      f"against {stream_lengths(256).mean():.0f}), {L} decode layers + {n_dit} LocDiT calls each, mean of {len(times)} passes, "
                      f"ggml CPU backend {'(' + ref.isa + ', OpenMP, ' + str(cores) + ' threads)' if ref is not None else 'restated in C, 1 thread'}",
            "ms_per_pass": mean * 1e3, "passes": len(times)}


def run_reference_arm(args, rank, world):
    """The reference's own CPU implementation of the path on this machine's cores: K timed passes (after W untimed ones)
    over a bounded sample of the streams.  Rank 0 alone runs it."""
    if rank != 0:
        return
    r = cpu_reference_throughput(args.cpu_sample_streams, max(args.steps, 1), max(args.warmup, 1), args.kv_type,
                                 CFM_STEPS - args.cfm_zero_init)
    line = {"impl": "reference", "metric": "patches/s", "value": r["value"], "unit": "patches/s", "n_gpus": args.gpus,
            "steps": r["passes"], "warmup": max(args.warmup, 1), "ms_per_step": r["ms_per_pass"],
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": args.kv_type, "data": "synthetic",
            "config": workload_config(args, args.streams),
            "notes": "host cores only; the reference serves streams one at a time; a step here is one pass over the sample",
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "patches/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def cpu_attention_us(B, n_q, n_kv, kv, causal, n_layers, iters=3):
    """Microseconds per layer of the reference's ggml CPU attention on this machine (all cores, OpenMP) for one of the
    configured shapes, on `n_layers` independent layers in one graph, median of `iters` runs after one warm-up."""
    vo, ref, oracle = cpu_checker()
    if ref is None:
        return None
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(B * 131 + n_kv)
    q = rng.standard_normal((n_layers, B, H, n_q, D)).astype(np.float32)
    k = rng.standard_normal((n_layers, B, HK, n_kv, D)).astype(np.float32)
    v = rng.standard_normal((n_layers, B, HK, n_kv, D)).astype(np.float32)
    if kv == "f16":
        q = q.astype(np.float16).astype(np.float32) if n_q > 1 else q
        ks, vs, kvt = k.astype(np.float16), v.astype(np.float16), vo.F16
    elif kv == "q8_0":
        ks, vs, kvt = oracle.quantize_q8_0(k), oracle.quantize_q8_0(v), vo.Q8_0
    else:
        ks, vs, kvt = k, v, vo.F32
    mask = oracle.causal_mask(np.arange(n_kv - n_q, n_kv), n_kv)[None, None] if causal else None
    _, ms = ref.attn(q, ks, vs, mask, kv_type=kvt, n_threads=cores, n_layers=n_layers, iters=iters + 1, return_ms=True)
    return {"us_per_layer": float(np.median(ms[1:])) * 1e3 / n_layers, "cores": cores, "kind": "reference",
            "sample": f"{n_layers} layers in one graph, median of {iters} runs, ggml CPU backend ({ref.isa}, OpenMP, {cores} threads)"}


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


class Timer:
    """CUDA-event timing on the current stream, optionally with L2 scrubbed between repetitions."""

    def __init__(self, torch):
        self.torch = torch
        self.stream = torch.cuda.current_stream()
        self.scrub = None

    def ms(self, fn, reps, cold=False):
        torch = self.torch
        if cold and self.scrub is None:
            self.scrub = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")  # > 126 MB of L2
        fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            if cold:
                self.scrub.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(self.stream)
            fn()
            b.record(self.stream)
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / reps


def time_prefill(pkg, torch, eng, timer, shapes, kv="f16", with_mask=False, cpu=False):
    """Causal prefill, 24 layers replayed from a CUDA graph: us per layer, causal-useful TFLOP/s, fraction of the
    measured dense bf16 peak (burst figure: the kernel is timed alone)."""
    _, tens, _ = measured_peaks()
    gen = torch.Generator(device="cuda").manual_seed(0)
    layers, out = BASE_LAYERS, []
    for L, B in shapes:
        q = torch.randn((layers, B, H, L, D), device="cuda", generator=gen).half().float()
        k = torch.randn((layers, B, HK, L, D), device="cuda", generator=gen).half()
        v = torch.randn((layers, B, HK, L, D), device="cuda", generator=gen).half()
        if kv == "q8_0":
            k, v = q8_0_blocks(k.float()), q8_0_blocks(v.float())
        o = torch.empty((layers, B, L, H, D), device="cuda")
        if with_mask:
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
        ms = timer.ms(graph.replay, 20)
        flops = layers * B * 4.0 * H * D * L * (L + 1) / 2
        r = {"config": f"prefill L={L} B={B} x {layers} layers, {kv} K/V" + (", mask tensor" if with_mask else ""),
             "us_per_layer": ms * 1e3 / layers, "tflops_causal_useful": flops / (ms * 1e-3) / 1e12,
             "frac_of_measured_bf16_peak": flops / (ms * 1e-3) / 1e12 / tens}
        if cpu:
            r["cpu_baseline"] = cpu_attention_us(B, L, L, kv, True, n_layers=2 if B > 1 else 4)
        out.append(r)
        del q, k, v, o, graph
    return out


def time_projection(pkg, torch, eng, timer, S, hidden=1024, layers=BASE_LAYERS + RES_LAYERS):
    """The batched Q/K/V projection with the rotary embedding in its epilogue (hidden -> 16 + 2 + 2 heads of 64, f16
    weights) for S streams, one launch pair per layer with weights of its own, replayed from a CUDA graph: us per layer
    with the weights where the previous replay left them (79 MB: they fit the L2) and with the L2 scrubbed first;
    roofline = the weight bytes / time against the measured HBM peak."""
    hbm, _, _ = measured_peaks()
    gen = torch.Generator(device="cuda").manual_seed(S)
    n_out = (H + 2 * HK) * D
    w = (torch.randn((layers, n_out, hidden), device="cuda", generator=gen) / hidden ** 0.5).half()
    x = torch.randn((layers, S, hidden), device="cuda", generator=gen)
    pos = torch.randint(0, 4096, (S,), device="cuda", dtype=torch.int32, generator=gen)
    table = eng.rope_table(pos)
    for l in range(layers):
        eng.qkv_project(x[l], w[l], H, HK, rope_table=table)
    eng.sync_status()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for l in range(layers):
            eng.qkv_project(x[l], w[l], H, HK, rope_table=table)
    warm, cold = timer.ms(graph.replay, 20), timer.ms(graph.replay, 10, cold=True)
    wbytes = n_out * hidden * 2.0
    return {"config": f"Q/K/V projection {hidden} -> {n_out}, {S} streams, f16 weights, rotary embedding in the epilogue, x {layers} layers",
            "warm_us_per_layer": warm * 1e3 / layers, "cold_us_per_layer": cold * 1e3 / layers, "weight_bytes_per_layer": wbytes,
            "cold_weight_gb_s": wbytes * layers / (cold * 1e-3) / 1e9, "cold_frac_of_measured_hbm": wbytes * layers / (cold * 1e-3) / 1e9 / hbm,
            "launches_per_layer": 2, "per_stream_in_the_reference": "one ggml_mul_mat + two ggml_rope_ext + two ggml_cpy nodes per stream and layer"}


def time_layer_linears(pkg, torch, eng, timer, S, hidden=1024, inter=4096, layers=BASE_LAYERS):
    """The other matrices of a decoder layer for S streams (vox_linear): output projection with the residual add, RMS norm +
    gate_up projection + SwiGLU (f16 out), down projection with the residual add; five launches per layer, every layer with
    weights of its own (30 MB of f16 per layer: 24 layers do not fit the L2), replayed from a CUDA graph.  us per layer
    and per matrix; roofline = the weight bytes / time against the measured HBM peak."""
    hbm, _, _ = measured_peaks()
    gen = torch.Generator(device="cuda").manual_seed(S + 1)
    w_o = (torch.randn((layers, hidden, hidden), device="cuda", generator=gen) / hidden ** 0.5).half()
    w_gu = (torch.randn((layers, 2 * inter, hidden), device="cuda", generator=gen) / hidden ** 0.5).half()
    w_dn = (torch.randn((layers, hidden, inter), device="cuda", generator=gen) / inter ** 0.5).half()
    norm = torch.ones((hidden,), device="cuda")
    attn = torch.randn((S, hidden), device="cuda", generator=gen)
    h0 = torch.randn((S, hidden), device="cuda", generator=gen)
    h1, h2 = torch.empty_like(h0), torch.empty_like(h0)
    fused = torch.empty((S, inter), device="cuda", dtype=torch.float16)  # leaves SwiGLU as f16, enters down_proj as f16

    def o_proj(l):
        eng.linear(attn, w_o[l], pkg.LINEAR_RESIDUAL, residual=h0, scale=0.3, out=h1)

    def gate_up(l):
        eng.linear(h1, w_gu[l], pkg.LINEAR_SWIGLU, norm_weight=norm, norm_eps=1e-5, out=fused)

    def down(l):
        eng.linear(fused, w_dn[l], pkg.LINEAR_RESIDUAL, residual=h1, scale=0.3, out=h2)

    def graph_of(fns):
        for l in range(layers):
            for f in fns:
                f(l)
        eng.sync_status()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for l in range(layers):
                for f in fns:
                    f(l)
        return g

    out = {"config": f"o_proj {hidden} -> {hidden} + residual; RMS norm + gate_up {hidden} -> 2 x {inter} + SwiGLU; down {inter} -> {hidden} + residual; "
                     f"{S} streams, f16 weights, x {layers} layers",
           "launches_per_layer": 5, "per_stream_in_the_reference": "three ggml_mul_mat, ggml_rms_norm, ggml_mul, ggml_swiglu_split, two ggml_scale and two ggml_add nodes per stream and layer"}
    wbytes = {"o_proj": hidden * hidden * 2.0, "gate_up": 2 * inter * hidden * 2.0, "down": hidden * inter * 2.0}
    for name, fns in (("o_proj", [o_proj]), ("gate_up", [gate_up]), ("down", [down]), ("layer", [o_proj, gate_up, down])):
        g = graph_of(fns)
        cold = timer.ms(g.replay, 10, cold=True)
        nbytes = sum(wbytes.values()) if name == "layer" else wbytes[name]
        out[name] = {"cold_us_per_layer": cold * 1e3 / layers, "weight_bytes_per_layer": nbytes,
                     "cold_weight_gb_s": nbytes * layers / (cold * 1e-3) / 1e9, "cold_frac_of_measured_hbm": nbytes * layers / (cold * 1e-3) / 1e9 / hbm}
    return out


def time_decode_shape(pkg, torch, eng, timer, L, B, kv, n_base, n_res, cpu=False):
    """Single-token attention of `n_base + n_res` layers over B streams of L rows each, issued from C as one step
    (no append): warm and cold (L2 scrubbed) us per layer, GB/s, fraction of the measured HBM peak; for one stream
    also the step replayed from a CUDA graph (issued call by call a single stream is bound by the host's launch rate)."""
    hbm, _, _ = measured_peaks()
    gen = torch.Generator(device="cuda").manual_seed(L + B)
    g = pkg.Group(eng, n_streams=B, max_len=L, kv_type=pkg.F16 if kv == "f16" else pkg.Q8_0, base_layers=n_base, res_layers=n_res,
                  n_heads=H, n_kv_heads=HK, locdit_layers=0, cfm_steps=0)
    lens = np.full(B, L, np.int32)
    g.set_kv_len(lens)
    g.fill_synthetic(seed=L + B)
    bufs = {n: torch.randn(s, device="cuda", generator=gen) for n, s in g.buffer_shapes().items() if n.startswith("lm_")}
    step = lambda: g.step(bufs, advance=False)
    n_layers = n_base + n_res
    nbytes = n_layers * lm_bytes_per_layer(lens, kv)
    warm, cold = timer.ms(step, 20), timer.ms(step, 10, cold=True)
    eng.sync_status()
    graph_us = None
    if B == 1:
        side, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
        g.set_bound(L)
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                g.step(bufs, advance=False, stream=side)
        graph_us = timer.ms(graph.replay, 20) * 1e3 / n_layers
        eng.sync_status()
    r = {"config": f"decode kv={L} B={B} {kv} x {n_layers} layers", "bytes_per_layer": nbytes / n_layers,
         "warm_us_per_layer": warm * 1e3 / n_layers, "cold_us_per_layer": cold * 1e3 / n_layers,
         "graph_replay_us_per_layer": graph_us,
         "warm_gb_s": nbytes / (warm * 1e-3) / 1e9, "cold_gb_s": nbytes / (cold * 1e-3) / 1e9,
         "cold_frac_of_measured_hbm": nbytes / (cold * 1e-3) / 1e9 / hbm, "cold_frac_of_8000": nbytes / (cold * 1e-3) / 1e9 / 8000.0}
    if cpu:
        r["cpu_baseline"] = cpu_attention_us(B, 1, L, kv, False, n_layers=max(1, min(n_layers, (256 << 20) // (B * L * HK * D * 4))))
    g.close()
    return r


def aux_workload(args, pkg, torch):
    """--workload prefill | decode_sweep | decode_c1: one more configuration on one GPU, as a line of its own."""
    eng = pkg.Engine(torch.cuda.current_device())
    hbm, tens, src = measured_peaks()
    timer = Timer(torch)
    out = {"workload": args.workload, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tens, "source": src}, "results": []}
    if args.workload == "prefill":
        shapes = [(int(x.split("x")[0]), int(x.split("x")[1])) for x in args.prefill_shapes.split(",")]
        out["results"] = time_prefill(pkg, torch, eng, timer, shapes, args.prefill_kv, args.prefill_mask, cpu=not args.no_cpu_baseline)
    elif args.workload == "decode_c1":
        out["results"] = [time_decode_shape(pkg, torch, eng, timer, 256, 1, "f16", BASE_LAYERS, 0, cpu=not args.no_cpu_baseline)]
    elif args.workload == "projection":
        out["results"] = [time_projection(pkg, torch, eng, timer, S) for S in (256, 32)]
    elif args.workload == "layer_linears":
        out["results"] = [time_layer_linears(pkg, torch, eng, timer, S) for S in (256, 32)]
    elif args.workload == "decode_profile":
        # a reduced instance of the serving launch for profiler captures: one layer, 128 streams of 4096 rows (268 MB of
        # f16 K/V, 142 MB of q8_0: more than the L2 holds, far less than the serving workload's 8 to 17 GB)
        out["results"] = [time_decode_shape(pkg, torch, eng, timer, 4096, 128, args.kv_type, 1, 0, cpu=False)]
    elif args.workload == "locdit_profile":
        # the same for the LocDiT launch: 64 patches x 8 layers, one CFM timestep per launch (85 MB per launch)
        g = pkg.Group(eng, n_streams=64, max_len=64, kv_type=pkg.F16, base_layers=0, res_layers=0, n_heads=H, n_kv_heads=HK,
                      locdit_layers=DIT_LAYERS, locdit_seq=DIT_SEQ, cfm_steps=2)
        bufs = {n: torch.randn(s, device="cuda") for n, s in g.buffer_shapes().items() if n.startswith("dit_")}
        ms = timer.ms(lambda: g.step(bufs, advance=False), 10)
        out["results"] = [{"config": "LocDiT 64 patches x 8 layers, 2 CFM timesteps per step", "us_per_launch": ms * 1e3 / 2}]
        g.close()
    else:
        for t in ("f16", "q8_0"):
            for B in (1, 32):
                for L in (1024, 2048, 4096, 8192):
                    out["results"].append(time_decode_shape(pkg, torch, eng, timer, L, B, t, BASE_LAYERS, RES_LAYERS,
                                                            cpu=not args.no_cpu_baseline and L in (1024, 8192)))
    return out


# ------------------------------------------------------------------ the serving step

class Serving:
    """One rank's share of the population: a stream group, its step buffers on the device, and the timings taken on it."""

    def __init__(self, pkg, torch, eng, lens, kv_type, rank, total_steps, rope=False, cfm_zero_init=0):
        self.pkg, self.torch, self.eng, self.lens, self.kv_type = pkg, torch, eng, lens, kv_type
        max_len = ((KV_HI + 2 * (total_steps + 8) + 63) // 64) * 64
        self.group = pkg.Group(eng, n_streams=len(lens), max_len=max_len, kv_type=pkg.F16 if kv_type == "f16" else pkg.Q8_0,
                               base_layers=BASE_LAYERS, res_layers=RES_LAYERS, n_heads=H, n_kv_heads=HK, locdit_layers=DIT_LAYERS,
                               locdit_seq=DIT_SEQ, cfm_steps=CFM_STEPS, cfm_zero_init_steps=cfm_zero_init)
        self.group.set_kv_len(lens)
        self.group.fill_synthetic(seed=rank)
        if rope:  # llama.rope.freq_base of the reference's GGUF defaults, per-frequency factors as LongRoPE ships them
            self.group.set_rope(freq_base=10000.0, attn_factor=1.0, freq_factors=np.linspace(1.0, 4.0, 32, dtype=np.float32))
        self.shapes = self.group.buffer_shapes()
        gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
        self.dev = {n: (torch.empty(s, device="cuda") if n.endswith("out") else torch.randn(s, device="cuda", generator=gen))
                    for n, s in self.shapes.items()}
        self.stream = torch.cuda.current_stream()

    def close(self):
        self.group.close()
        self.dev = None

    def timed_steps(self, warmup, steps, barrier):
        """W untimed steps, then K steps between CUDA events with a barrier and a synchronize on both sides."""
        torch = self.torch
        for _ in range(warmup):
            self.group.step(self.dev, advance=True)
        self.eng.sync_status()
        barrier()
        l0 = self.eng.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for _ in range(steps):
            self.group.step(self.dev, advance=True)
        e1.record(self.stream)
        barrier()
        self.eng.sync_status()
        return e0.elapsed_time(e1) / steps, self.eng.launches - l0

    def decode_launch_us(self, reps=5):
        """Mean duration of one layer's decode launch by CUDA events on the launching stream over reps x 30 back-to-back
        launches issued from C (gaps between launches included), lengths as they now stand."""
        torch = self.torch
        lm_only = {n: x for n, x in self.dev.items() if n.startswith("lm_")}
        n_lm = BASE_LAYERS + RES_LAYERS
        self.group.step(lm_only, advance=False)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(self.stream)
        for _ in range(reps):
            self.group.step(lm_only, advance=False)
        b.record(self.stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / (reps * n_lm), lm_bytes_per_layer(self.group.kv_len(), self.kv_type)

    def e2e(self, steps, barrier, max_over_ranks):
        """The same step through the host-buffer entry point: pinned host inputs, H2D + launches + D2H every step."""
        torch = self.torch
        host = {n: torch.empty(s, dtype=torch.float32).pin_memory() for n, s in self.shapes.items()}
        for n, x in host.items():
            if not n.endswith("out"):
                x.copy_(self.dev[n])
        self.group.step_host(host, advance=True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.group.step_host(host, advance=True)
        barrier()
        return max_over_ranks(time.perf_counter() - t0) / steps


def locdit_latency(pkg, torch, eng, kv_type):
    """One patch for one stream: 10 launches issued call by call, and the same replayed from a CUDA graph."""
    gen = torch.Generator(device="cuda").manual_seed(99)
    one = pkg.Group(eng, n_streams=1, max_len=64, kv_type=pkg.F16 if kv_type == "f16" else pkg.Q8_0, base_layers=0, res_layers=0,
                    n_heads=H, n_kv_heads=HK, locdit_layers=DIT_LAYERS, locdit_seq=DIT_SEQ, cfm_steps=CFM_STEPS)
    one_t = {n: torch.randn(s, device="cuda", generator=gen) for n, s in one.buffer_shapes().items()}
    stream = torch.cuda.current_stream()
    for _ in range(3):
        one.step(one_t, advance=False)
    torch.cuda.synchronize()
    lb, reps = eng.launches, 20
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(reps):
        one.step(one_t, advance=False)  # the 10 CFM launches are issued back to back from C
    b.record(stream)
    torch.cuda.synchronize()
    issued_us = a.elapsed_time(b) * 1e3 / reps
    launches_per_step = (eng.launches - lb) / (reps * CFM_STEPS)
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
    return {"us_per_patch_single_stream": issued_us, "us_per_patch_single_stream_graph_replay": replayed_us,
            "launches_per_cfm_step": launches_per_step}


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

    if args.workload != "serving":
        if rank == 0:
            print(json.dumps(aux_workload(args, pkg, torch)))
        return

    hbm, tens, peak_src = measured_peaks()
    eng = pkg.Engine(local)
    total_steps = args.warmup + args.steps
    lens = streams_of_rank(args.scaling, args.streams, rank, world, pkg.partition_streams)
    clocks = ClockSampler(local)
    if rank == 0:
        clocks.start()

    # ---- device-resident throughput of this rank's share; the job's time is the slowest rank's
    srv = Serving(pkg, torch, eng, lens, args.kv_type, rank, total_steps + 8, args.rope, args.cfm_zero_init)
    my_ms, launches = srv.timed_steps(args.warmup, args.steps, barrier)
    ms_per_step = ranks.max(my_ms)
    total_streams = ranks.sum(float(len(lens)))
    value = total_streams / (ms_per_step * 1e-3)
    my_rows = float(np.sum(lens.astype(np.float64)))
    imbalance = {"kv_rows_max_over_mean": ranks.max(my_rows) / (ranks.sum(my_rows) / world),
                 "ms_max_over_mean": ms_per_step / (ranks.sum(my_ms) / world),
                 "streams_per_gpu_max": int(ranks.max(float(len(lens)))), "ms_per_step_slowest": ms_per_step,
                 "ms_per_step_mean": ranks.sum(my_ms) / world}

    # ---- roofline of the dominant kernel (split-KV decode) on this rank's launch
    dec_us, layer_bytes = srv.decode_launch_us()
    achieved = layer_bytes / (dec_us * 1e-6) / 1e9
    kernel = f"decode_kernel<{args.kv_type}>"
    ratio = dram_traffic_ratio(kernel)
    roofline = {"bound": "hbm", "kernel": kernel + " (one-wave grid over the flattened tile list; partials folded by the last CTA of each stream and kv head)",
                "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                "traffic": layer_bytes * ratio if ratio else None,
                "traffic_source": "DRAM bytes per algorithmic byte from an ncu capture of this kernel on a reduced instance, applied to this launch's algorithmic bytes" if ratio else None,
                "peak_source": peak_src, "us_per_launch": dec_us, "algorithmic_bytes_per_launch": layer_bytes,
                "frac_of_nominal_8000": achieved / 8000.0}

    # ---- end to end through the host-buffer entry point
    e2e = None
    if not args.no_e2e:
        h2d = ranks.sum(float(srv.group.step_bytes(0) + srv.group.step_bytes(2)))
        d2h = ranks.sum(float(srv.group.step_bytes(1) + srv.group.step_bytes(3)))
        e2e_steps = max(2, min(args.steps, 5))
        dt = srv.e2e(e2e_steps, barrier, ranks.max)
        e2e = {"value": total_streams / dt, "unit": "patches/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": dt * 1e3, "steps": e2e_steps}
    srv.close()

    # ---- N > 1: the weak-scaling figure beside the partitioned one (a full population per GPU)
    weak = None
    if world > 1 and args.scaling == "strong":
        wl = streams_of_rank("weak", args.streams, rank, world, pkg.partition_streams)
        ws = Serving(pkg, torch, eng, wl, args.kv_type, rank, total_steps + 8, args.rope, args.cfm_zero_init)
        w_ms, _ = ws.timed_steps(args.warmup, max(5, args.steps // 2), barrier)
        w_ms = ranks.max(w_ms)
        weak = {"value": world * args.streams / (w_ms * 1e-3), "unit": "patches/s", "streams_total": world * args.streams,
                "ms_per_step": w_ms, "note": "a population of its own on every GPU (per-GPU work held fixed)"}
        ws.close()

    clock_info = clocks.stop() if rank == 0 else None

    # ---- rank 0 at N = 1: LocDiT latency, the CPU baseline, and the other configured shapes
    locdit = cpu = extras = None
    if rank == 0 and world == 1:
        locdit = locdit_latency(pkg, torch, eng, args.kv_type)
        if not args.no_cpu_baseline:
            try:
                r = cpu_reference_throughput(args.cpu_sample_streams, 3, 1, args.kv_type, CFM_STEPS - args.cfm_zero_init)
                cpu = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
            except Exception as ex:  # the baseline is a report, it must not take the bench line down
                cpu = {"value": None, "unit": "patches/s", "cores": 0, "kind": "unavailable", "sample": repr(ex)}
        if not args.no_extras:
            extras = other_shapes(args, pkg, torch, eng, total_steps)

    if rank == 0:
        cfg = workload_config(args, total_streams)
        notes = {"host_numa_node": numa_node,
                 "rope": "rotary embedding of Q and the new K rows inside the decode launches" if args.rope else "applied by the caller",
                 "arithmetic": "f16 K/V (or q8_0), f32 Q and output, f16 tensor-core products with hi+lo split of Q and P, "
                               "f32 accumulation; LocDiT f32 throughout"}
        line = {"metric": "patches/s", "value": value, "unit": "patches/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": "f16" if args.kv_type == "f16" else "q8_0", "data": "synthetic", "config": cfg,
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clock_info,
                "imbalance": imbalance, "weak_scaling": weak, "locdit": locdit, "engine_notes": notes,
                "decode": {"gb_per_s": achieved, "pct_of_measured_peak": 100 * achieved / hbm, "pct_of_8000": 100 * achieved / 8000}}
        if extras:
            line.update(extras)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def other_shapes(args, pkg, torch, eng, total_steps):
    """The other configured shapes, each a fraction of a second on the GPU: causal prefill 512 x 1 and 512 x 8, the
    serving step on the other cache type, the long-form decode sweep and single-stream decode at 256 rows — each with
    the reference's ggml CPU attention on this machine's cores beside it (bounded: a few layers per shape)."""
    timer = Timer(torch)
    cpu = not args.no_cpu_baseline
    out = {}
    out["prefill"] = time_prefill(pkg, torch, eng, timer, [(512, 1), (512, 8), (2048, 2)], "f16", False, cpu=cpu)
    other = "q8_0" if args.kv_type == "f16" else "f16"
    srv = Serving(pkg, torch, eng, stream_lengths(args.streams, 0), other, 0, total_steps + 8)
    ms, _ = srv.timed_steps(args.warmup, max(5, args.steps // 2), lambda: torch.cuda.synchronize())
    us, nbytes = srv.decode_launch_us()
    hbm, _, _ = measured_peaks()
    out["decode_" + other] = {"config": f"the serving step on a {other} cache, {args.streams} streams", "patches_per_s": args.streams / (ms * 1e-3),
                              "ms_per_step": ms, "decode_us_per_launch": us, "decode_gb_s": nbytes / (us * 1e-6) / 1e9,
                              "frac_of_measured_hbm": nbytes / (us * 1e-6) / 1e9 / hbm, "algorithmic_bytes_per_launch": nbytes}
    srv.close()
    sweep = []
    for t in ("f16", "q8_0"):
        for B in (1, 32):
            for L in (1024, 2048, 4096, 8192):
                sweep.append(time_decode_shape(pkg, torch, eng, timer, L, B, t, BASE_LAYERS, RES_LAYERS, cpu=cpu and L in (1024, 8192)))
    out["decode_sweep"] = sweep
    out["decode_c1"] = time_decode_shape(pkg, torch, eng, timer, 256, 1, "f16", BASE_LAYERS, 0, cpu=cpu)
    out["qkv_projection"] = [time_projection(pkg, torch, eng, timer, S) for S in (256, 32)]
    out["layer_linears"] = [time_layer_linears(pkg, torch, eng, timer, S) for S in (256, 32)]
    if cpu:
        out["locdit_cpu_baseline"] = cpu_attention_us(2, DIT_SEQ, DIT_SEQ, "f32", False, n_layers=CFM_STEPS * DIT_LAYERS)
    return out


if __name__ == "__main__":
    main()
