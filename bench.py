#!/usr/bin/env python3
"""Benchmark of the decode-time KV path: append of RoPE'd K/V + GQA flash-decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg1|cfg2|cfg3]

One "step" = one decode step of the whole model stack of the workload: every layer appends one token per sequence
and runs attention over its cache.  Default workload (`cfg1`): 28-layer Qwen3-0.6B shape (16 q / 8 kv heads,
head_dim 128), batch 1, fp16 cache, context 4096 growing by one token per step, synthetic seeded N(0,1) inputs.

Prints ONE JSON line (rank 0).  `value` is device-timed throughput with inputs resident in HBM; `e2e` is the same
metric through the host-buffer entry point (er_kv_decode_step_host) with H2D/D2H copies inside the timed region;
`roofline` is the attention kernel's algorithmic bytes over its CUDA-event-timed duration against the measured
copy bandwidth; `cpu_baseline` times the CPU restatement of the reference path on the host cores.

Multi-GPU (`--gpus N`, launched by torchrun, one rank per GPU): the path shards by sequence with no data-path
collective -- every rank advances its own sequence(s) -- so scaling is weak and `value` sums all ranks.

`--impl reference` times the reference's own CPU implementation of the path (its Swift sources cannot be built
here, so this is the C restatement under oracle/) with all host threads, on the same workload.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_kv_append_attention_tokens_per_s"
WORKLOADS = {
    # BASELINE.json configs[1]: the configuration the metric is quoted on
    "cfg1": dict(name="cfg1: Qwen3-0.6B shape, 28 layers, batch 1, fp16 KV, context 4096, 1 token appended per step",
                 layers=28, batch=1, heads=16, kv_heads=8, ctx=4096, precision="float16", layout="head_major", theta=1.0e6),
    "cfg1_token_major": dict(name="cfg1 with the reference's token-major [slot][kvHead][dim] ring layout",
                             layers=28, batch=1, heads=16, kv_heads=8, ctx=4096, precision="float16", layout="token_major",
                             theta=1.0e6),
    "cfg1_long": dict(name="cfg1 shape at context 32768 (asymptotic kernel bandwidth; not a BASELINE configuration)",
                      layers=28, batch=1, heads=16, kv_heads=8, ctx=32768, precision="float16", layout="head_major", theta=1.0e6),
    # BASELINE.json configs[2]
    "cfg2": dict(name="cfg2: Qwen3-0.6B shape, 28 layers, batch 8, TurboQuant turbo4 K / turbo3 V, fp16 norms, context 32768",
                 layers=28, batch=8, heads=16, kv_heads=8, ctx=32768, precision="turboquant", kbits=4, vbits=3, norm="float16",
                 layout="head_major", theta=1.0e6, outliers=True),
    # next-tier row of the scope table: the q8_0 KV format on the cfg1 shape
    "cfg1_q8": dict(name="cfg1 shape with a q8_0 KV cache (34-byte blocks of 32: fp16 scale + int8), context 4096",
                    layers=28, batch=1, heads=16, kv_heads=8, ctx=4096, precision="q8_0", layout="head_major", theta=1.0e6),
    "cfg1_q8_long": dict(name="cfg1 shape with a q8_0 KV cache at context 32768, batch 8",
                         layers=28, batch=8, heads=16, kv_heads=8, ctx=32768, precision="q8_0", layout="head_major", theta=1.0e6),
    "cfg3_4layers": dict(name="cfg3 shape with 4 of its 32 layers and 16 of its 64 sequences (profiler captures)",
                         layers=4, batch=16, heads=32, kv_heads=8, ctx=16384, ragged=(1024, 16384), precision="float16", layout="paged",
                         page_size=16, theta=5.0e5),
    "cfg1_q8_4layers": dict(name="cfg1 shape with a q8_0 KV cache at context 32768, batch 8, 4 of the 28 layers (profiler captures)",
                            layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, precision="q8_0", layout="head_major", theta=1.0e6),
    "cfg2_4layers": dict(name="cfg2 shape with 4 of its 28 layers (about 1 GB on the device: the size profiler captures use)",
                         layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, precision="turboquant", kbits=4, vbits=3,
                         norm="float16", layout="head_major", theta=1.0e6, outliers=True),
    # BASELINE.json configs[3] (single-GPU form: all kv heads on one GPU)
    "cfg3": dict(name="cfg3: Llama-3.1-8B shape, 32 layers, batch 64, fp16 KV in 16-token pages, context U[1024,16384]",
                 layers=32, batch=64, heads=32, kv_heads=8, ctx=16384, ragged=(1024, 16384), precision="float16", layout="paged",
                 page_size=16, theta=5.0e5),
    "cfg3_contiguous": dict(name="cfg3 heads (32 q / 8 kv) on contiguous head-major rows, 8 layers, batch 8, context 32768 "
                                 "(separates the page gather from the kernel; not a BASELINE configuration)",
                            layers=8, batch=8, heads=32, kv_heads=8, ctx=32768, precision="float16", layout="head_major", theta=5.0e5),
    # BASELINE.json configs[4], its prefill leg: one 2048-token chunk of one sequence and one layer against the context
    # already in the cache (Qwen3-4B heads, TurboQuant turbo4/turbo4 rows in 64-token pages); tensor-core bound
    "cfg4_prefill": dict(name="cfg4 prefill chunk: Qwen3-4B heads, 2048 query rows at the end of a 131072-token context, "
                              "turbo4/turbo4 in 64-token pages, one layer, one sequence per step",
                         prefill=True, heads=32, kv_heads=8, ctx=131072 - 2048, chunk=2048, precision="turboquant", kbits=4, vbits=4,
                         norm="float16", layout="paged", page_size=64, theta=1.0e6),
    "cfg4_prefill_f16": dict(name="cfg4 prefill chunk on an fp16 cache (same shape, 32768-token context)",
                             prefill=True, heads=32, kv_heads=8, ctx=32768, chunk=2048, precision="float16", layout="paged",
                             page_size=64, theta=1.0e6),
}
D = 128


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only-device-leg", action="store_true",
                    help="run only the device-resident timed leg (short runs under a profiler)")
    ap.add_argument("--shard", default="sequence", choices=["sequence", "heads"],
                    help="N > 1: 'sequence' = one replica of the workload per GPU (weak scaling, no collective); 'heads' = the kv "
                         "heads of the one workload split over the GPUs, outputs exchanged by an NCCL all-gather per step (strong "
                         "scaling; device leg only)")
    ap.add_argument("--cta-timeline", action="store_true",
                    help="with --only-device-leg: one extra step with the kernel's per-CTA phase stamps (er_kv_set_trace), reported "
                         "as cta_timeline_us = [min, median, max] over the CTAs, microseconds after the first CTA started")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU work budget of the cpu_baseline leg")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            p = json.load(open(path))
            return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch from the committed ncu capture of the same
# workload (profiles/flash_decode_dense_g2_cfg1.md); None where no capture exists.
NCU_TRAFFIC_BYTES_PER_LAUNCH = {"cfg1": 471218688 + 4663040}


def row_bytes(w):
    """Algorithmic cache bytes per (token, kv head): K row + V row (+ stored norms)."""
    if w["precision"] == "float16":
        return 2 * D * 2
    if w["precision"] == "q8_0":
        return 2 * (D // 32) * 34
    nb = 2 if w.get("norm", "float32") == "float16" else 4
    return (D * w["kbits"] + 31) // 32 * 4 + (D * w["vbits"] + 31) // 32 * 4 + 2 * nb


def sequence_lengths(w, seed=2):
    if "ragged" in w:
        lo, hi = w["ragged"]
        rng = np.random.Generator(np.random.PCG64(seed))
        return [int(x) for x in rng.integers(lo, hi + 1, size=w["batch"])]
    return [w["ctx"]] * w["batch"]


def step_bytes(w, lens, step_index):
    """Algorithmic bytes of one decode step: every cache row read once per kv head, one row written per
    (layer, sequence, kv head), Q read and O written."""
    rb = row_bytes(w)
    read = sum((n + step_index + 1) for n in lens) * w["kv_heads"] * rb * w["layers"]
    write = len(lens) * w["kv_heads"] * rb * w["layers"]
    qo = len(lens) * w["layers"] * w["heads"] * D * 4 * 2
    return read + write + qo


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 20 ms.  The sampler is started before the warm-up and
    stopped after a load window (the timed steps repeated for ~1.5 s right after the timed region, which by itself
    lasts only tens of milliseconds); samples taken while the GPU was idle (before the first launch) are dropped by
    keeping only those with power draw above half the maximum seen."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                rows.append((float(f[1]), float(f[2]), float(f[3]), [n for n, v in zip(names, f[5:9]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": []}
        pmax = max(r[2] for r in rows)
        load = [r for r in rows if r[2] >= 0.5 * pmax] or rows
        reasons = sorted({n for r in load for n in r[3]})
        return {"sm_mhz": statistics.median(r[0] for r in load), "sm_max_mhz": max(r[1] for r in rows), "power_w_max": pmax,
                "samples": len(load), "reasons": reasons,
                "window": "warm-up + timed steps + the same steps repeated for ~1.5 s, sampled every 20 ms"}


# ------------------------------------------------------------------------------------------------- CPU legs

def cpu_reference_leg(w, lens, budget_s, steps=None, warmup=1):
    """Times the CPU restatement of the reference path (oracle/) with every host thread on a bounded sample of the
    workload: `layers_sampled` of the model's layers per step, throughput scaled to the full layer count."""
    from oracle import er_oracle as oracle
    oracle.build()
    # torchrun exports OMP_NUM_THREADS=1 to its ranks; only one rank runs this leg, so it takes the cores the process may
    # use (the oracle passes the count in a num_threads clause, which overrides the environment)
    threads = max(oracle.max_threads(), len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    L, B, H, Hkv = w["layers"], len(lens), w["heads"], w["kv_heads"]
    rng = np.random.Generator(np.random.PCG64(7))
    turbo = w["precision"] == "turboquant"
    q8 = w["precision"] == "q8_0"
    max_len = max(lens) + 64
    # one layer's cache per sampled layer; lengths as in the workload
    def make_layer():
        if turbo:
            kw, vw = (D * w["kbits"] + 31) // 32, (D * w["vbits"] + 31) // 32
            return [dict(kc=rng.integers(0, 2 ** 32, size=(max_len * Hkv, kw), dtype=np.uint32),
                         kn=np.abs(rng.standard_normal(max_len * Hkv).astype(np.float32)) + 10,
                         vc=rng.integers(0, 2 ** 32, size=(max_len * Hkv, vw), dtype=np.uint32),
                         vn=np.abs(rng.standard_normal(max_len * Hkv).astype(np.float32)) + 10) for _ in range(B)]
        if q8:
            return [dict(k=rng.integers(0, 256, size=(max_len, Hkv, 136), dtype=np.uint8),
                         v=rng.integers(0, 256, size=(max_len, Hkv, 136), dtype=np.uint8)) for _ in range(B)]
        return [dict(k=rng.standard_normal((max_len, Hkv, D), dtype=np.float32).astype(np.float16).view(np.uint16),
                     v=rng.standard_normal((max_len, Hkv, D), dtype=np.float32).astype(np.float16).view(np.uint16)) for _ in range(B)]

    def one_layer_step(layer, s):
        for b in range(B):
            q = rng.standard_normal((H, D), dtype=np.float32)
            k = rng.standard_normal((Hkv, D), dtype=np.float32)
            v = rng.standard_normal((Hkv, D), dtype=np.float32)
            c = layer[b]
            if turbo:
                oracle.decode_step_turboquant(q, k, v, c["kc"], c["kn"], w["kbits"], c["vc"], c["vn"], w["vbits"], lens[b] + s,
                                              w["theta"], norm_fp16=w.get("norm") == "float16", threads=threads)
            elif q8:
                oracle.decode_step_q8(q, k, v, c["k"], c["v"], lens[b] + s, w["theta"], threads=threads)
            else:
                oracle.decode_step_f16(q, k, v, c["k"], c["v"], lens[b] + s, w["theta"], threads=threads)

    probe_layer = make_layer()
    t0 = time.perf_counter()
    one_layer_step(probe_layer, 0)
    t_layer = time.perf_counter() - t0
    if steps is None:
        layers_sampled = max(1, min(L, int(budget_s / max(t_layer, 1e-6) / 4)))
        steps = max(1, min(32, int(budget_s / (t_layer * layers_sampled))))
    else:
        total = steps + warmup
        layers_sampled = max(1, min(L, int(150.0 / max(t_layer * total, 1e-6))))
    layers = [probe_layer] + [make_layer() for _ in range(layers_sampled - 1)]
    for s in range(warmup):
        for layer in layers:
            one_layer_step(layer, s)
    t0 = time.perf_counter()
    for s in range(steps):
        for layer in layers:
            one_layer_step(layer, warmup + s)
    dt = time.perf_counter() - t0
    per_step_full = dt / steps * (L / layers_sampled)
    sample = "%d decode steps x %d of %d layers (batch %d, context %d), time scaled by %d/%d" % (
        steps, layers_sampled, L, B, max(lens), L, layers_sampled)
    return dict(value=B / per_step_full, unit="tokens/s", cores=threads, kind="port", sample=sample,
                ms_per_step=per_step_full * 1e3, steps=steps)


def run_reference_impl(args, w, lens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_reference_leg(w, lens, args.cpu_seconds, steps=args.steps, warmup=max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"], "implementation": "CPU restatement of the reference path (oracle/er_oracle.c), "
                   "OpenMP over heads; the reference's Swift/Metal sources cannot be built in this environment"},
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------- GPU leg

def build_cache(er, torch, w, lens, extra_tokens):
    B, L, Hkv = len(lens), w["layers"], w["kv_heads"]
    cap = (max(lens) + extra_tokens + 15) // 16 * 16
    layout = {"head_major": er.Layout.head_major, "token_major": er.Layout.token_major, "paged": er.Layout.paged}[w["layout"]]
    kw = {}
    if layout == er.Layout.paged:
        ps = w["page_size"]
        need = sum((n + extra_tokens + ps - 1) // ps for n in lens)
        kw = dict(page_size=ps, num_pages=need)
    if w["precision"] == "float16":
        cache = er.KVCache(cap, L, Hkv, D, er.Precision.float16, max_batch=B, layout=layout, **kw)
    elif w["precision"] == "q8_0":
        cache = er.KVCache(cap, L, Hkv, D, er.Precision.q8_0, max_batch=B, layout=layout, **kw)
    else:
        nf = er.NormFormat.float16 if w.get("norm") == "float16" else er.NormFormat.float32
        cache = er.KVCache(cap, L, Hkv, D, er.Precision.turboquantV2, key_type=w["kbits"], value_type=w["vbits"], norm_format=nf,
                           max_batch=B, layout=layout, **kw)
    if layout == er.Layout.paged:
        rng = np.random.Generator(np.random.PCG64(2))
        # ER_BENCH_IDENTITY_PAGES=1: pages in order instead of the random permutation (separates DRAM locality from the gather)
        alloc = er.BlockTableAllocator(kw["num_pages"], w["page_size"], free_order=(np.arange(kw["num_pages"]) if os.environ.get("ER_BENCH_IDENTITY_PAGES") else rng.permutation(kw["num_pages"])))
        for b, n in enumerate(lens):
            cache.set_block_table(b, alloc.ensure(b, n + extra_tokens))
    return cache


def fill_cache(er, torch, cache, w, lens, sp, seed):
    """Pre-fills every (layer, sequence) with seeded N(0,1) rows (cast to fp16) through the bulk append entry point."""
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    Hkv = w["kv_heads"]
    scale_k = scale_v = None
    if w.get("outliers"):
        rng = np.random.Generator(np.random.PCG64(seed))
        scale_k = torch.as_tensor(np.where(rng.random((Hkv, D)) < 0.01, 20.0, 1.0).astype(np.float32)).cuda()
        scale_v = torch.as_tensor(np.where(rng.random((Hkv, D)) < 0.01, 20.0, 1.0).astype(np.float32)).cuda()
    chunk = 8192
    for l in range(w["layers"]):
        for b, n in enumerate(lens):
            for s in range(0, n, chunk):
                c = min(chunk, n - s)
                k = torch.randn((c, Hkv, D), generator=g, device="cuda", dtype=torch.float32)
                v = torch.randn((c, Hkv, D), generator=g, device="cuda", dtype=torch.float32)
                if scale_k is not None:
                    k, v = k * scale_k, v * scale_v
                k, v = k.half().float(), v.half().float()
                cache.write_rows(l, b, s, c, k, v, sp)
    torch.cuda.synchronize()


def run_ours(args, w, lens):
    import torch
    import torch.distributed as dist
    import edgerunner_b200 as er
    from edgerunner_b200.sharding import max_over_ranks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit("--gpus %d needs torchrun with %d ranks (WORLD_SIZE=%d)" % (args.gpus, args.gpus, world))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    shard_heads = args.shard == "heads" and world > 1
    if shard_heads:
        # rank r owns kv heads [r * Hkv / N, (r + 1) * Hkv / N) and their q heads: its cache and its q/k/v hold only those
        if w["kv_heads"] % world:
            raise SystemExit("--shard heads needs kv_heads %% gpus == 0")
        w = dict(w, heads=w["heads"] // world, kv_heads=w["kv_heads"] // world)
        args.only_device_leg = True
    L, B, H, Hkv = w["layers"], len(lens), w["heads"], w["kv_heads"]
    K, W = args.steps, max(args.warmup, 0)
    sp = er.step_params(rope_theta=w["theta"])
    cache = build_cache(er, torch, w, lens, K + W + 8)
    fill_cache(er, torch, cache, w, lens, sp, seed=1000 + rank)
    base_positions = list(lens)

    def set_start():
        for b, n in enumerate(base_positions):
            cache.set_position(n, seq=b)

    g = torch.Generator(device="cuda")
    g.manual_seed(5 + rank)
    pool = min(K + W, 64)      # distinct per-step inputs, cycled (a step's cost does not depend on their values)
    qs = torch.randn((pool, L, B, H, D), generator=g, device="cuda").half().float()
    ks = torch.randn((pool, L, B, Hkv, D), generator=g, device="cuda").half().float()
    vs = torch.randn((pool, L, B, Hkv, D), generator=g, device="cuda").half().float()
    out = torch.empty((L, B, H, D), device="cuda", dtype=torch.float32)
    gathered = torch.empty((world, L, B, H, D), device="cuda", dtype=torch.float32) if shard_heads else None
    stream = torch.cuda.current_stream()

    def exchange():
        if shard_heads:      # every rank ends the step with all heads' outputs: [rank][L][B][H / N][128]
            dist.all_gather_into_tensor(gathered, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- leg 1: device-resident inputs, whole step through er_kv_decode_step ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    set_start()
    for s in range(W):
        cache.decode_step(qs[s % pool], ks[s % pool], vs[s % pool], out, H, sp, stream=stream)
        exchange()
    barrier()
    launches0 = er.lib().er_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for s in range(K):
        i = (W + s) % pool
        cache.decode_step(qs[i], ks[i], vs[i], out, H, sp, stream=stream)
        exchange()
    e1.record(stream)
    barrier()
    launches = er.lib().er_kernel_launch_count() - launches0
    ms_total = max_over_ranks(e0.elapsed_time(e1), device="cuda")
    # load window for the clock samples: the same steps again (positions rewound so the cache capacity holds)
    t_load = time.perf_counter()
    while rank == 0 and time.perf_counter() - t_load < 1.5:
        set_start()
        for s in range(min(K + W, 128)):
            cache.decode_step(qs[s % pool], ks[s % pool], vs[s % pool], out, H, sp, stream=stream)
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    for b, n in enumerate(base_positions):      # restore the post-run state the checks below expect
        cache.set_position(n + W + K, seq=b)
    assert cache.device_status() == 0, "device-side wait timed out"
    for b, n in enumerate(base_positions):
        assert cache.total_written(0, b) == n + W + K
    tokens = B * K * (1 if shard_heads else world)
    value = tokens / (ms_total * 1e-3)
    bytes_total = sum(step_bytes(w, lens, W + s) for s in range(K))
    hbm_gbs = bytes_total / (ms_total * 1e-3) / 1e9       # per GPU

    if args.only_device_leg:
        timeline = None
        if args.cta_timeline and rank == 0:
            n_ctas = cache.set_trace(None, 0)
            stamps = torch.zeros(n_ctas, 8, dtype=torch.int64, device="cuda")
            cache.set_trace(stamps, n_ctas)
            set_start()
            cache.decode_step(qs[0], ks[0], vs[0], out, H, sp, stream=stream)
            torch.cuda.synchronize()
            cache.set_trace(None, 0)
            t = stamps.cpu().numpy().astype(np.float64)
            t = (t - t[:, 0].min()) / 1e3
            names = ["cta_start", "work_list_built", "first_tile_landed", "streaming_done", "before_exit_sync", "after_exit_sync", "cta_end"]
            timeline = {nm: [round(float(f(t[:, i])), 2) for f in (np.min, np.median, np.max)] for i, nm in enumerate(names)}
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                              "ms_per_step": ms_total / K, "hbm_gbs_per_gpu": round(hbm_gbs, 1), "gpu_launches": int(launches),
                              "scaling": "strong" if shard_heads else "weak",
                              "config": {"workload": w["name"],
                                         "sharding": ("kv heads split over the GPUs, NCCL all-gather of the outputs every step" if shard_heads
                                                      else "by sequence, one replica per GPU, no collective") if world > 1 else "single GPU"},
                              "note": "device leg only", **({"cta_timeline_us": timeline} if timeline else {})}))
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- leg 2: per-kernel durations (append / attention) with CUDA events, same steps, split entry points ----
    set_start()
    for s in range(W):
        cache.decode_step(qs[s % pool], ks[s % pool], vs[s % pool], out, H, sp, stream=stream)
    torch.cuda.synchronize()
    n_probe = min(K, 64)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_probe)]
    for s in range(n_probe):
        i = (W + s) % pool
        evs[s][0].record(stream)
        cache.append_rope_kv(ks[i], vs[i], sp, stream=stream)
        evs[s][1].record(stream)
        cache.attention_decode(qs[i], out, H, sp, pending=1, stream=stream)
        evs[s][2].record(stream)
        cache.advance(1, stream=stream)
    torch.cuda.synchronize()
    t_append = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    t_attn = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    attn_bytes = statistics.mean(step_bytes(w, lens, W + s) for s in range(n_probe)) - B * Hkv * row_bytes(w) * L
    peak, peak_src = measured_peaks()
    split_attn_ms = t_attn
    fused_single_launch = int(launches) == K        # fp16 rows: the timed region is K launches of the one fused kernel
    if fused_single_launch:
        # the kernel's average launch duration is the timed region itself (events around the K launches of leg 1);
        # the split-call figure above pays an event pair and a second launch per step
        t_attn = ms_total / K
        attn_bytes = bytes_total / K
    achieved = attn_bytes / (t_attn * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "flash_decode_kernel", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(args.workload),
                "traffic_source": ("ncu capture summarised in profiles/flash_decode_dense_g2_cfg1.md, taken at context ~4100 where the "
                                   "algorithmic bytes are 475.8 MB; the timed steps here run a few hundred tokens further")
                if args.workload == "cfg1" else None,
                "peak_source": peak_src,
                "algorithmic_bytes_per_launch": int(attn_bytes), "launch_ms": round(t_attn, 5),
                "append_kernel_ms": round(t_append, 5), "frac_of_8tbs": round(achieved / 8000.0, 4),
                "timed_as": ("the K launches of the timed region (append fused into the kernel)" if fused_single_launch
                             else "attention launch between per-step CUDA events (split entry points)"),
                "split_call_attention_launch_ms": round(split_attn_ms, 5)}

    # ---- leg 3: end to end through the host-buffer entry point (H2D q/k/v + D2H out every step) ----
    hq = torch.empty((pool, L, B, H, D), dtype=torch.float32).pin_memory().copy_(qs.cpu())
    hk = torch.empty((pool, L, B, Hkv, D), dtype=torch.float32).pin_memory().copy_(ks.cpu())
    hv = torch.empty((pool, L, B, Hkv, D), dtype=torch.float32).pin_memory().copy_(vs.cpu())
    hout = torch.empty((L, B, H, D), dtype=torch.float32).pin_memory()
    set_start()
    # raw addresses of the pinned buffers (the entry point takes plain pointers; slicing tensors per step would add tens of
    # microseconds of interpreter time to an 84 us step) and a numpy view for reading the result on the host
    hq_p = [hq[i].data_ptr() for i in range(pool)]
    hk_p = [hk[i].data_ptr() for i in range(pool)]
    hv_p = [hv[i].data_ptr() for i in range(pool)]
    hout_p, hout_np, stream_p = hout.data_ptr(), hout.numpy(), stream.cuda_stream
    for s in range(W):
        cache.decode_step_host(hq_p[s % pool], hk_p[s % pool], hv_p[s % pool], hout_p, H, sp, stream=stream_p)
    barrier()
    e0.record(stream)
    t0 = time.perf_counter()
    checksum = 0.0
    for s in range(K):
        i = (W + s) % pool
        cache.decode_step_host(hq_p[i], hk_p[i], hv_p[i], hout_p, H, sp, stream=stream_p)
        checksum += float(hout_np[0, 0, 0, 0])       # the host reads the step's result
    e1.record(stream)
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), wall_ms), device="cuda")
    assert math.isfinite(checksum)
    e2e = {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
           "h2d_bytes_per_step": int(hq[0].numel() + hk[0].numel() + hv[0].numel()) * 4, "d2h_bytes_per_step": int(hout.numel()) * 4,
           "entry_point": "er_kv_decode_step_host"}

    # ---- leg 4: one launch per layer (how a model that interleaves its own projections would call it), plain
    #      launches and replayed as a CUDA graph of the 28 launches (positions live on the device, so one captured
    #      step can be replayed for every following step) ----
    def per_layer_step(i):
        for l in range(L):
            cache.decode_step(qs[i, l], ks[i, l], vs[i, l], out[l], H, sp, layer_begin=l, layer_end=l + 1, stream=torch.cuda.current_stream())

    set_start()
    for s in range(min(W, 4)):
        per_layer_step(s % pool)
    torch.cuda.synchronize()
    n_pl = min(K, 32)
    e0.record(stream)
    for s in range(n_pl):
        per_layer_step((W + s) % pool)
    e1.record(stream)
    torch.cuda.synchronize()
    per_layer_tok_s = B * n_pl / (e0.elapsed_time(e1) * 1e-3)
    per_layer_graph_tok_s = None
    try:
        set_start()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            per_layer_step(0)                      # warm the capture stream
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            per_layer_step(0)
        set_start()
        for _ in range(4):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n_pl):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        per_layer_graph_tok_s = B * n_pl / (e0.elapsed_time(e1) * 1e-3)
        assert cache.total_written(0, 0) == base_positions[0] + 4 + n_pl
    except Exception as exc:   # graph capture is an optional extra figure
        per_layer_graph_tok_s = "unavailable: %s" % (str(exc).splitlines()[0][:120] if str(exc) else type(exc).__name__)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = cpu_reference_leg(w, lens, args.cpu_seconds)
        cpu = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "layers": L, "batch_per_gpu": B, "q_heads": H, "kv_heads": Hkv, "head_dim": D,
                       "kv_storage": w["precision"], "layout": w["layout"],
                       "launch": "layer-batched: one append + one persistent attention launch per step for all layers",
                       "sharding": "by sequence, one replica of the workload per GPU, no collective" if world > 1 else "single GPU",
                       "l2": "cache bytes read per step (%.0f MB) exceed the 126 MB L2; no flush needed" % (step_bytes(w, lens, W) / 1e6),
                       "per_layer_launch_tokens_per_s": per_layer_tok_s,
                       "per_layer_launch_cuda_graph_tokens_per_s": per_layer_graph_tok_s},
            "hbm_gbs_per_gpu": round(hbm_gbs, 1), "frac_of_8tbs": round(hbm_gbs / 8000.0, 4),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args, w):
    """Chunked-prefill attention (er_kv_attention_prefill): step = one chunk of one sequence and one layer.  Useful FLOPs
    4 * S * (ctx + (S + 1) / 2) * Hq * 128 (causal), against the measured cuBLAS bf16 peak."""
    import torch
    import edgerunner_b200 as er
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    H, Hkv, ctx, S = w["heads"], w["kv_heads"], w["ctx"], w["chunk"]
    T = ctx + S
    n_pages = (T + w["page_size"] - 1) // w["page_size"]
    kw = dict(layout=er.Layout.paged, page_size=w["page_size"], num_pages=n_pages)
    if w["precision"] == "float16":
        cache = er.KVCache(T, 1, Hkv, D, er.Precision.float16, **kw)
    else:
        cache = er.KVCache(T, 1, Hkv, D, er.Precision.turboquantV2, key_type=w["kbits"], value_type=w["vbits"],
                           norm_format=er.NormFormat.float16, **kw)
    cache.set_block_table(0, np.random.Generator(np.random.PCG64(4)).permutation(n_pages).astype(np.int32))
    sp = er.step_params(rope_theta=w["theta"])
    g = torch.Generator(device="cuda").manual_seed(9)
    for s0 in range(0, T, 8192):
        n = min(8192, T - s0)
        cache.write_rows(0, 0, s0, n, torch.randn((n, Hkv, D), device="cuda", generator=g).half().float(),
                         torch.randn((n, Hkv, D), device="cuda", generator=g).half().float(), sp)
    q = torch.randn((S, H, D), device="cuda", generator=g).half().float()
    out = torch.empty((S, H, D), device="cuda")
    K, W = args.steps, max(args.warmup, 0)
    for _ in range(W):
        cache.attention_prefill(0, 0, q, out, H, S, sp)
    torch.cuda.synchronize()
    launches0 = er.lib().er_kernel_launch_count()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        cache.attention_prefill(0, 0, q, out, H, S, sp)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / K
    flops = 4.0 * S * (ctx + (S + 1) / 2.0) * H * D
    tflops = flops / ms / 1e9
    peak = None
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        peak_src = "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        peak, peak_src = 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"
    print(json.dumps({
        "metric": "prefill_attention_tflops", "value": round(tflops, 1), "unit": "TFLOP/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "dtype": "f16 operands (hi+lo pairs), f32 accumulate", "data": "synthetic",
        "query_tokens_per_s_per_layer": round(S / ms * 1e3, 1),
        "config": {"workload": w["name"], "q_heads": H, "kv_heads": Hkv, "context": ctx, "chunk": S,
                   "l2": "K/V of a kv head are shared by the chunk's CTAs through L2 by design; inputs exceed L2 at this context"},
        "roofline": {"bound": "tensor", "achieved": round(tflops, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(tflops / peak, 4),
                     "peak_source": peak_src, "traffic": None,
                     "note": "useful FLOPs; the kernel issues twice as many (fp16 hi+lo operand pairs)"},
        "gpu_launches": int(er.lib().er_kernel_launch_count() - launches0), "clocks": clocks}))


def main():
    args = parse_args()
    w = WORKLOADS[args.workload]
    if w.get("prefill"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the prefill workloads are measured on the GPU path only"}))
            return
        run_prefill(args, w)
        return
    lens = sequence_lengths(w)
    if args.impl == "reference":
        run_reference_impl(args, w, lens)
    else:
        run_ours(args, w, lens)


if __name__ == "__main__":
    main()
