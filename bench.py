#!/usr/bin/env python3
"""Benchmark of the decode-time KV path: append of RoPE'd K/V + GQA flash-decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--legs cfg1,cfg2]

One "step" = one decode step of the whole model stack of the workload: every layer appends one token per sequence
and runs attention over its cache.  Default workload (`cfg3`, the largest configuration that fits one GPU): 32-layer
Llama-3.1-8B shape (32 q / 8 kv heads, head_dim 128), batch 64 with context lengths uniform in [1024, 16384], fp16 cache
in 16-token pages behind a seeded random block table, synthetic seeded N(0,1) inputs.

Multi-GPU (`--gpus N`, launched by torchrun, one rank per GPU): the kv heads of that ONE workload are split over the
ranks (strong scaling: `value` = the batch's tokens per second of the whole job).  Every rank ends each step holding the
outputs of all heads as [layers, batch, heads, 128]: the decode kernel's merge epilogue stores its rows into every
peer's buffer (CUDA IPC, plain stores) and a 4-byte all-reduce orders the step's completion (`--exchange p2p`, default),
or an NCCL all-gather plus a re-layout kernel (`--exchange nccl`).  The exchange is inside the timed region; before
timing, the exchanged tensor of a small case is checked bit for bit against the shards computed on the rank's own GPU.

Prints ONE JSON line (rank 0).  `value` is device-timed (CUDA events, max over ranks, median of `--repeats` timed
regions of K steps) with inputs resident in HBM; `e2e` is the same metric with this step's q/k/v copied from pinned host
memory and the result copied back inside the timed region (er_kv_decode_step_host on one GPU); `roofline` is the
attention kernel's algorithmic bytes over its CUDA-event-timed duration against the measured copy bandwidth;
`cpu_baseline` times the CPU restatement of the reference path on the host cores; `legs` (one GPU only) carries the same
figures for the other single-GPU configurations (cfg1: 28 layers, batch 1, context 4096; cfg2: TurboQuant K4/V3, batch 8,
context 32768).

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
    # benchmark contract, configuration [1]
    "cfg1": dict(name="cfg1: Qwen3-0.6B shape, 28 layers, batch 1, fp16 KV, context 4096, 1 token appended per step",
                 layers=28, batch=1, heads=16, kv_heads=8, ctx=4096, precision="float16", layout="head_major", theta=1.0e6),
    "cfg1_per_layer": dict(name="cfg1 with one call per layer (28 launches per step: how a model that interleaves its own projections calls the path)",
                           layers=28, batch=1, heads=16, kv_heads=8, ctx=4096, precision="float16", layout="head_major", theta=1.0e6, per_layer=True),
    "cfg1_token_major": dict(name="cfg1 with the reference's token-major [slot][kvHead][dim] ring layout",
                             layers=28, batch=1, heads=16, kv_heads=8, ctx=4096, precision="float16", layout="token_major",
                             theta=1.0e6),
    "cfg1_long": dict(name="cfg1 shape at context 32768 (asymptotic kernel bandwidth; not one of the contract's configurations)",
                      layers=28, batch=1, heads=16, kv_heads=8, ctx=32768, precision="float16", layout="head_major", theta=1.0e6),
    # benchmark contract, configuration [2]
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
    # third next-tier row of the scope table: balanced / aggressive rows (32 high-precision channels, QJL signs) on the cfg2 shape
    "cfg2_balanced": dict(name="cfg2 shape with balanced TurboQuant rows (3 / 5 bits, 96-byte rows), residual terms on",
                          layers=28, batch=8, heads=16, kv_heads=8, ctx=32768, precision="balanced", residual_scale=1.0 / 128,
                          layout="head_major", theta=1.0e6, outliers=True),
    "cfg2_balanced_4layers": dict(name="cfg2 shape with balanced TurboQuant rows, 4 of its 28 layers (profiler captures)",
                                  layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, precision="balanced", residual_scale=1.0 / 128,
                                  layout="head_major", theta=1.0e6, outliers=True),
    "cfg2_balanced_4layers_simt": dict(name="cfg2 shape with balanced TurboQuant rows, 4 of its 28 layers, on the SIMT kernel",
                                       layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, precision="balanced", residual_scale=1.0 / 128,
                                       decode_kernel=3, layout="head_major", theta=1.0e6, outliers=True),
    "cfg2_balanced_4layers_contract": dict(name="cfg2 shape with balanced TurboQuant rows, 4 of its 28 layers, residual scales 0 (the reference's contract)",
                                           layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, precision="balanced", residual_scale=0.0,
                                           layout="head_major", theta=1.0e6, outliers=True),
    "cfg2_aggressive_4layers": dict(name="cfg2 shape with aggressive TurboQuant rows (2 / 3 bits, 80-byte rows), 4 of its 28 layers",
                                    layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, precision="aggressive", residual_scale=1.0 / 128,
                                    layout="head_major", theta=1.0e6, outliers=True),
    # layers whose keys and values use different row formats (two caches): the cfg2 shape with 4 layers, decode attention only
    **{"pair_%s_%s%s" % (k_, v_, "_simt" if simt_ else ""): dict(
        name="cfg2 shape, 4 layers: %s keys with %s values in two caches, decode attention%s" % (k_, v_, " on the SIMT kernel" if simt_ else ""),
        layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, keys=k_, values=v_, simt=simt_, theta=1.0e6)
       for k_, v_ in (("q8_0", "turbo3"), ("turbo3", "q8_0"), ("turbo4", "float16"), ("float16", "turbo3"), ("q8_0", "float16"))
       for simt_ in (False, True)},
    "cfg2_4layers": dict(name="cfg2 shape with 4 of its 28 layers (about 1 GB on the device: the size profiler captures use)",
                         layers=4, batch=8, heads=16, kv_heads=8, ctx=32768, precision="turboquant", kbits=4, vbits=3,
                         norm="float16", layout="head_major", theta=1.0e6, outliers=True),
    # benchmark contract, configuration [3]: the largest configuration that fits one GPU (73 GB of cache) -- the default workload
    "cfg3": dict(name="cfg3: Llama-3.1-8B shape, 32 layers, batch 64, fp16 KV in 16-token pages, context U[1024,16384]",
                 layers=32, batch=64, heads=32, kv_heads=8, ctx=16384, ragged=(1024, 16384), precision="float16", layout="paged",
                 page_size=16, theta=5.0e5),
    "cfg3_contiguous": dict(name="cfg3 heads (32 q / 8 kv) on contiguous head-major rows, 8 layers, batch 8, context 32768 "
                                 "(separates the page gather from the kernel; not one of the contract's configurations)",
                            layers=8, batch=8, heads=32, kv_heads=8, ctx=32768, precision="float16", layout="head_major", theta=5.0e5),
    # benchmark contract, configuration [4] as a whole job (run_cfg4): prefill chunk over all layers, then 128 decode steps
    "cfg4": dict(name="cfg4: Qwen3-4B shape, 36 layers, context 131072, TurboQuant turbo4 K / turbo4 V in 64-token pages; one 2048-token "
                      "prefill chunk per sequence, then 128 decode steps",
                 layers=36, batch=16, heads=32, kv_heads=8, ctx=131072, chunk=2048, decode_steps=128, precision="turboquant", kbits=4, vbits=4,
                 norm="float16", layout="paged", page_size=64, theta=1.0e6),
    # benchmark contract, configuration [4], decode leg on one GPU: 2 of the 16 sequences with all heads (an 8-GPU run gives each pair of
    # GPUs 4 sequences and each GPU half of the heads: the same 10 GB of codes per GPU)
    "cfg4_decode_slice": dict(name="cfg4 decode, one GPU's share: Qwen3-4B shape, 36 layers, 2 of the 16 sequences at context 131072, "
                                   "TurboQuant turbo4 K / turbo4 V, fp16 norms, 64-token pages",
                              layers=36, batch=2, heads=32, kv_heads=8, ctx=131072, precision="turboquant", kbits=4, vbits=4,
                              norm="float16", layout="paged", page_size=64, theta=1.0e6),
    "cfg4_decode_4layers": dict(name="cfg4 decode shape with 4 of its 36 layers and 2 sequences (about 1.1 GB on the device: profiler captures)",
                                layers=4, batch=2, heads=32, kv_heads=8, ctx=131072, precision="turboquant", kbits=4, vbits=4,
                                norm="float16", layout="paged", page_size=64, theta=1.0e6),
    # benchmark contract, configuration [4], its prefill leg: one 2048-token chunk of one sequence and one layer against the context
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
DEFAULT_WORKLOAD = "cfg3"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--legs", default=None,
                    help="comma-separated extra single-GPU workloads reported under `legs` (default: cfg1,cfg2 with the default "
                         "workload on one GPU, none otherwise; '' = none)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only-device-leg", action="store_true",
                    help="run only the device-resident timed leg (short runs under a profiler)")
    ap.add_argument("--shard", default="heads", choices=["sequence", "heads"],
                    help="N > 1: 'heads' = the kv heads of the one workload split over the GPUs, every GPU ends a step with all "
                         "heads' outputs (strong scaling); 'sequence' = one replica of the workload per GPU, no exchange (weak scaling)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="--shard heads: 'p2p' = peer stores from the decode kernel's epilogue + a 4-byte all-reduce; 'nccl' = "
                         "all-gather + re-layout kernel")
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


# DRAM traffic of one attention launch relative to its algorithmic bytes, from the committed ncu captures
# (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the captured launch): the captures are
# taken on a slice of the workload (a few GB on the device) and traffic grows in proportion to the rows processed, so
# the full launch's traffic is the ratio times its algorithmic bytes.
NCU_TRAFFIC_RATIO = {
    "float16/group2": (475.9 / 475.8, "profiles/flash_decode_dense_g2_cfg1.md (cfg1, full launch)"),
    "float16/group4": ((2252.2 + 5.4) / (2250.7 + 1.0 + 5.4), "profiles/flash_decode_dense_mma_g4_cfg3.md (cfg3, 4 of 32 layers, 16 of 64 sequences)"),
    "turboquant/group2": ((973.9 + 10.0) / (973.1 + 0.5 + 10.0), "profiles/flash_decode_turbo_mma_cfg2.md (cfg2, 4 of 28 layers)"),
    "q8_0/group2": ((2282.5 + 7.2) / (2281.7 + 7.2), "profiles/flash_decode_q8_g2.md (batch 8, context 32768, 4 of 28 layers)"),
}


def row_bytes(w):
    """Algorithmic cache bytes per (token, kv head): K row + V row (+ stored norms)."""
    if w["precision"] == "float16":
        return 2 * D * 2
    if w["precision"] == "q8_0":
        return 2 * (D // 32) * 34
    if w["precision"] in ("balanced", "aggressive"):
        # codes + side bits, mask 16 B, signs 16 B, two float norms, padded to 16 bytes: 96 / 80 bytes per row and side
        return 2 * (96 if w["precision"] == "balanced" else 80)
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
    pad = 96 + (steps or 0) + warmup      # rows the timed steps append
    max_len = max(lens) + pad
    # one layer's cache per sampled layer; lengths as in the workload
    base16 = rng.standard_normal(1 << 22, dtype=np.float32).astype(np.float16).view(np.uint16)

    def rows16(shape):
        """fp16 N(0,1) rows: a 4M-element seeded block repeated (the values do not change the work done)."""
        return np.resize(base16, int(np.prod(shape))).reshape(shape)

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
        return [dict(k=rows16((lens[b] + pad, Hkv, D)), v=rows16((lens[b] + pad, Hkv, D))) for b in range(B)]

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
        "scaling": "strong" if (args.shard == "heads" or args.gpus == 1) else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(w, lens, args.gpus, args.shard == "heads", args),
        "implementation": "CPU restatement of the reference path (oracle/er_oracle.c), OpenMP over heads, on rank 0's host cores; the "
                          "reference's Swift/Metal sources cannot be built in this environment",
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
    elif w["precision"] in ("balanced", "aggressive"):
        prec = er.Precision.turboQuantBalanced if w["precision"] == "balanced" else er.Precision.turboQuantAggressive
        cache = er.KVCache(cap, L, Hkv, D, prec, max_batch=B, layout=layout, key_residual_scale=w.get("residual_scale", 0.0),
                           value_residual_scale=w.get("residual_scale", 0.0), decode_kernel=w.get("decode_kernel", 0), **kw)
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


class Context:
    """Process-wide handles of a GPU run: torch, torch.distributed, the package, rank layout, the launch stream."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        import edgerunner_b200 as er
        self.torch, self.dist, self.er = torch, dist, er
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if args.gpus > 1 and self.world != args.gpus:
            raise SystemExit("--gpus %d needs torchrun with %d ranks (WORLD_SIZE=%d)" % (args.gpus, args.gpus, self.world))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        from edgerunner_b200.sharding import max_over_ranks
        return max_over_ranks(x, device="cuda")


def measure_decode(cx, args, w_full, lens, K, W, repeats, shard_heads, extras=()):
    """Times the decode step of one workload on this process's GPU (and, with shard_heads, its peers).  Returns the
    figures of the JSON line as a dict; rank-local values are already reduced (max over ranks) where the contract says so."""
    torch, dist, er = cx.torch, cx.dist, cx.er
    from edgerunner_b200.sharding import HeadShardedDecoder
    world, rank = (cx.world, cx.rank) if shard_heads or args.shard == "sequence" else (1, 0)
    sharded = shard_heads and world > 1
    w = dict(w_full, heads=w_full["heads"] // world, kv_heads=w_full["kv_heads"] // world) if sharded else dict(w_full)
    if sharded and w_full["kv_heads"] % world:
        raise SystemExit("--shard heads needs kv_heads %% gpus == 0")
    L, B, H, Hkv = w["layers"], len(lens), w["heads"], w["kv_heads"]
    Hfull = w_full["heads"]
    sp = er.step_params(rope_theta=w["theta"])
    cache = build_cache(er, torch, w, lens, K + W + 8)
    fill_cache(er, torch, cache, w, lens, sp, seed=1000 + rank)
    dec = HeadShardedDecoder(cache, L, B, Hfull, w_full["kv_heads"], world if sharded else 1, rank if sharded else 0,
                             exchange=args.exchange) if shard_heads else None
    stream = cx.stream

    def set_start():
        for b, n in enumerate(lens):
            cache.set_position(n, seq=b)

    g = torch.Generator(device="cuda")
    g.manual_seed(5 + rank)
    pool = min(K + W, 24 if L * B * H > 32768 else 64)   # distinct per-step inputs, cycled (a step's cost does not depend on their values)
    qs = torch.randn((pool, L, B, H, D), generator=g, device="cuda").half().float()
    ks = torch.randn((pool, L, B, Hkv, D), generator=g, device="cuda").half().float()
    vs = torch.randn((pool, L, B, Hkv, D), generator=g, device="cuda").half().float()
    out = dec.full if dec is not None else torch.empty((L, B, H, D), device="cuda", dtype=torch.float32)

    # raw addresses of every (step, layer) slice: one call per layer must not pay for tensor slicing in the interpreter
    layer_ptrs = None
    if not sharded and (w.get("per_layer") or "per_layer" in extras):
        layer_ptrs = [[(qs[i, l].data_ptr(), ks[i, l].data_ptr(), vs[i, l].data_ptr(), out[l].data_ptr()) for l in range(L)] for i in range(pool)]
    stream_raw = stream.cuda_stream

    def per_layer_step(i, on=None):
        on = stream_raw if on is None else on
        for l in range(L):
            a = layer_ptrs[i][l]
            cache.decode_step(a[0], a[1], a[2], a[3], H, sp, layer_begin=l, layer_end=l + 1, stream=on)

    def step(i, exchange=True):
        if w.get("per_layer") and not sharded:
            per_layer_step(i)
        elif dec is not None:
            dec.step(qs[i], ks[i], vs[i], sp, stream=stream, exchange=exchange)
        else:
            cache.decode_step(qs[i], ks[i], vs[i], out, H, sp, stream=stream)

    def timed_regions(n, exchange=True):
        """n regions of K steps (after W warm-up steps each, positions rewound): per-region ms, max over ranks."""
        ms, launches = [], None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(n):
            set_start()
            for s in range(W):
                step(s % pool, exchange)
            cx.barrier()
            l0 = er.lib().er_kernel_launch_count()
            e0.record(stream)
            for s in range(K):
                step((W + s) % pool, exchange)
            e1.record(stream)
            cx.barrier()
            if launches is None:
                launches = int(er.lib().er_kernel_launch_count() - l0)
            ms.append(cx.max_over_ranks(e0.elapsed_time(e1)) if (sharded or args.shard == "sequence") else e0.elapsed_time(e1))
        return ms, launches

    # ---- leg 1: device-resident inputs, whole step (and the exchange) inside the timed region ----
    sampler = ClockSampler(cx.local_rank)
    if rank == 0:
        sampler.start()
    regions, launches = timed_regions(repeats)
    ms_region = statistics.median(regions)
    for b, n in enumerate(lens):
        assert cache.total_written(0, b) == n + W + K
    compute_regions = None
    if sharded:      # the same steps without the exchange (and without the peer stores): the rank's own compute
        dec.set_peer_stores(False)
        compute_regions, _ = timed_regions(max(3, repeats // 2 + 1), exchange=False)
        dec.set_peer_stores(True)
    # load window for the clock samples: the same steps again for about a second
    t_load = time.perf_counter()
    while rank == 0 and not sharded and time.perf_counter() - t_load < 1.0:
        set_start()
        for s in range(min(K + W, 64)):
            step(s % pool)
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    assert cache.device_status() == 0, "device status word is set (timeout / out of pages)"
    replicas = cx.world if (args.shard == "sequence" and not shard_heads) else 1
    tokens = B * K * replicas
    value = tokens / (ms_region * 1e-3)
    bytes_region = sum(step_bytes(w, lens, W + s) for s in range(K))        # this GPU's rows
    ms_compute = statistics.median(compute_regions) if compute_regions else ms_region
    hbm_gbs = bytes_region / (ms_compute * 1e-3) / 1e9
    res = {"value": value, "ms_per_step": ms_region / K, "regions_ms": [round(x, 4) for x in regions], "gpu_launches": launches,
           "hbm_gbs_per_gpu": round(hbm_gbs, 1), "clocks": clocks, "tokens_per_region": tokens}
    if sharded:
        res["exchange"] = {"kind": dec.exchange, "compute_only_ms_per_step": ms_compute / K,
                           "share_of_step": round(max(0.0, 1.0 - ms_compute / ms_region), 4),
                           "payload_bytes_per_gpu_per_step": L * B * H * D * 4 * (world - 1),
                           "note": ("peer stores from the decode kernel's merge epilogue into every GPU's [layers, batch, heads, 128] buffer "
                                    "+ one 4-byte NCCL all-reduce behind the launch" if dec.exchange == "p2p" else
                                    "NCCL all-gather of [layers, batch, heads / N, 128] + re-layout kernel")}
        if getattr(dec, "p2p_refused", None):
            res["exchange"]["p2p_refused"] = dec.p2p_refused

    if args.only_device_leg:
        if args.cta_timeline and rank == 0:
            n_ctas = cache.set_trace(None, 0)
            stamps = torch.zeros(n_ctas, 8, dtype=torch.int64, device="cuda")
            cache.set_trace(stamps, n_ctas)
            set_start()
            step(0)
            torch.cuda.synchronize()
            cache.set_trace(None, 0)
            t = stamps.cpu().numpy().astype(np.float64)
            t = (t - t[:, 0].min()) / 1e3
            names = ["cta_start", "work_list_built", "first_tile_landed", "streaming_done", "before_exit_sync", "after_exit_sync", "cta_end"]
            res["cta_timeline_us"] = {nm: [round(float(f(t[:, i])), 2) for f in (np.min, np.median, np.max)] for i, nm in enumerate(names)}
        _close(dec, cache)
        return res

    # ---- roofline of the attention kernel ----
    peak, peak_src = measured_peaks()
    # fp16 rows: the timed region is K launches of the one fused kernel (plus K re-layout launches behind an NCCL all-gather)
    fused_single_launch = launches == K or (sharded and dec.exchange == "nccl" and w["precision"] == "float16" and launches == 2 * K)
    t_append = 0.0
    kernel_name = "simt_decode_kernel" if w.get("decode_kernel") == 3 else "flash_decode_kernel"
    if w.get("per_layer") and launches == K * L:
        # one fused launch per layer: the region's time over its K * L launches
        t_attn, attn_bytes, timed_as = ms_compute / (K * L), bytes_region / (K * L), "the K x layers launches of the timed region, back to back on one stream"
        split_attn_ms, kernel_name = None, "decode_slim_kernel"
    elif fused_single_launch:
        t_attn, attn_bytes, timed_as = ms_compute / K, bytes_region / K, "the K launches of the timed region (append fused into the kernel)"
        split_attn_ms = None
    else:
        # q8_0 / TurboQuant rows: append kernel + attention kernel; the attention launch between per-step events
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
        t_append = statistics.median(e[0].elapsed_time(e[1]) for e in evs)
        t_attn = statistics.median(e[1].elapsed_time(e[2]) for e in evs)
        attn_bytes = statistics.mean(step_bytes(w, lens, W + s) for s in range(n_probe)) - B * Hkv * row_bytes(w) * L
        split_attn_ms, timed_as = t_attn, "attention launch between per-step CUDA events (split entry points), median"
    achieved = attn_bytes / (t_attn * 1e-3) / 1e9
    ratio = NCU_TRAFFIC_RATIO.get("%s/group%d" % (w["precision"], H // Hkv))
    res["roofline"] = {"bound": "hbm", "kernel": kernel_name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                       "frac": round(achieved / peak, 4),
                       "traffic": int(attn_bytes * ratio[0]) if ratio else None,
                       "traffic_source": ("algorithmic bytes x %.4f, the DRAM-traffic ratio of the ncu capture in %s" % ratio) if ratio else None,
                       "peak_source": peak_src, "algorithmic_bytes_per_launch": int(attn_bytes), "launch_ms": round(t_attn, 5),
                       "append_kernel_ms": round(t_append, 5), "frac_of_8tbs": round(achieved / 8000.0, 4), "timed_as": timed_as,
                       "per_gpu": True}
    if split_attn_ms is not None:
        res["roofline"]["split_call_attention_launch_ms"] = round(split_attn_ms, 5)

    # ---- end to end: this step's q/k/v from pinned host memory, the result back to the host, every step ----
    if "e2e" in extras:
        hq = torch.empty((pool, L, B, H, D), dtype=torch.float32).pin_memory().copy_(qs.cpu())
        hk = torch.empty((pool, L, B, Hkv, D), dtype=torch.float32).pin_memory().copy_(ks.cpu())
        hv = torch.empty((pool, L, B, Hkv, D), dtype=torch.float32).pin_memory().copy_(vs.cpu())
        hout = torch.empty((L, B, Hfull if dec is not None else H, D), dtype=torch.float32).pin_memory()
        hout_np = hout.numpy()
        if dec is None or not sharded:
            # one GPU: the host-buffer entry point of the C ABI (raw addresses: slicing tensors per step would add tens of
            # microseconds of interpreter time to a step)
            if dec is not None:
                dec.close()
                dec = None
            hq_p, hk_p, hv_p = [hq[i].data_ptr() for i in range(pool)], [hk[i].data_ptr() for i in range(pool)], [hv[i].data_ptr() for i in range(pool)]
            hout_p, stream_p = hout.data_ptr(), stream.cuda_stream

            def host_step(i):
                cache.decode_step_host(hq_p[i], hk_p[i], hv_p[i], hout_p, H, sp, stream=stream_p)
            entry = "er_kv_decode_step_host"
        else:
            hout = torch.empty((L, B, H, D), dtype=torch.float32).pin_memory()      # this rank's heads; the ranks' buffers together = the result
            hout_np = hout.numpy()

            def host_step(i):
                dec.step_host(hq[i], hk[i], hv[i], hout if dec.exchange != "p2p" else None, sp, stream=stream)
            entry = ("HeadShardedDecoder.step_host: pinned host q/k/v slices in (pulled by the decode kernel), exchange on the device, "
                     "every rank's own heads [layers, batch, heads / N, 128] out to pinned host memory")
        e2e_regions = []
        checksum = 0.0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(max(3, repeats // 2 + 1)):
            set_start()
            for s in range(W):
                host_step(s % pool)
            cx.barrier()
            e0.record(stream)
            t0 = time.perf_counter()
            for s in range(K):
                host_step((W + s) % pool)
                checksum += float(hout_np[0, 0, 0, 0]) if (dec is None or dec.host_rows is None) else float(dec.host_rows[0, 0, 0, 0])   # the host reads the step's result
            e1.record(stream)
            cx.barrier()
            wall_ms = (time.perf_counter() - t0) * 1e3
            x = max(e0.elapsed_time(e1), wall_ms)
            e2e_regions.append(cx.max_over_ranks(x) if sharded else x)
        assert math.isfinite(checksum)
        e2e_ms = statistics.median(e2e_regions)
        res["e2e"] = {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                      "h2d_bytes_per_step": int(hq[0].numel() + hk[0].numel() + hv[0].numel()) * 4 * (world if sharded else 1),
                      "d2h_bytes_per_step": int(hout.numel()) * 4 * (world if sharded else 1), "entry_point": entry,
                      "regions_ms": [round(x, 4) for x in e2e_regions]}

    # ---- one launch per layer (how a model that interleaves its own projections calls it), plain launches and replayed
    #      as a CUDA graph of the layer launches (positions live on the device, so one captured step replays for every
    #      following step) ----
    if "per_layer" in extras and dec is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
        pl_ms = e0.elapsed_time(e1) / n_pl
        res["per_layer_launch"] = {"tokens_per_s": B / (pl_ms * 1e-3), "us_per_layer_launch": round(pl_ms * 1e3 / L, 3)}
        try:
            set_start()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                per_layer_step(0, side.cuda_stream)    # warm the capture stream
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                per_layer_step(0, torch.cuda.current_stream().cuda_stream)
            set_start()
            for _ in range(4):
                graph.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(n_pl):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            g_ms = e0.elapsed_time(e1) / n_pl
            assert cache.total_written(0, 0) == lens[0] + 4 + n_pl
            res["per_layer_launch"]["cuda_graph_tokens_per_s"] = B / (g_ms * 1e-3)
            res["per_layer_launch"]["cuda_graph_us_per_layer_launch"] = round(g_ms * 1e3 / L, 3)
        except Exception as exc:   # graph capture is an optional extra figure
            res["per_layer_launch"]["cuda_graph_tokens_per_s"] = "unavailable: %s" % (str(exc).splitlines()[0][:120] if str(exc) else type(exc).__name__)

    _close(dec, cache)
    del qs, ks, vs
    torch.cuda.empty_cache()
    return res


def _close(dec, cache):
    if dec is not None:
        dec.close()
    cache.close()


def config_of(w, lens, world, shard_heads, args):
    return {"workload": w["name"], "layers": w["layers"], "batch": len(lens), "q_heads": w["heads"], "kv_heads": w["kv_heads"],
            "head_dim": D, "kv_storage": w["precision"], "layout": w["layout"],
            "launch": "layer-batched: one persistent attention launch per step for all layers (fp16 rows: the append is fused into it; "
                      "q8_0 / TurboQuant rows: one append launch first)",
            "sharding": ("kv heads split over the %d GPUs (%d kv heads each); every GPU ends a step with all heads' outputs, exchange "
                         "inside the timed region" % (world, w["kv_heads"] // world)) if (shard_heads and world > 1) else
                        ("by sequence, one replica of the workload per GPU, no collective" if world > 1 else "single GPU, all kv heads"),
            "l2": "cache bytes read per step per GPU (%.0f MB) exceed the 126 MB L2; no flush needed" % (step_bytes(w, lens, 0) / max(world if shard_heads else 1, 1) / 1e6),
            "timing": "median of %d timed regions of %d steps, CUDA events, max over ranks" % (args.repeats, args.steps)}


def run_ours(args, w, lens):
    cx = Context(args)
    torch, dist = cx.torch, cx.dist
    K, W = args.steps, max(args.warmup, 0)
    shard_heads = args.shard == "heads"
    sharded = shard_heads and cx.world > 1
    verified = None
    if sharded:
        from edgerunner_b200.sharding import verify_exchange
        # parity first: the exchanged [layers, batch, heads, 128] tensor of a small paged case, bit for bit against the
        # shards computed on this rank's own GPU (raises on any difference)
        verified = verify_exchange(cx.er, cx.world, cx.rank, args.exchange)
    extras = () if args.only_device_leg else ("e2e",) + (("per_layer",) if w["batch"] == 1 and not sharded else ())
    res = measure_decode(cx, args, w, lens, K, W, args.repeats, shard_heads, extras)

    legs = {}
    leg_names = args.legs
    if leg_names is None:
        leg_names = "cfg1,cfg2" if (args.workload == DEFAULT_WORKLOAD and cx.world == 1 and not args.only_device_leg) else ""
    for name in [x for x in leg_names.split(",") if x]:
        if cx.world > 1:
            break                       # the other configurations are single-GPU figures
        lw = WORKLOADS[name]
        llens = sequence_lengths(lw)
        lk = max(K, 100) if lw["batch"] == 1 else K        # a cfg1 step is ~80 us: 100 steps per region
        r = measure_decode(cx, args, lw, llens, lk, max(W, 8), args.repeats, False, ("e2e",) + (("per_layer",) if lw["batch"] == 1 else ()))
        legs[name] = {"config": {"workload": lw["name"]}, "value": r["value"], "unit": "tokens/s", "ms_per_step": r["ms_per_step"],
                      "steps": lk, "regions_ms": r["regions_ms"], "hbm_gbs": r["hbm_gbs_per_gpu"], "roofline": r.get("roofline"),
                      "e2e": r.get("e2e"), "gpu_launches": r["gpu_launches"], **({"per_layer_launch": r["per_layer_launch"]} if "per_layer_launch" in r else {})}

    cpu = None
    if cx.rank == 0 and cx.world == 1 and not args.no_cpu_baseline and not args.only_device_leg and w["precision"] not in ("balanced", "aggressive"):
        r = cpu_reference_leg(w, lens, args.cpu_seconds)
        cpu = {"value": r["value"], "unit": "tokens/s", "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]}

    if cx.rank == 0:
        line = {
            "metric": METRIC, "value": res["value"], "unit": "tokens/s", "n_gpus": cx.world, "steps": K, "warmup": W,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if (shard_heads or cx.world == 1) else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": config_of(w, lens, cx.world, shard_heads, args),
            "repeats": args.repeats, "regions_ms": res["regions_ms"],
            "hbm_gbs_per_gpu": res["hbm_gbs_per_gpu"], "frac_of_8tbs": round(res["hbm_gbs_per_gpu"] / 8000.0, 4),
            "roofline": res.get("roofline"), "cpu_baseline": cpu, "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches"],
            "clocks": res["clocks"],
        }
        if "exchange" in res:
            line["exchange"] = dict(res["exchange"], verified_before_timing="exchanged outputs of a small paged case equal the per-shard "
                                    "reference bit for bit on every rank (%s)" % verified)
        if "per_layer_launch" in res:
            line["per_layer_launch"] = res["per_layer_launch"]
        if "cta_timeline_us" in res:
            line["cta_timeline_us"] = res["cta_timeline_us"]
        if args.only_device_leg:
            line["note"] = "device leg only"
        if legs:
            line["legs"] = legs
        print(json.dumps(line))
    if cx.world > 1:
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


PAIR_SIDES = {   # cache arguments and cached bytes per (token, kv head) of one side
    "float16": (lambda er: dict(precision=er.Precision.float16, layout=er.Layout.head_major), 256),
    "q8_0": (lambda er: dict(precision=er.Precision.q8_0), 136),
    "turbo2": (lambda er: dict(precision=er.Precision.turboquantV2, key_type=2, value_type=2, norm_format=er.NormFormat.float16), 34),
    "turbo3": (lambda er: dict(precision=er.Precision.turboquantV2, key_type=3, value_type=3, norm_format=er.NormFormat.float16), 50),
    "turbo4": (lambda er: dict(precision=er.Precision.turboquantV2, key_type=4, value_type=4, norm_format=er.NormFormat.float16), 66),
}


def run_pair(args, w):
    """Decode attention of layers whose keys and values live in two caches of different row formats (er_kv_attention_decode_pair):
    step = one attention launch over all layers and sequences of the workload, rows resident; achieved = the cached bytes of the
    key side of one cache and the value side of the other, per launch, over CUDA-event time."""
    import torch
    import edgerunner_b200 as er
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    L, B, H, Hkv, ctx = w["layers"], w["batch"], w["heads"], w["kv_heads"], w["ctx"]
    (kargs, kbytes), (vargs, vbytes) = PAIR_SIDES[w["keys"]], PAIR_SIDES[w["values"]]
    dk = 3 if w.get("simt") else 0
    mk = lambda side: er.KVCache(ctx + 64, L, Hkv, D, side(er).pop("precision"), max_batch=B, decode_kernel=dk,
                                 **{k_: v_ for k_, v_ in side(er).items() if k_ != "precision"})
    kc, vc = mk(kargs), mk(vargs)
    sp = er.step_params(rope_theta=w["theta"])
    g = torch.Generator(device="cuda").manual_seed(5)
    for cache in (kc, vc):
        for l in range(L):
            for b in range(B):
                for s0 in range(0, ctx, 8192):
                    n = min(8192, ctx - s0)
                    cache.write_rows(l, b, s0, n, torch.randn((n, Hkv, D), device="cuda", generator=g).half().float(),
                                     torch.randn((n, Hkv, D), device="cuda", generator=g).half().float(), sp)
    q = torch.randn((L, B, H, D), device="cuda", generator=g).half().float()
    out = torch.empty_like(q)
    K, W = args.steps, max(args.warmup, 0)
    for _ in range(W):
        kc.attention_decode_with_values_of(vc, q, out, H, sp)
    torch.cuda.synchronize()
    launches0 = er.lib().er_kernel_launch_count()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        kc.attention_decode_with_values_of(vc, q, out, H, sp)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    assert kc.device_status() == 0
    ms = e0.elapsed_time(e1) / K
    nbytes = L * B * Hkv * ctx * (kbytes + vbytes) + 2 * L * B * H * D * 4
    peak, peak_src = measured_peaks()
    achieved = nbytes / ms / 1e6
    print(json.dumps({
        "metric": "decode_attention_launches_per_s", "value": round(1e3 / ms, 2), "unit": "launches/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["name"], "layers": L, "batch": B, "q_heads": H, "kv_heads": Hkv, "context": ctx, "keys": w["keys"],
                   "values": w["values"], "kernel": "simt_decode_kernel" if dk else "flash_decode_kernel"},
        "roofline": {"bound": "hbm", "kernel": "simt_decode_kernel" if dk else "flash_decode_kernel", "achieved": round(achieved, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": int(nbytes)},
        "gpu_launches": int(er.lib().er_kernel_launch_count() - launches0), "clocks": clocks}))


def run_cfg4(args):
    """benchmark contract, configuration [4]: Qwen3-4B shape (36 layers, 32 q / 8 kv heads), TurboQuant turbo4 K / turbo4 V rows with fp16 norms in
    64-token pages, sequences at context 131072: ONE chunked-prefill step that appends 2048 tokens per sequence (causal,
    tensor-core kernel, every layer), then 128 decode steps.  GPUs are split by sequence x kv-head group: pairs of GPUs
    share 4 sequences and hold 4 kv heads each (outputs exchanged inside the pair); one GPU alone runs 2 sequences with all
    heads -- the same 10 GB of codes per GPU at every N, so `scaling` is weak and `value` counts all sequences."""
    cx = Context(args)
    torch, dist, er = cx.torch, cx.dist, cx.er
    from edgerunner_b200.sharding import HeadShardedDecoder, HeadShard
    w = WORKLOADS["cfg4"]
    L, Hfull, Hkv_full, ctx, chunk, ps = w["layers"], w["heads"], w["kv_heads"], w["ctx"], w["chunk"], w["page_size"]
    steps = args.steps if args.steps != 20 else w["decode_steps"]       # 128 unless --steps says otherwise
    head_groups = 2 if cx.world > 1 else 1
    if cx.world > 1 and cx.world % 2:
        raise SystemExit("cfg4 needs 1 GPU or an even number of GPUs (pairs share sequences)")
    pair = cx.rank // head_groups
    B = 2 if cx.world == 1 else 4
    total_seqs = B * max(cx.world // head_groups, 1)
    group = None
    if cx.world > 1:
        groups = [dist.new_group([2 * g, 2 * g + 1]) for g in range(cx.world // 2)]
        group = groups[pair]
    shard = HeadShard(Hfull, Hkv_full, head_groups, cx.rank % head_groups)
    H, Hkv = shard.local_heads, shard.local_kv_heads
    T = ctx + chunk + steps + 8
    pages_per_seq = (T + ps - 1) // ps
    cache = er.KVCache(T, L, Hkv, D, er.Precision.turboquantV2, key_type=w["kbits"], value_type=w["vbits"], norm_format=er.NormFormat.float16,
                       max_batch=B, layout=er.Layout.paged, page_size=ps, num_pages=pages_per_seq * B)
    rng = np.random.Generator(np.random.PCG64(2 + pair))
    alloc = er.BlockTableAllocator(pages_per_seq * B, ps, free_order=rng.permutation(pages_per_seq * B))
    for b in range(B):
        cache.set_block_table(b, alloc.ensure(b, T))
    sp = er.step_params(rope_theta=w["theta"])
    g = torch.Generator(device="cuda")
    g.manual_seed(100 + cx.rank)
    for l in range(L):
        for b in range(B):
            for s0 in range(0, ctx, 16384):
                n = min(16384, ctx - s0)
                cache.write_rows(l, b, s0, n, torch.randn((n, Hkv, D), generator=g, device="cuda").half().float(),
                                 torch.randn((n, Hkv, D), generator=g, device="cuda").half().float(), sp)
    torch.cuda.synchronize()
    stream = cx.stream
    # ---- the prefill step: per layer and sequence, append the chunk's K / V rows, then causal attention of its 2048 query rows ----
    kc = torch.randn((chunk, Hkv, D), generator=g, device="cuda").half().float()
    vc = torch.randn((chunk, Hkv, D), generator=g, device="cuda").half().float()
    qc = torch.randn((chunk, H, D), generator=g, device="cuda").half().float()
    oc = torch.empty((chunk, H, D), device="cuda")
    og = torch.empty((head_groups, chunk, H, D), device="cuda") if cx.world > 1 else None
    # untimed warm-up: the pair's communicator is created at its first collective (hundreds of ms), and the first chunk loads
    # the kernels; the chunk written here is written again, to the same rows, by the timed loop
    cache.write_rows(0, 0, ctx, chunk, kc, vc, sp, stream=stream)
    cache.attention_prefill(0, 0, qc, oc, H, chunk, sp, stream=stream)
    if og is not None:
        dist.all_gather_into_tensor(og, oc, group=group)
    torch.cuda.synchronize()
    cx.barrier()
    sampler = ClockSampler(cx.local_rank)
    if cx.rank == 0:
        sampler.start()
    launches0 = er.lib().er_kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for l in range(L):
        for b in range(B):
            cache.write_rows(l, b, ctx, chunk, kc, vc, sp, stream=stream)
            cache.attention_prefill(l, b, qc, oc, H, chunk, sp, stream=stream)
            if og is not None:
                dist.all_gather_into_tensor(og, oc, group=group)      # the pair ends the chunk with all heads' rows
    e1.record(stream)
    cx.barrier()
    prefill_ms = cx.max_over_ranks(e0.elapsed_time(e1))
    prefill_launches = int(er.lib().er_kernel_launch_count() - launches0)
    flops_rank = 4.0 * chunk * (ctx + (chunk + 1) / 2.0) * H * D * L * B
    # ---- 128 decode steps ----
    dec = HeadShardedDecoder(cache, L, B, Hfull, Hkv_full, head_groups, cx.rank % head_groups, exchange=args.exchange, group=group)
    pool = 8
    qs = torch.randn((pool, L, B, H, D), generator=g, device="cuda").half().float()
    ks = torch.randn((pool, L, B, Hkv, D), generator=g, device="cuda").half().float()
    vs = torch.randn((pool, L, B, Hkv, D), generator=g, device="cuda").half().float()
    for s in range(max(args.warmup, 1)):
        dec.step(qs[s % pool], ks[s % pool], vs[s % pool], sp, stream=stream)
    for b in range(B):
        cache.set_position(ctx + chunk, seq=b)
    cx.barrier()
    launches0 = er.lib().er_kernel_launch_count()
    e0.record(stream)
    for s in range(steps):
        dec.step(qs[s % pool], ks[s % pool], vs[s % pool], sp, stream=stream)
    e1.record(stream)
    cx.barrier()
    decode_ms = cx.max_over_ranks(e0.elapsed_time(e1))
    decode_launches = int(er.lib().er_kernel_launch_count() - launches0)
    clocks = sampler.stop() if cx.rank == 0 else None
    assert cache.device_status() == 0
    wl = dict(w, precision="turboquant", heads=H, kv_heads=Hkv, norm="float16")
    lens = [ctx + chunk] * B
    dec_bytes = sum(step_bytes(wl, lens, s) for s in range(steps))
    peak, peak_src = measured_peaks()
    tpeak = None
    try:
        tpeak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
    except Exception:
        pass
    if cx.rank == 0:
        total_ms = prefill_ms + decode_ms
        tokens = total_seqs * (chunk + steps)
        print(json.dumps({
            "metric": METRIC, "value": tokens / (total_ms * 1e-3), "unit": "tokens/s", "n_gpus": cx.world, "steps": steps, "warmup": args.warmup,
            "ms_per_step": decode_ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "layers": L, "sequences": total_seqs, "sequences_per_gpu_group": B, "q_heads": Hfull, "kv_heads": Hkv_full,
                       "sharding": ("%d sequence groups x %d kv-head groups; outputs exchanged inside each pair of GPUs" % (cx.world // head_groups, head_groups))
                       if cx.world > 1 else "single GPU: 2 sequences, all kv heads (one GPU's share of the 8-GPU split)",
                       "value_is": "all tokens of the job (prefill chunk + decode steps) over prefill time + decode time"},
            "prefill": {"ms": prefill_ms, "tflops_per_gpu": round(flops_rank / prefill_ms / 1e9, 1), "peak_tflops_sustained": tpeak,
                        "frac_of_sustained_bf16": round(flops_rank / prefill_ms / 1e9 / tpeak, 4) if tpeak else None,
                        "chunk_tokens_per_s": total_seqs * chunk / (prefill_ms * 1e-3), "gpu_launches": prefill_launches,
                        "note": "useful FLOPs 4 S (ctx + (S+1)/2) Hq 128 per layer and sequence; includes the chunk's append and the expansion of "
                                "the sequence's codes to fp16 hi + lo rows that the tensor-core kernel reads"},
            "decode": {"ms_per_step": decode_ms / steps, "tokens_per_s": total_seqs * steps / (decode_ms * 1e-3),
                       "hbm_gbs_per_gpu": round(dec_bytes / (decode_ms * 1e-3) / 1e9, 1), "frac_of_measured_copy_peak": round(dec_bytes / (decode_ms * 1e-3) / 1e9 / peak, 4),
                       "peak_source": peak_src, "gpu_launches": decode_launches, "exchange": dec.exchange},
            "gpu_launches": prefill_launches + decode_launches, "clocks": clocks}))
    dec.close()
    cache.close()
    if cx.world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    w = WORKLOADS[args.workload]
    if args.workload == "cfg4":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "cfg4 is measured on the GPU path only (the CPU leg runs the default workload)"}))
            return
        run_cfg4(args)
        return
    if w.get("prefill") or w.get("keys"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the prefill and cache-pair workloads are measured on the GPU path only"}))
            return
        (run_prefill if w.get("prefill") else run_pair)(args, w)
        return
    lens = sequence_lengths(w)
    if args.impl == "reference":
        run_reference_impl(args, w, lens)
    else:
        run_ours(args, w, lens)


if __name__ == "__main__":
    main()
