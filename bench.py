"""Benchmark of the codec-frame token loop: Qwen3-TTS-1.7B talker architecture, random bf16 weights,
64 concurrent sessions per GPU, one decode tick (talker step + 15 code-predictor sub-steps) per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0). `value`: codec frames/s over all GPUs with every tick's inputs already in HBM
(`omni_talker_run_ticks`), timed per tick with CUDA events on the model's stream, max over ranks. `e2e`: the same
metric through the public `Model.step` call with host draws (H2D staging and D2H frame read-back inside each step).
`--impl reference` times the reference's own implementation of this path: it is CUDA-only (no CPU decode exists in
the reference), so the arm runs the reference's kernels — compiled from its sources into oracle/_ref — sequenced as
its manifest emits them with cuBLAS GEMMs, one CUDA graph per tick, on every rank's GPU with the same sessions and
positions. `cpu_baseline` (rank 0, N = 1) is the CPU restatement on all host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "codec frames/sec at 64 sessions per GPU (Qwen3-TTS talker)"
UNIT = "frames/s"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.t0 = self.t1 = None

    def mark_start(self):
        """The timed region begins now: only samples read between the two marks are summarised."""
        self.t0 = time.monotonic()

    def mark_end(self):
        self.t1 = time.monotonic()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()  # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # a sample is printed up to one period after it was taken: keep those read inside the timed window, widened by
        # one period at the end; when the window is shorter than the sampling period, the nearest sample after its start
        rows = [r for t, r in self.rows if self.t0 is None or (self.t0 <= t <= (self.t1 or t) + 0.06)]
        if not rows and self.rows and self.t0 is not None:
            later = [r for t, r in self.rows if t >= self.t0]
            rows = later[:1] or [self.rows[-1][1]]
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def workload(cfg, sessions, prompt_len, seed):
    from pega_omni_b200.model import Prompt
    rng = np.random.default_rng(seed)
    # 128-token prompts, uniform text ids, no codec-track tokens (NO_CODEC on every row)
    return [Prompt(list(rng.integers(0, cfg.text_vocab_size, prompt_len)), [-1] * prompt_len) for _ in range(sessions)]


def draws_for(ticks, sessions, seed):
    from pega_omni_b200.model import Draw
    rng = np.random.default_rng(seed)
    u = rng.random((ticks, sessions, 16)).astype(np.float32)
    return [[Draw(list(u[t, s])) for s in range(sessions)] for t in range(ticks)]


def replay_baseline(cfg, ck, sessions, prompt_len, warmup, steps, seed=0, clocks=None):
    """The reference's own kernels (compiled for sm_100a into oracle/_ref) sequenced as its manifest does, GEMMs on
    cuBLAS, one CUDA graph per tick like its `decode` program: the 'reference build on the same box'. Returns None
    when the cubins are not there. Timing: CUDA events around `steps` graph replays on torch's current stream."""
    import torch
    from oracle import ref_kernels
    if not ref_kernels.available():
        return None
    rng = np.random.default_rng(seed)
    prompts = workload(cfg, sessions, prompt_len, seed=seed)
    r = ref_kernels.RefTalker(cfg, ck, sessions, prompt_len + warmup + steps + 8)
    free = np.full((sessions, 16), -1, dtype=np.int32)
    r.start(prompts, rng.random((sessions, 16)).astype(np.float32), free)
    for _ in range(max(3, warmup)):
        r.step(rng.random((sessions, 16)).astype(np.float32), free, graph=True)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    us = [rng.random((sessions, 16)).astype(np.float32) for _ in range(steps)]
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.mark_start()
    ev[0].record()
    for t in range(steps):
        r._stage(us[t], free)
        r.graph.replay()
        r.n_frames += 1
        ev[t + 1].record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.mark_end()
    ms = np.array([ev[t].elapsed_time(ev[t + 1]) for t in range(steps)])
    return {"value": sessions * steps / (ms.sum() * 1e-3), "unit": UNIT, "ms_per_step": float(ms.mean()),
            "elapsed_s": float(ms.sum()) * 1e-3, "h2d_bytes_per_step": int(2 * sessions * 16 * 4),
            "tick_p99_ms": float(np.percentile(ms, 99)), "graph_nodes": int(r.graph_nodes),
            "what": "reference qwen3.cu + talker.cu kernels (sm_100a cubins) + cuBLAS bf16 GEMMs, one CUDA graph per "
                    "tick, no codec tail; input staging copies inside the timed region"}


def cpu_baseline(cfg, ck_host, threads=None, sessions=4, prompt_len=16, warmup=1, ticks=4, seed=0):
    """The CPU oracle (a port of the reference's arithmetic) timed on a bounded sample of the same architecture:
    `sessions` sessions, short prompts, `ticks` decode ticks. Returns frames/s, cores used, per-tick seconds."""
    from oracle import cpu as orc
    lib = orc.load()
    # every host core, asked for by name: a launcher may have set OMP_NUM_THREADS=1 in this process's environment
    lib.orc_set_threads(threads or os.cpu_count() or 1)
    cores = lib.orc_max_threads()
    o = orc.CpuOracle(cfg, ck_host)
    prompts = workload(cfg, sessions, prompt_len, seed)
    sids = [o.open(prompt_len, warmup + ticks + 2) for _ in range(sessions)]
    d = draws_for(warmup + ticks + 1, sessions, seed)
    o.start(sids, prompts, d[0])
    for t in range(warmup):
        o.step(sids, d[1 + t])
    per_tick = []
    for t in range(ticks):
        t0 = time.perf_counter()
        o.step(sids, d[1 + warmup + t])
        per_tick.append(time.perf_counter() - t0)
    o.close()
    total = sum(per_tick)
    return {"value": sessions * ticks / total, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{sessions} sessions x {ticks} decode ticks of the same architecture, {prompt_len}-token "
                      f"prompts (the GPU workload runs 64 sessions x 128-token prompts)"}, per_tick


CONFIG_WORKLOAD = ("configs[1]: Qwen3-TTS-12Hz-1.7B talker (28L h2048 16q/8kv d128 i6144, head 3072) + "
                   "code predictor (5L h1024, 15 codebooks x 2048), random bf16 weights N(0,0.02)")


def run_reference(args, rank, world, local):
    """The reference arm: the reference's own kernels on this rank's GPU (see replay_baseline), the same sessions,
    prompts and positions as the library's arm; every rank runs its replica, the time is the max over ranks. Rank 0
    prints the line. With N = 1 the line also carries the CPU restatement's number (`cpu_baseline`)."""
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device: the reference's path is CUDA-only"}))
        return
    from oracle import ref_kernels
    if not ref_kernels.available():
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref holds no reference cubins (built from "
                              "the reference checkout by __graft_entry__.build())"}))
        return
    from pega_omni_b200.config import presets
    from pega_omni_b200.synthetic import random_checkpoint
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    W, K = max(3, args.warmup), args.steps
    cfg = presets["qwen3-tts-1.7b"]()
    ck = random_checkpoint(cfg, seed=0, device="cuda")
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    with ClockSampler(local) as clocks:
        rep = replay_baseline(cfg, ck, args.sessions, args.prompt, W, K, seed=rank, clocks=clocks)
    t_el = torch.tensor([rep["elapsed_s"]], device="cuda", dtype=torch.float64)
    t_p99 = torch.tensor([rep["tick_p99_ms"]], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_el, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_p99, op=dist.ReduceOp.MAX)
        dist.barrier()
        dist.destroy_process_group()  # the other ranks leave here; rank 0 alone may go on to the CPU leg
    if rank != 0:
        return
    value = args.sessions * world * K / float(t_el.item())
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * float(t_el.item()) / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": CONFIG_WORKLOAD, "sessions_per_gpu": args.sessions, "prompt_tokens": args.prompt,
                       "kv_page": 16, "sampling": "top-k 50, T 0.9, repetition penalty 1.05, host uniforms",
                       "step": "one decode tick = %d frames per GPU" % args.sessions,
                       "parallelism": f"{world} replica(s), no collective",
                       "engine": rep["what"]},
            "tick_p99_ms": float(t_p99.item()), "graph_nodes": rep["graph_nodes"], "clocks": clocks.summary(),
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": rep["h2d_bytes_per_step"], "d2h_bytes_per_step": 0,
                    "timing": "the arm's timed region already holds its per-tick input staging copies"},
            "gpu_launches": int(rep["graph_nodes"] * K),
            "reference_kind": "reference (its CUDA sources compiled unmodified for sm_100a into oracle/_ref; the Rust "
                              "runtime that sequences them is not in the reference tree, so the sequencing and the "
                              "cuBLAS calls are this repository's)"}
    if world == 1 and not args.no_cpu_baseline:
        del ck
        torch.cuda.empty_cache()
        ck_host = {k: v.cpu() for k, v in random_checkpoint(cfg, seed=0, device="cuda").items()}
        base, _ = cpu_baseline(cfg, ck_host)
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)


def run_higgs(args, rank, world, local):
    """The Higgs-style step (36-layer h2560 20q/4kv body, 8 x 1026 tied head) at `--sessions` sequences per GPU with
    `--prompt`-token prompts: W warm-up steps, K timed steps through `HiggsModel.step`; device time per step from the
    library's CUDA events. Per-op launches, no CUDA graph."""
    import torch
    import torch.distributed as dist
    from pega_omni_b200.higgs import HIGGS_PRESETS, HiggsDraw, HiggsModel, higgs_random_checkpoint
    W, K = max(3, args.warmup), args.steps
    n = args.sessions if args.sessions != 64 else 32  # configs[4]: 32 sessions
    plen = args.prompt if args.prompt != 128 else 256
    import dataclasses
    c = dataclasses.replace(HIGGS_PRESETS["higgs-4b"], audio_adapter=args.audio_adapter)
    ck = higgs_random_checkpoint(c, seed=0, device=f"cuda:{local}", embed_std=0.02)
    b = c.body
    kv_token = b.num_hidden_layers * 2 * b.num_key_value_heads * b.head_dim * 2
    kv_gib = 1.3 * n * (plen + W + K + 32) * kv_token / 2 ** 30
    model = HiggsModel.load(local, ck, c, max_batch=n, max_tokens=max(2048, plen), kv_gib=max(kv_gib, 0.5))
    model.warmup()  # every bucket's graph before the first live step, as the reference's Model::warmup does
    del ck
    torch.cuda.empty_cache()
    rng = np.random.default_rng(200 + rank)
    seqs = [model.open(plen, W + K + 16) for _ in range(n)]
    per_call = max(1, 2048 // plen)
    for i in range(0, n, per_call):
        part = seqs[i:i + per_call]
        prompts = [rng.integers(0, b.vocab_size, plen).astype(np.int32) for _ in part]
        model.start([(s, p, HiggsDraw([float(v) for v in rng.random(8)])) for s, p in zip(part, prompts)])

    def draws():
        return [HiggsDraw([float(v) for v in rng.random(8)]) for _ in range(n)]

    for _ in range(W):
        model.step(list(zip(seqs, draws())))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    dev_ms, launches = [], 0
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()  # after the sampler's start-up
        for _ in range(K):
            model.step(list(zip(seqs, draws())))
            ms, launches = model.stats()
            dev_ms.append(ms)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0  # before the sampler's shutdown
    t_wall = torch.tensor([wall], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_wall, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, peak_kind = measured_peaks()
        mean_len = plen + 1 + W + (K - 1) / 2 + 1
        step_bytes = c.step_weight_bytes() + n * mean_len * kv_token
        step_s = float(np.mean(dev_ms)) * 1e-3
        print(json.dumps({
            "metric": "Higgs-style step ms (device) at %d sequences per GPU" % n, "value": float(np.mean(dev_ms)),
            "unit": "ms", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": 1e3 * float(t_wall.item()) / K,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "configs[4]: Higgs-style body (36L h2560 20q/4kv d128 i9728) + tied 8 x 1026 head, "
                                   "random bf16 weights", "sessions_per_gpu": n, "prompt_tokens": plen,
                       "audio_adapter": bool(c.audio_adapter),
                       "sampling": "T 1.0, top-k 50, delay-pattern ramp",
                       "engine": "one kernel per op, one CUDA graph per session bucket"},
            "step_p50_ms": float(np.percentile(dev_ms, 50)), "step_p99_ms": float(np.percentile(dev_ms, 99)),
            "rows_per_s": n * world * K / float(t_wall.item()),
            "gpu_launches": int(launches * K), "launches_per_step": int(launches), "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "kernel": "whole step (%d launches)" % launches,
                         "achieved": step_bytes / step_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": step_bytes / step_s / 1e9 / peak, "peak_source": f"of {peak_kind}", "traffic": None},
            "reference_published": "about 9 ms per step at 1 sequence on a 48 GB sm_89 card "
                                   "(docs/higgs-audio.md:127-137 of the reference)"}))
    model.close()


def run_codec(args, rank, world, local):
    """The Qwen3-TTS streaming codec decoder at `--sessions` streams per GPU: every step decodes one frame of 16 codes
    of every stream into 1,920 samples through `Codec.decode` (codes staged from host memory, the waveform read back);
    device time per step from the library's CUDA events around the frame's kernels. One CUDA graph per bucket."""
    import torch
    import torch.distributed as dist
    from pega_omni_b200.codec import CODEC_PRESETS, Codec, codec_random_checkpoint
    W, K, n = max(3, args.warmup), args.steps, args.sessions
    c = CODEC_PRESETS["qwen3-tts-12hz"]
    torch.cuda.set_device(local)
    model = Codec(c, codec_random_checkpoint(c, seed=0), max_batch=n, device=local)
    model.warmup()
    streams = [model.open() for _ in range(n)]
    rng = np.random.default_rng(300 + rank)
    frames = rng.integers(0, c.codebook_size, size=(W + K, n, 16)).astype(np.int32)
    for f in range(W):
        model.decode(streams, frames[f])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    dev_ms, launches = [], 0
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        for f in range(K):
            model.decode(streams, frames[W + f])
            ms, launches = model.stats()
            dev_ms.append(ms)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    t_wall = torch.tensor([wall], device="cuda", dtype=torch.float64)
    t_dev = torch.tensor([float(np.sum(dev_ms)) * 1e-3], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_wall, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_dev, op=dist.ReduceOp.MAX)
    if rank == 0:
        flops = c.flops_per_frame() * n
        step_s = float(np.mean(dev_ms)) * 1e-3
        peak, kind = 1590.0, "fallback"
        if (ROOT / "MEASURED_PEAKS.json").exists():
            mp = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
            peak, kind = float(mp.get("bf16_tflops_sustained") or mp["bf16_tflops"]), "measured"
        print(json.dumps({
            "metric": "codec frames decoded per second at %d streams per GPU (Qwen3-TTS 12 Hz decoder)" % n,
            "value": n * world * K / float(t_dev.item()), "unit": "frames/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * float(t_dev.item()) / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "Qwen3-TTS-12Hz codec decoder (16 x 2048 RVQ, 8L h512 window-72 transformer, x2 x2 "
                                   "ConvNeXt upsamplers, 1536-wide SnakeBeta decoder x8 x5 x4 x3), random bf16 weights",
                       "streams_per_gpu": n, "samples_per_frame": c.samples_per_frame,
                       "step": "one frame of every stream", "l2": "each step streams %.0f MB of weights and about 1 GB "
                       "of activations, larger than the 126 MB L2" % (c.weight_bytes() / 1e6),
                       "engine": "one kernel per op, one CUDA graph per stream bucket"},
            "step_p50_ms": float(np.percentile(dev_ms, 50)), "step_p99_ms": float(np.percentile(dev_ms, 99)),
            "realtime_factor": n * world * K * c.samples_per_frame / 24000.0 / float(t_dev.item()),
            "e2e": {"value": n * world * K / float(t_wall.item()), "unit": "frames/s",
                    "h2d_bytes_per_step": int(n * 18 * 4), "d2h_bytes_per_step": int(n * c.samples_per_frame * 4 + 4),
                    "timing": "wall clock around K Codec.decode calls (codes from host memory, waveform read back)"},
            "gpu_launches": int(launches * K), "launches_per_step": int(launches), "clocks": clocks.summary(),
            "roofline": {"bound": "tensor", "kernel": "whole step (%d launches)" % launches,
                         "achieved": flops / step_s / 1e12, "peak": peak, "unit": "TFLOP/s",
                         "frac": flops / step_s / 1e12 / peak, "peak_source": f"of {kind}", "traffic": None,
                         "flops_per_step": flops},
            "reference_published": "1.0 ms of the reference's 8.27 ms tick at 64 sessions is its codec decoder "
                                   "(docs/bench.md:156-160 of the reference, other hardware)"}))
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_duplex(args, rank, world, local):
    """The PersonaPlex-7B tick (Helium 32 x 4096 + depformer 8 x 6 x 1024) at `--sessions` sessions per GPU: W warm-up
    ticks, K timed ticks through `Model.tick` (host staging and read-back inside), CUDA-event device time per tick from
    the library. One kernel per op, the tick replayed as one CUDA graph per session bucket (captured by `warmup`).
    `--prompt` rows are prefilled per session, so `--prompt 2990` measures the full 3,000-slot ring."""
    import dataclasses
    import torch
    import torch.distributed as dist
    from pega_omni_b200.duplex import PRESETS, Model, Prompt, Step, random_checkpoint
    W, K, n = max(3, args.warmup), args.steps, args.sessions
    tp = args.tp if args.tp > 1 else 1
    if tp > 1 and (world % tp or tp != 2):
        raise SystemExit("--tp 2 needs an even number of ranks (torchrun --nproc-per-node 2)")
    c = dataclasses.replace(PRESETS["personaplex-7b"], context=args.context)
    ck = random_checkpoint(c, seed=0, device=f"cuda:{local}", head_std=0.05)
    plen = args.prompt if args.prompt != 128 else 4  # --prompt: rows prefilled per session (default 4: near-empty ring)
    model = Model.load(local, ck, c, max_sessions=n, max_prefill=max(2048, plen), tp_rank=rank % tp, tp_size=tp)
    if tp > 1:  # ranks 2g and 2g + 1 form a pair: each maps the other's exchange region
        handles = [None] * world
        dist.all_gather_object(handles, model.tp_export())
        model.tp_connect(handles[rank ^ 1])
    model.warmup()  # every bucket's graph before the first live tick (model.rs:202-240 of the reference)
    del ck
    torch.cuda.empty_cache()
    rng = np.random.default_rng(100 + rank // tp)  # the two ranks of a pair play the same sessions
    sessions = [model.open() for _ in range(n)]
    per_call = max(1, 2048 // plen)  # prompts per prefill call
    for i in range(0, n, per_call):
        part = sessions[i:i + per_call]
        prompts = []
        for _ in part:
            rows = rng.integers(0, c.card, (plen, 17)).astype(np.int32)
            rows[:, 0] = rng.integers(0, c.text_vocab, plen)
            prompts.append(Prompt(rows, [int(v) for v in rows[-1]], [int(v) for v in rng.integers(0, c.card, 7)]))
        model.start(list(zip(part, prompts)))

    def steps_for(t):
        return [Step(caller=[int(v) for v in rng.integers(0, c.card, 8)], seed=(t << 20) | i) for i in range(n)]

    for t in range(W):
        model.tick(list(zip(sessions, steps_for(t))))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    dev_ms, launches = [], 0
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()  # after the sampler's start-up
        for t in range(K):
            model.tick(list(zip(sessions, steps_for(W + t))))
            ms, launches = model.stats()
            dev_ms.append(ms)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0  # before the sampler's shutdown
    t_wall = torch.tensor([wall], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_wall, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, peak_kind = measured_peaks()
        mean_len = plen + W + (K - 1) / 2 + 1
        kv_bytes = n * min(mean_len, c.context) * c.layers * (2 * c.heads * 128 + 2 * c.heads * 4)
        tick_bytes = c.tick_weight_bytes() + kv_bytes
        if tp > 1:  # per GPU: half of Helium's layer weights and of the ring, everything else whole
            layers_bytes = 2 * c.layers * (4 * c.dim * c.dim + 3 * c.hidden * c.dim)
            tick_bytes = c.tick_weight_bytes() - layers_bytes // 2 + kv_bytes / 2
        tick_s = float(np.mean(dev_ms)) * 1e-3
        print(json.dumps({
            "metric": "PersonaPlex tick ms (device) at %d sessions per GPU" % n, "value": float(np.mean(dev_ms)),
            "unit": "ms", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": 1e3 * float(t_wall.item()) / K,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (FP8 E4M3 ring KV)",
            "data": "synthetic",
            "config": {"workload": "configs[3]: PersonaPlex-7B shapes (Helium 32L d4096 32 heads hidden 11264; depformer "
                                   "8 steps x 6L d1024), random bf16 weights", "sessions_per_gpu": n,
                       "context": c.context, "positions": [plen + W, plen + W + K - 1],
                       "engine": "one kernel per op, one CUDA graph per session bucket"},
            "tick_p50_ms": float(np.percentile(dev_ms, 50)), "tick_p99_ms": float(np.percentile(dev_ms, 99)),
            "frames_per_s": n * (world // tp) * K / float(t_wall.item()),
            "tensor_parallel": None if tp == 1 else {
                "ranks_per_model": tp, "exchanges_per_tick": 2 * c.layers,
                "nvlink_bytes_per_tick_per_direction": 2 * c.layers * n * c.dim * 2,
                "how": "partial rows of the o and down projections read from the peer's buffer inside the add + norm "
                       "kernel (plain peer loads, flag words, bounded waits); no collective library on the data path"},
            "gpu_launches": int(launches * K), "launches_per_tick": int(launches), "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "kernel": "whole tick (%d launches)" % launches,
                         "achieved": tick_bytes / tick_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": tick_bytes / tick_s / 1e9 / peak, "peak_source": f"of {peak_kind}", "traffic": None},
            "reference_published": "15.0 ms p50 / 15.9 ms p99 at 128 sessions on GB300, Mimi codec included "
                                   "(docs/personaplex.md:105-111 of the reference)"}))
    if tp > 1:
        dist.barrier()  # neither rank unmaps its exchange region while the other may still be reading it
    model.close()


def run_sweep(args, rank, world, local):
    """configs[2]: the headline model at `--sessions` sessions per GPU with prompt lengths uniform in [--prompt,
    --prompt-max] and `--steps` decode frames per session. Buckets go up to 128 sessions, so larger counts run as
    consecutive groups of at most 128 (a tick of 256 sessions = two launches); the line reports the whole-tick time.
    Device-resident timing as in the headline arm; the reference's kernels are replayed at the mean prompt length for
    counts their shapes allow (<= 128)."""
    import torch
    import torch.distributed as dist
    from pega_omni_b200.config import presets
    from pega_omni_b200.model import Limits, Model
    from pega_omni_b200.synthetic import random_checkpoint
    W, K, n = max(3, args.warmup), args.steps, args.sessions
    lo, hi = args.prompt, max(args.prompt, args.prompt_max or args.prompt)
    cfg = presets["qwen3-tts-1.7b"]()
    ck = random_checkpoint(cfg, seed=0, device="cuda")
    rng = np.random.default_rng(2000 + rank)
    lens = [int(v) for v in rng.integers(lo, hi + 1, n)]
    frames_cap = W + K + 8
    group = min(n, 128)
    kv_gib = max(1.0, 1.15 * sum(l + frames_cap + 16 for l in lens) * cfg.talker.kv_bytes_per_token() / 2 ** 30)
    model = Model.load(local, ck, cfg, Limits(n, 16 * hi, kv_gib))
    from pega_omni_b200.model import Prompt
    prompts = [Prompt(list(rng.integers(0, cfg.text_vocab_size, l)), [-1] * l) for l in lens]
    seqs = [model.open(l, frames_cap) for l in lens]
    d0 = draws_for(1, n, seed=rank)[0]
    i = 0
    while i < n:  # prefill in calls that fit the token limit
        j, tokens = i, 0
        while j < n and j - i < group and tokens + lens[j] <= 16 * hi:
            tokens += lens[j]
            j += 1
        model.start(list(zip(seqs[i:j], prompts[i:j], d0[i:j])))
        i = j
    groups = [list(range(g, min(g + 128, n))) for g in range(0, n, 128)]
    for g in groups:
        model.run_ticks([seqs[k] for k in g], draws_for(W, len(g), seed=10 + rank))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    tick_ms = np.zeros(K)
    for g in groups:
        _, ms = model.run_ticks([seqs[k] for k in g], draws_for(K, len(g), seed=20 + rank))
        tick_ms += ms
    torch.cuda.synchronize()
    t_el = torch.tensor([float(tick_ms.sum()) * 1e-3], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_el, op=dist.ReduceOp.MAX)
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        peak, peak_kind = measured_peaks()
        mean_len = float(np.mean(lens)) + 1 + W + (K - 1) / 2 + 1
        tick_bytes = (len(groups) * (cfg.tick_weight_bytes() - cfg.tick_folded_bytes(min(n, 128))) +
                      cfg.talker.kv_bytes_per_token() * n * (mean_len + 1))
        tick_s = float(t_el.item()) / K
        line = {"metric": "codec frames/sec at %d sessions per GPU (Qwen3-TTS talker), ragged prompts" % n,
                "value": n * world * K / float(t_el.item()), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": 1e3 * tick_s, "tick_p99_ms": float(np.percentile(tick_ms, 99)), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "configs[2]: " + CONFIG_WORKLOAD, "sessions_per_gpu": n,
                           "prompt_tokens": [lo, hi], "frames": K, "launches_per_tick": len(groups),
                           "parallelism": f"{world} replica(s), no collective"},
                "roofline": {"bound": "hbm", "achieved": tick_bytes / tick_s / 1e9, "peak": peak, "unit": "GB/s",
                             "frac": tick_bytes / tick_s / 1e9 / peak, "peak_source": f"of {peak_kind}",
                             "note": "weights counted once per launch of a tick (%d)" % len(groups)}}
        if not args.no_replay and world == 1 and n <= 128:
            model.close()
            torch.cuda.empty_cache()
            rep = replay_baseline(cfg, ck, n, int(np.mean(lens)), W, K)
            if rep is not None:
                line["reference_replay"] = rep
                line["vs_replay"] = line["value"] / rep["value"]
        print(json.dumps(line), flush=True)
    model.close()


def run_attend(args):
    """The stand-alone decode-attention op (`omni_op_rope_attend`: per-head norm + RoPE + K/V write, then paged GQA
    attention) at the headline head shape (16 query / 8 kv heads of 128) with `--sessions` rows, one line per context
    length: device time between two events on the op context's stream (L2 flushed before every call), the KV bytes it
    must read, and the marginal rate between consecutive context lengths, which leaves the two launches' fixed cost out."""
    import torch
    from pega_omni_b200.ops import Ops
    ops = Ops(0)
    hq, hk, d, rows = 16, 8, 128, args.sessions
    peak, peak_kind = measured_peaks()
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    dev = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")
    prev = None
    for ctx in (16, 144, 384, 1024, 2048):
        per = (ctx + 15) // 16
        n_pages = rows * per
        kv = torch.randn((n_pages, hk, 2, 16, d), generator=g, device="cuda").to(torch.bfloat16)
        qkv0 = torch.randn((rows, (hq + 2 * hk) * d), generator=g, device="cuda").to(torch.bfloat16)
        gain = torch.ones(d, dtype=torch.bfloat16, device="cuda")
        pages = np.random.default_rng(0).permutation(n_pages).astype(np.int32)
        slot = [int(pages[s * per + (ctx - 1) // 16]) * 16 + (ctx - 1) % 16 for s in range(rows)]
        dpos, dslot, dseq = dev(np.full(rows, ctx - 1)), dev(slot), dev(np.arange(rows))
        dind, dpages = dev(np.arange(rows + 1) * per), dev(pages)
        out = torch.zeros((rows, hq * d), dtype=torch.bfloat16, device="cuda")
        times = []
        for it in range(max(3, args.warmup) + args.steps):
            qkv = qkv0.clone()
            flush.fill_(it & 255)
            torch.cuda.synchronize()
            ops.mark(0)
            ops.rope_attend(qkv, gain, gain, kv, n_pages, dpos, dslot, dseq, dind, dpages, hq, hk, d, 1e-6, 1e6, out)
            ops.mark(1)
            ops.sync()
            times.append(ops.elapsed_ms())
        t = float(np.median(times[max(3, args.warmup):])) * 1e-3
        kv_bytes = rows * ctx * hk * 2 * d * 2
        line = {"workload": "omni_op_rope_attend, %d rows, 16q/8kv heads of 128, paged bf16 KV" % rows, "context": ctx,
                "us": t * 1e6, "kv_mb": kv_bytes / 1e6, "gbs": kv_bytes / t / 1e9, "frac": kv_bytes / t / 1e9 / peak,
                "peak_source": f"of {peak_kind}", "l2": "flushed before every call"}
        if prev is not None:
            line["marginal_gbs"] = (kv_bytes - prev[0]) / (t - prev[1]) / 1e9
            line["marginal_frac"] = line["marginal_gbs"] / peak
        prev = (kv_bytes, t)
        print(json.dumps(line), flush=True)
        del kv
    ops.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sessions", type=int, default=64, help="sessions per GPU")
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--no-replay", action="store_true", help="skip timing the reference's kernels on this GPU")
    ap.add_argument("--per-op", action="store_true", help="one kernel per op (CUDA graph) instead of the tick kernel")
    ap.add_argument("--tp", type=int, default=1, help="duplex: 2 = Helium split over a pair of GPUs (run under torchrun with 2 ranks)")
    ap.add_argument("--audio-adapter", action="store_true",
                    help="higgs: every layer carries the audio-only MLP of configs[4] beside its MLP (run on every decode row)")
    ap.add_argument("--cluster-predictor", action="store_true",
                    help="tick_kernel = 3: the predictor's sub-steps as one launch of thread-block clusters (measured slower)")
    ap.add_argument("--prompt-max", type=int, default=0, help="sweep: prompt lengths uniform in [--prompt, --prompt-max]")
    ap.add_argument("--workload", default="talker", choices=["talker", "duplex", "higgs", "sweep", "attend", "codec"],
                    help="talker: the headline Qwen3-TTS tick (default); duplex: the PersonaPlex-7B tick (configs[3]); "
                         "higgs: the Higgs-style 4B step (configs[4]); codec: the streaming codec decoder, one frame of every stream per "
                         "step; sweep: configs[2]; attend: the paged attention kernel alone")
    ap.add_argument("--context", type=int, default=3000, help="duplex: KV ring length")
    ap.add_argument("--no-codec", action="store_true", help="talker: skip the tick + codec decoder arm (with_codec)")
    ap.add_argument("--e2e-waited", action="store_true", help="talker: the end-to-end arm waits on every step (Model.step) "
                    "instead of keeping two steps under way (step_begin / step_end)")
    ap.add_argument("--trace", default=None, help="talker: write the tick kernel's per-phase device timestamps here")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world, local)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    if args.workload == "duplex":
        run_duplex(args, rank, world, local)
        return
    if args.workload == "codec":
        return run_codec(args, rank, world, local)
    if args.workload == "higgs":
        run_higgs(args, rank, world, local)
        return
    if args.workload == "attend":
        run_attend(args)
        return
    if args.workload == "sweep":
        run_sweep(args, rank, world, local)
        return

    from pega_omni_b200 import replicas
    from pega_omni_b200.config import presets
    from pega_omni_b200.model import Limits, Model
    from pega_omni_b200.synthetic import random_checkpoint

    W, K = max(3, args.warmup), args.steps
    cfg = presets["qwen3-tts-1.7b"]()
    ck = random_checkpoint(cfg, seed=0, device="cuda")
    frames_cap = W + K + 8
    kv_gib = max(1.0, 1.25 * args.sessions * (args.prompt + frames_cap + 16) * cfg.talker.kv_bytes_per_token() / 2 ** 30)
    model = Model.load(local, ck, cfg, Limits(args.sessions, args.sessions * args.prompt, kv_gib),
                       use_graphs=not args.no_graphs, tick_kernel=0 if args.per_op else (3 if args.cluster_predictor else 1))
    if args.trace:
        model.trace(args.trace)
    ck_host = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        ck_host = {k: v.cpu() for k, v in ck.items()}
    if not (rank == 0 and world == 1 and not args.no_replay):
        del ck
        torch.cuda.empty_cache()

    # this rank's share of the global sessions (round-robin), a full replica per GPU
    mine = replicas.local_sessions(args.sessions * world, rank, world)
    n = len(mine)
    prompts = workload(cfg, n, args.prompt, seed=1000 + rank)
    seqs = [model.open(args.prompt, frames_cap) for _ in range(n)]
    d0 = draws_for(1, n, seed=rank)[0]
    prefill_ms = 0.0
    for i in range(0, n, 32):  # prefill in calls of at most 32 prompts (the split-K scratch is sized for decode)
        model.start(list(zip(seqs[i:i + 32], prompts[i:i + 32], d0[i:i + 32])))
        prefill_ms += model.stats().last_call_gpu_ms  # prefill + first frame of these prompts, device time

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident arm: W warm-up ticks, then exactly K timed ticks ----
    # (the clock sampler starts before the warm-up: the timed region can be shorter than nvidia-smi's start-up)
    with ClockSampler(local) as clocks:
        model.run_ticks(seqs, draws_for(W, n, seed=10 + rank))
        draws = draws_for(K, n, seed=20 + rank)
        first_frame = seqs[0].frames
        barrier()
        clocks.mark_start()
        _, tick_ms = model.run_ticks(seqs, draws)
        barrier()
        clocks.mark_end()
        time.sleep(0.12)  # two more sampling periods, so that a sample taken inside the window has been printed
    launches_per_tick = model.stats().last_call_launches // K
    elapsed = float(tick_ms.sum()) * 1e-3
    lens = [args.prompt + first_frame - 1 + t for t in range(K)]  # the position every session's row sits at
    t_el = torch.tensor([elapsed], device="cuda", dtype=torch.float64)
    t_p99 = torch.tensor([float(np.percentile(tick_ms, 99))], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_el, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_p99, op=dist.ReduceOp.MAX)
    elapsed_max = float(t_el.item())
    value = args.sessions * world * K / elapsed_max

    # ---- end-to-end arm: Model.step with host draws, staging and read-back inside every step ----
    # (each step's draws sit ready in host memory, laid out as the C ABI takes them, as an engine's staging buffer would)
    # On fresh sessions with the same prompts and the same W warm-up ticks, so that the timed steps sit at the same
    # positions (the same KV lengths) as the device-resident arm's and the reference arm's.
    from pega_omni_b200.model import DrawBatch
    for s in seqs:
        model.release(s)
    seqs = [model.open(args.prompt, frames_cap) for _ in range(n)]
    for i in range(0, n, 32):
        model.start(list(zip(seqs[i:i + 32], prompts[i:i + 32], d0[i:i + 32])))
    e2e_rng = np.random.default_rng(30 + rank)
    e2e_draws = [DrawBatch(e2e_rng.random((n, 16)).astype(np.float32)) for _ in range(W + K)]
    out = None
    for t in range(W):
        out = model.step_batch(seqs, e2e_draws[t], out)
    assert seqs[0].frames == first_frame
    barrier()
    t0 = time.perf_counter()
    dev_ms = 0.0
    if args.e2e_waited:  # one waited call per step, as the reference's engine drives its model
        for t in range(K):
            out = model.step_batch(seqs, e2e_draws[W + t], out)
            dev_ms += model.stats().last_call_gpu_ms
    else:  # step_begin / step_end, two steps under way: every step still stages its draws and reads its frames back
        model.step_begin(seqs, e2e_draws[W])
        for t in range(1, K):
            model.step_begin(seqs, e2e_draws[W + t])
            out = model.step_end(n, out)
            dev_ms += model.stats().last_call_gpu_ms
        out = model.step_end(n, out)
        dev_ms += model.stats().last_call_gpu_ms
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t_e2e = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    e2e_value = args.sessions * world * K / float(t_e2e.item())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()  # the other ranks are done; rank 0 alone runs the comparison legs below
    bucket = model.stats().bucket
    pages_per_seq = lens[-1] // 16 + 1
    h2d = 4 * (bucket * (1 + 1 + 16 + 16 + 1 + 1) + bucket + 1) + 4 * n * pages_per_seq  # staged front block (approx.)
    d2h = 4 * (bucket * 16 + 1)

    # ---- with the codec decoder behind every tick: what a serving engine runs per 80 ms frame (rank 0 only) ----
    with_codec = None
    if rank == 0 and not args.no_codec:
        from pega_omni_b200.codec import CODEC_PRESETS, Codec, codec_random_checkpoint
        cc = CODEC_PRESETS["qwen3-tts-12hz"]
        codec = Codec(cc, codec_random_checkpoint(cc, seed=0), max_batch=n, device=local)
        codec.warmup()
        for s_ in seqs:
            model.release(s_)
        model.attach_codec(codec)  # from here on start / step decode the frames they return into Out.wav
        seqs = [model.open(args.prompt, frames_cap) for _ in range(n)]
        for i in range(0, n, 32):
            model.start(list(zip(seqs[i:i + 32], prompts[i:i + 32], d0[i:i + 32])))
        kc = min(K, 32)
        out = None
        tick_ms = codec_ms = 0.0
        for t in range(W + kc):
            if t == W:
                torch.cuda.synchronize()
                t0 = time.perf_counter()
            out = model.step_batch(seqs, e2e_draws[t], out)
            if t >= W:
                tick_ms += model.stats().last_call_gpu_ms
                codec_ms += codec.stats()[0]
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        assert float(np.abs(out.wav).max()) > 0.0
        with_codec = {"ms_per_step": 1e3 * wall / kc, "value": n * kc / wall, "unit": UNIT, "steps": kc,
                      "device_ms": {"tick": tick_ms / kc, "codec_decoder": codec_ms / kc},
                      "what": "every step: omni_talker_step with the codec decoder attached (host draws in; codes and "
                              "1,920 f32 samples per session out); wall clock, one GPU, the tick and the decoder back "
                              "to back",
                      "reference_published": "8.27 ms per step at 64 sessions with its codec decoder, of which 1.00 ms "
                                             "codec (docs/bench.md:156-160 of the reference, other hardware)"}
        for s_ in seqs:
            model.release(s_)
        seqs = []
        model.attach_codec(None)
        codec.close()

    if rank == 0:
        peak, peak_kind = measured_peaks()
        mean_len = float(np.mean(lens)) + 1
        weight_bytes = cfg.tick_weight_bytes() - (cfg.tick_folded_bytes(n) if launches_per_tick <= 2 else 0)
        tick_bytes = weight_bytes + cfg.talker.kv_bytes_per_token() * n * (mean_len + 1)
        tick_s = elapsed / K
        # two more readings of the same time: against the nominal 8 TB/s, and counting the predictor's weights once per tick
        # (they are one L2's worth: 14 of the 15 passes can be served on chip)
        p_cfg, t_cfg = cfg.predictor, cfg.talker
        per_pass = p_cfg.num_hidden_layers * p_cfg.layer_weight_bytes() + 2 * p_cfg.hidden_size * t_cfg.hidden_size
        once_bytes = tick_bytes - (cfg.num_code_groups - 2) * per_pass
        # the dominant kernel IS the tick: one persistent cooperative launch per step (or, with --per-op, the graph)
        roof = {"bound": "hbm", "kernel": ("tick_kernel (one launch = one decode tick)" if launches_per_tick == 1 else
                           "tick_kernel + pred_kernel" if launches_per_tick == 2 else "per-op graph"),
                "achieved": tick_bytes / tick_s / 1e9, "peak": peak, "unit": "GB/s",
                "frac": tick_bytes / tick_s / 1e9 / peak, "peak_source": f"of {peak_kind}",
                "frac_nominal": tick_bytes / tick_s / 1e9 / 8000.0, "peak_nominal": 8000.0,
                "frac_predictor_weights_once": once_bytes / tick_s / 1e9 / peak,
                "bytes_per_launch": int(tick_bytes), "us_per_launch": tick_s * 1e6,
                # ncu cannot run inside the timed region: the DRAM bytes of one captured tick (6,231 MB read + written
                # for 6,129 MB algorithmic at positions 131-132) scaled to this run's algorithmic bytes; the traffic
                # grows with the KV length as they do
                "traffic": int(tick_bytes * 6230.8 / 6129.2) if launches_per_tick <= 2 else None,
                "traffic_note": "ncu dram__bytes_read+write of one captured tick (6.231 GB for 6.129 GB algorithmic), "
                                "scaled by this run's algorithmic bytes"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * elapsed_max / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": CONFIG_WORKLOAD,
                       "sessions_per_gpu": args.sessions, "prompt_tokens": args.prompt, "kv_page": 16,
                       "sampling": "top-k 50, T 0.9, repetition penalty 1.05, host uniforms (reference sampler)",
                       "step": "one decode tick = 64 frames per GPU", "positions": [lens[0], lens[-1]],
                       "parallelism": f"{world} replica(s), sessions round-robin, no collective",
                       "l2": "each tick streams 5.3 GB of weights, far larger than the 126 MB L2",
                       "engine": "persistent tick kernel" if launches_per_tick == 1 else "persistent talker kernel + cluster predictor kernel" if launches_per_tick == 2 else "per-op CUDA graph"},
            "tick_p99_ms": float(t_p99.item()), "tick_p50_ms": float(np.percentile(tick_ms, 50)),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "timing": "wall clock around K steps through the C ABI, each staging its draws from host memory and reading its frame back; "
                              + ("one waited call per step" if args.e2e_waited else "step_begin / step_end with two steps under way") + ", max over ranks",
                    "device_ms_per_step": dev_ms / K},
            "gpu_launches": int(launches_per_tick * K),
            "launches_per_tick": int(launches_per_tick),
            "clocks": clocks.summary(),
            "roofline": roof,
            "prefill": {"device_ms": prefill_ms, "prompt_tokens": int(n * args.prompt),
                        "tokens_per_s": n * args.prompt / (prefill_ms * 1e-3) if prefill_ms > 0 else None,
                        "what": "omni_talker_start in calls of at most 32 prompts: ragged prefill + first frame, untimed "
                                "by the headline metric (includes first-call plan building)"},
            "tick_bytes": {"weights": int(weight_bytes), "kv": int(tick_bytes - weight_bytes), "mean_kv_len": mean_len,
                           "folded_at_load": int(cfg.tick_weight_bytes() - weight_bytes)},
        }
        if with_codec is not None:
            line["with_codec"] = with_codec
        if not args.no_replay and world == 1:
            model.close()
            torch.cuda.empty_cache()
            rep = replay_baseline(cfg, ck, args.sessions, args.prompt, W, K)  # same positions as the arm above
            del ck
            if rep is not None:
                line["reference_replay"] = rep
                line["vs_replay"] = value / rep["value"]
        if ck_host is not None and world == 1:
            base, _ = cpu_baseline(cfg, ck_host)
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    model.close()


if __name__ == "__main__":
    main()
