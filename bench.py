#!/usr/bin/env python3
"""Decode throughput of the LFM2.5-1.2B-shaped model (random bf16 weights) on one B200.

    python bench.py --gpus 1 --steps K --warmup W

A "step" is one decode step of a batch of 8 requests at a context of 8,192 tokens.  The line
printed at the end holds
  value      decoded tokens a second from the device time of the K timed steps (CUDA events
             around each step's work on the stream: table copy, the captured decode graph,
             the sampling kernel),
  e2e        the same K steps by the wall clock through the Python entry point (Engine.step):
             scheduler, pinned-host tables in, sampled ids out,
  prefill    one 2,048-token prompt in one step,
  roofline   bytes the decode step has to read (every weight once, the live requests' keys and
             values and states) over its time, against the measured copy bandwidth,
  points     decode tokens a second at batch 1 and 64 (same context).
Peaks come from MEASURED_PEAKS.json beside this file when it exists, else the fallback figures.
For more than one GPU it prints one line that says so and exits with 2: the engine is
single-GPU.  `--impl reference` answers that the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tuff_b200.config.lfm2 import LFM2_1P2B_SHAPE as LFM2_1P2B      # the sizes of configs[2], no weights

CONTEXT = 8192
BATCH = 8
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return dict(sm_mhz=mhz[len(mhz) // 2] if mhz else None, sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(mhz))


def model_numbers(cfg_dict):
    """Bytes of weights a decode step reads, cache bytes per token and per request, matmul parameters."""
    from tuff_b200.config import config_from_dict
    from tuff_b200.models import Model
    import math
    arch, cfg = config_from_dict(cfg_dict)
    model = Model(arch.model_spec(cfg))
    exp = model.expected_tensors()
    n_params = sum(math.prod(d.shape) for d in exp.values())
    weight_bytes = sum(math.prod(d.shape) * (4 if d.role == "vector" else 2) for d in exp.values())
    embed = cfg.vocab_size * cfg.hidden_size
    # the embedding table is read as the head (all rows) and as B gathered rows: count it once
    matmul_params = sum(math.prod(d.shape) for n, d in exp.items() if d.role == "matrix" and len(d.shape) == 2)
    if not cfg.tie_embedding:
        matmul_params -= embed                       # the untied embedding is gathered, not multiplied
    n_attn = len(cfg.full_attn_idxs)
    kv_bytes_per_token = n_attn * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    state_bytes = len(cfg.conv_idxs) * (cfg.conv_L_cache - 1) * cfg.hidden_size * 4
    return cfg, dict(n_params=n_params, weight_bytes=weight_bytes, matmul_params=matmul_params,
                     kv_bytes_per_token=kv_bytes_per_token, state_bytes=state_bytes, n_attn=n_attn)


def prefill_flops(cfg, nums, T):
    """Multiply-adds x 2 of a T-token prompt from an empty cache: matrices (the head for the last
    row only) and causal attention."""
    d, V = cfg.hidden_size, cfg.vocab_size
    body = nums["matmul_params"] - V * d
    f = 2.0 * body * T + 2.0 * V * d
    f += nums["n_attn"] * 2.0 * 2.0 * cfg.num_attention_heads * cfg.head_dim * (T * (T + 1) / 2)
    return f


def measure_decode(engine, batch, context, steps, warmup, rng, genuine_prefill):
    """Brings `batch` requests to `context - steps - warmup - 1` cached tokens, then times decode steps.
    Returns (device seconds per step list, wall seconds for the timed steps, launches per step)."""
    import torch
    from tuff_b200.kernels import ops
    from tuff_b200.sampling import SamplingParams
    sch, runner = engine.scheduler, engine.runner
    n_new = steps + warmup + 2
    prompt_len = context - n_new
    vocab = runner.vocab_size
    sp = SamplingParams(max_new_tokens=n_new)
    reqs = []
    from tuff_b200.engine import StepEntry
    from tuff_b200.engine.scheduler import RequestStatus
    for i in range(batch):
        r = sch.add(("bench", batch, i), rng.integers(0, vocab, prompt_len).tolist(), sp)
        sch.waiting.remove(r)
        r.cache = runner.open(r.request_id)
        if genuine_prefill:
            # the prompt but its last token, through the step function in portions of the token budget
            for lo in range(0, prompt_len - 1, sch.max_batched_tokens):
                runner.step([StepEntry(r.cache, r.prompt[lo:min(prompt_len - 1, lo + sch.max_batched_tokens)], [])])
        else:
            # a long context whose content does not matter: pages are taken, not computed
            runner.synthetic_fill(r.cache, prompt_len - 1)
        r.status = RequestStatus.RUNNING
        sch.running.append(r)
        reqs.append(r)
    engine.step()                                         # the last prompt token of each: now all decode
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    dev_ms = []
    launches0 = ops.LAUNCHES["n"]
    replays0 = runner.graph_replays
    t0 = time.perf_counter()
    for _ in range(steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        engine.step()                                     # ends with the read of the sampled ids
        e.record()
        e.synchronize()
        dev_ms.append(s.elapsed_time(e))
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    eager_launches = ops.LAUNCHES["n"] - launches0
    replays = runner.graph_replays - replays0
    g = runner._graphs.get(batch)
    launches = eager_launches + replays * (g["launches"] if g and "launches" in g else 0)
    for r in reqs:
        if r.cache is not None:
            sch.abort(r)
    ops.check_tc_status()
    return dev_ms, wall, launches


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (recorded)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points and the prefill")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "niihelium/tuff is a C/CUDA CMake project for sm_86 with no Python package "
                          "(pip: neither setup.py nor pyproject.toml), and needs Q4_K_M GGUF files and a llama.cpp checkout"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "tuff_b200 is a single-GPU engine: run with --gpus 1", "n_gpus": args.gpus}))
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import numpy as np
    import torch

    from tuff_b200.engine.engine import Engine
    from tuff_b200.kernels import ops

    cfg_dict = dict(LFM2_1P2B)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        cfg_dict["num_hidden_layers"] = args.layers
        cfg_dict["full_attn_idxs"] = [i for i in cfg_dict["full_attn_idxs"] if i < args.layers]
    cfg, nums = model_numbers(cfg_dict)
    pk, pk_src = peaks()
    rng = np.random.default_rng(0)

    page_size = 64
    biggest = BATCH if args.no_points else 64
    engine = Engine(None, dtype="bfloat16", ctx_size=CONTEXT, max_tokens=biggest * CONTEXT + 4096, page_size=page_size,
                    max_batched_tokens=PREFILL_TOKENS, max_running=biggest, config=cfg_dict, weight_seed=0)
    runner = engine.runner
    runner.randomize_cache(1)

    # ---- prefill of 2,048 tokens in one step ---------------------------------------------
    prefill = None
    if not args.no_points:
        from tuff_b200.engine import StepEntry
        times = []
        for i in range(3 + 3):
            rc = runner.open(("prefill", i))
            toks = rng.integers(0, cfg.vocab_size, PREFILL_TOKENS).tolist()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            runner.step([StepEntry(rc, toks, [PREFILL_TOKENS - 1])])
            e.record()
            e.synchronize()
            runner.close(rc)
            if i >= 3:
                times.append(s.elapsed_time(e))
        ms = sorted(times)[len(times) // 2]
        fl = prefill_flops(cfg, nums, PREFILL_TOKENS)
        prefill = dict(value=round(PREFILL_TOKENS / ms * 1e3, 1), tokens=PREFILL_TOKENS, ms=round(ms, 3),
                       frac=round(fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4))

    # ---- the headline: batch 8 at context 8,192 ------------------------------------------
    sampler = ClockSampler()
    sampler.start()
    dev_ms, wall, launches = measure_decode(engine, BATCH, CONTEXT, steps, warmup, rng, genuine_prefill=True)
    clocks = sampler.stop()
    total_ms = sum(dev_ms)
    ms_per_step = total_ms / steps
    value = BATCH * steps / (total_ms * 1e-3)
    e2e_value = BATCH * steps / wall
    ctx_mid = CONTEXT - (steps + 2) / 2.0
    step_bytes = nums["weight_bytes"] + BATCH * (ctx_mid * nums["kv_bytes_per_token"] + 2 * nums["state_bytes"])
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9

    points = {}
    if not args.no_points:
        for b in (1, 64):
            d, _, _ = measure_decode(engine, b, CONTEXT, min(steps, 32), warmup, rng, genuine_prefill=(b == 1))
            points[f"decode_b{b}"] = round(b * len(d) / (sum(d) * 1e-3), 1)

    h2d = 4 * (8 * (BATCH + 4) + (BATCH * ((CONTEXT + page_size - 1) // page_size) + 4))
    out = {
        "metric": "decode tok/s at batch 8, context 8192 (LFM2.5-1.2B shape)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random N(0,0.02) bf16 weights, uniform random token ids)",
        "config": {"model": "LFM2.5-1.2B shape", "global_batch": BATCH, "seq_len": CONTEXT, "parallelism": "single GPU",
                   "layers": cfg.num_hidden_layers, "layers_of_config": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size, "conv_L_cache": cfg.conv_L_cache,
                   "attn_layers": nums["n_attn"], "page_size": page_size, "l2": "inputs larger than L2 (2.6 GB per step)",
                   "peaks": pk_src, "points_cache": "b64 context filled without computing it"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * BATCH},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill:
        out["prefill"] = prefill
    if points:
        out["points"] = points
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
