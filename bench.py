#!/usr/bin/env python3
"""Decode throughput of the LFM2.5-1.2B-shaped model (random bf16 weights) on one B200.

    python bench.py --gpus 1 --steps K --warmup W

A "step" is one decode step of a batch of 8 requests at a context of 8,192 tokens.  After W warm-up
steps the K steps are timed RUNS times over (the reference's way: at least three runs, mean and
half-range, src/main.c:1891-1904).  The line printed at the end holds
  value      decoded tokens a second from the device time of K steps (CUDA events before the first and
             after the last step's work on the stream; nothing waits in between), mean over the runs,
  e2e        the same steps by the wall clock through the Python entry point (Engine.step):
             scheduler, pinned-host tables in, sampled ids out into pinned host memory,
  prefill    one 2,048-token prompt in one step,
  roofline   bytes the decode step has to read (every weight once, the live requests' keys and
             values and states) over its time, against the measured copy bandwidth,
  points     the rest of the matrix, flat: `<point>` is tokens a second, `<point>_pm` the half-range
             over the runs, `<point>_frac` the fraction of the roofline (HBM for decode, the bf16
             peak for prefill).  Points: decode at batch 1 and 64 (context 8,192); decode at batch
             1, 8, 64 from a 16-token prompt; the 2,048-token prompt as four portions of 512; the
             same model with a feed-forward width of 8,192 at batch 1; the LFM2-350M shape serving
             64 requests (prompts U[16,2048], U[32,512] new tokens) through Engine.generate; the
             LFM2-2.6B shape: an 8,192-token prompt in portions of 2,048, then decode at batch 1, 8
             and 64 at a context of 16,384.
Peaks come from MEASURED_PEAKS.json beside this file when it exists, else the fallback figures.
For more than one GPU it prints one line that says so and exits with 2: the engine is
single-GPU.  `--impl reference` answers that the reference cannot run here.
`--print-config NAME` prints one of the shapes below as a config.json and exits.
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

# The sizes of the measured models as config.json dictionaries (no weights: they are drawn at random).
_LFM2 = dict(architectures=["Lfm2ForCausalLM"], block_multiple_of=256, vocab_size=65536, rope_theta=1e6,
             norm_eps=1e-5, conv_L_cache=3, tie_embedding=True, max_position_embeddings=128000,
             num_key_value_heads=8)
SHAPES = {
    "lfm2.5-1.2b": dict(_LFM2, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, intermediate_size=8192,
                        block_auto_adjust_ff_dim=True, full_attn_idxs=[2, 5, 8, 10, 12, 14]),
    # the width the reference's own engine reads from its checkpoint (src/lfm25_model.c:100)
    "lfm2.5-1.2b-f8192": dict(_LFM2, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
                              intermediate_size=8192, block_auto_adjust_ff_dim=False,
                              full_attn_idxs=[2, 5, 8, 10, 12, 14]),
    "lfm2-350m": dict(_LFM2, hidden_size=1024, num_hidden_layers=16, num_attention_heads=16, intermediate_size=6656,
                      block_auto_adjust_ff_dim=True, full_attn_idxs=[2, 5, 8, 10, 12, 14]),
    "lfm2-2.6b": dict(_LFM2, hidden_size=2048, num_hidden_layers=30, num_attention_heads=32, intermediate_size=10752,
                      block_auto_adjust_ff_dim=True, full_attn_idxs=[2, 6, 10, 14, 18, 21, 24, 27]),
}

CONTEXT = 8192
BATCH = 8
PREFILL_TOKENS = 2048
RUNS = 3
PAGE = 64
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


def decode_bytes(nums, batch, context):
    """What a decode step of `batch` rows at `context` cached tokens has to read: every weight once, each
    row's keys and values, each row's states read and written."""
    return nums["weight_bytes"] + batch * (context * nums["kv_bytes_per_token"] + 2 * nums["state_bytes"])


def mean_pm(xs):
    return sum(xs) / len(xs), (max(xs) - min(xs)) / 2.0


def measure_decode(engine, batch, context, steps, warmup, rng, genuine_prefill, runs=RUNS):
    """Brings `batch` requests to `context - runs * steps - warmup - 2` cached tokens, then times `runs`
    times `steps` decode steps through `Engine.step`.  Returns per run the device seconds (CUDA events
    before the first and after the last step; no wait in between) and the wall seconds, the kernel
    launches of all timed steps, and the mean context of the timed steps."""
    import torch
    from tuff_b200.engine import StepEntry
    from tuff_b200.engine.scheduler import RequestStatus
    from tuff_b200.kernels import ops
    from tuff_b200.sampling import SamplingParams
    sch, runner = engine.scheduler, engine.runner
    n_new = runs * steps + warmup + 2
    prompt_len = context - n_new
    vocab = runner.vocab_size
    sp = SamplingParams(max_new_tokens=n_new)
    for i in range(batch):
        r = sch.add(("bench", batch, context, i), rng.integers(0, vocab, prompt_len).tolist(), sp)
        sch.waiting.remove(r)
        r.cache = runner.open(r.request_id)
        if genuine_prefill:
            # the prompt but its last token, through the step function in portions of the token budget
            for lo in range(0, prompt_len - 1, sch.max_batched_tokens):
                runner.step([StepEntry(r.cache, r.prompt[lo:min(prompt_len - 1, lo + sch.max_batched_tokens)], [])])
        elif prompt_len > 1:
            # a long context whose content does not matter: pages are taken, not computed
            runner.synthetic_fill(r.cache, prompt_len - 1)
        r.status = RequestStatus.RUNNING
        sch.running.append(r)
    engine.step()                                         # the last prompt token of each: now all decode
    for _ in range(warmup):
        engine.step()
    dev_s, wall_s = [], []
    launches0, replays0 = ops.LAUNCHES["n"], runner.graph_replays
    for _ in range(runs):
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        s.record()
        for _ in range(steps):
            engine.step()                                 # ends with the read of a step's sampled ids
        e.record()
        e.synchronize()
        wall_s.append(time.perf_counter() - t0)
        dev_s.append(s.elapsed_time(e) * 1e-3)
    g = runner._graphs.get(batch)
    launches = (ops.LAUNCHES["n"] - launches0) + (runner.graph_replays - replays0) * (g["launches"] if g and "launches" in g else 0)
    engine.reset()
    ops.check_tc_status()
    ctx_mid = prompt_len + 1 + warmup + runs * steps / 2.0
    return dev_s, wall_s, launches, ctx_mid


def decode_point(points, name, engine, nums, pk, batch, context, steps, warmup, rng, genuine):
    dev_s, _, _, ctx_mid = measure_decode(engine, batch, context, steps, warmup, rng, genuine)
    v, pm = mean_pm([batch * steps / t for t in dev_s])
    points[name] = round(v, 1)
    points[name + "_pm"] = round(pm, 1)
    points[name + "_frac"] = round(decode_bytes(nums, batch, ctx_mid) / (batch / v) / 1e9 / pk["hbm_gbs"], 4)


def measure_prefill(runner, cfg, rng, total, portion, runs=RUNS, warmup=2):
    """A prompt of `total` tokens from an empty cache in portions of `portion`; logits of the last token
    only.  Returns the device seconds of each run."""
    import torch
    from tuff_b200.engine import StepEntry
    out = []
    for i in range(warmup + runs):
        rc = runner.open(("prefill", total, portion, i))
        toks = rng.integers(0, cfg.vocab_size, total).tolist()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for lo in range(0, total, portion):
            hi = min(total, lo + portion)
            runner.step([StepEntry(rc, toks[lo:hi], [hi - lo - 1] if hi == total else [])])
        e.record()
        e.synchronize()
        runner.close(rc)
        if i >= warmup:
            out.append(s.elapsed_time(e) * 1e-3)
    return out


def prefill_point(points, name, runner, cfg, nums, pk, rng, total, portion):
    secs = measure_prefill(runner, cfg, rng, total, portion)
    v, pm = mean_pm([total / t for t in secs])
    points[name] = round(v, 1)
    points[name + "_pm"] = round(pm, 1)
    points[name + "_frac"] = round(prefill_flops(cfg, nums, total) / (total / v) / (pk["bf16_tflops"] * 1e12), 4)


def serve_point(points, name, engine, rng, n_requests=64, runs=RUNS):
    """`n_requests` requests at once through `Engine.generate`: prompts of U[16, 2048] tokens, U[32, 512] new
    tokens each, chunked prompts beside decoding rows.  Tokens a second over everything (prompt and new
    tokens), the split, the steps, the preemptions, and the share of the wall time that the host spent
    laying out and launching steps."""
    import torch
    from tuff_b200.sampling import SamplingParams
    vocab = engine.runner.vocab_size
    prompts = [rng.integers(0, vocab, int(rng.integers(16, 2049))).tolist() for _ in range(n_requests)]
    params = [SamplingParams(max_new_tokens=int(rng.integers(32, 513))) for _ in range(n_requests)]
    n_prompt, n_new = sum(len(p) for p in prompts), sum(p.max_new_tokens for p in params)
    engine.generate(prompts, params)                      # warm-up: the decode graphs of every row count are captured
    rates, host = [], []
    for _ in range(runs):
        before = engine.stats()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = engine.generate(prompts, params)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        after = engine.stats()
        assert sum(len(o) for o in outs) == n_new
        rates.append((n_prompt + n_new) / wall)
        host.append((after["step_seconds"] - before["step_seconds"]) / wall)
        steps = after["steps"] - before["steps"]
        preempted = after["preemptions"] - before["preemptions"]
    # once more with every step bracketed by events: the time the device worked, against the wall
    engine.step_events = []
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.generate(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    busy = sum(a.elapsed_time(b) for a, b, _ in engine.step_events) * 1e-3
    mixed = [(a.elapsed_time(b), n) for a, b, n in engine.step_events if n > n_requests]
    engine.step_events = None
    v, pm = mean_pm(rates)
    points[name] = round(v, 1)
    points[name + "_pm"] = round(pm, 1)
    points[name + "_device_share"] = round(busy / wall, 3)
    points[name + "_mixed_steps"] = len(mixed)
    points[name + "_mixed_step_ms"] = round(sum(t for t, _ in mixed) / max(1, len(mixed)), 3)
    points[name + "_prompt_tokens"] = n_prompt
    points[name + "_new_tokens"] = n_new
    points[name + "_steps"] = int(steps)
    points[name + "_preemptions"] = int(preempted)
    points[name + "_host_share"] = round(sum(host) / len(host), 3)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (recorded)")
    ap.add_argument("--no-points", action="store_true", help="the headline only: no prefill, no other points")
    ap.add_argument("--print-config", choices=sorted(SHAPES), default=None, help="print a shape as a config.json and exit")
    args = ap.parse_args()
    if args.print_config:
        print(json.dumps(SHAPES[args.print_config], indent=1))
        return 0
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

    cfg_dict = dict(SHAPES["lfm2.5-1.2b"])
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        cfg_dict["num_hidden_layers"] = args.layers
        cfg_dict["full_attn_idxs"] = [i for i in cfg_dict["full_attn_idxs"] if i < args.layers]
    cfg, nums = model_numbers(cfg_dict)
    pk, pk_src = peaks()
    rng = np.random.default_rng(0)
    few = min(steps, 32)

    def make_engine(config, context, biggest):
        eng = Engine(None, dtype="bfloat16", ctx_size=context, max_tokens=biggest * context + 4096, page_size=PAGE,
                     max_batched_tokens=PREFILL_TOKENS, max_running=biggest, config=config, weight_seed=0)
        eng.runner.randomize_cache(1)
        return eng

    biggest = BATCH if args.no_points else 64
    engine = make_engine(cfg_dict, CONTEXT, biggest)
    runner = engine.runner
    points = {}

    # ---- prefill of 2,048 tokens in one step ---------------------------------------------
    prefill = None
    if not args.no_points:
        secs = measure_prefill(runner, cfg, rng, PREFILL_TOKENS, PREFILL_TOKENS)
        ms = sum(secs) / len(secs) * 1e3
        prefill = dict(value=round(PREFILL_TOKENS / ms * 1e3, 1), tokens=PREFILL_TOKENS, ms=round(ms, 3),
                       frac=round(prefill_flops(cfg, nums, PREFILL_TOKENS) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4))

    # ---- the headline: batch 8 at context 8,192 ------------------------------------------
    sampler = ClockSampler()
    sampler.start()
    dev_s, wall_s, launches, ctx_mid = measure_decode(engine, BATCH, CONTEXT, steps, warmup, rng, genuine_prefill=True)
    clocks = sampler.stop()
    value, value_pm = mean_pm([BATCH * steps / t for t in dev_s])
    e2e_value, e2e_pm = mean_pm([BATCH * steps / t for t in wall_s])
    ms_per_step = BATCH / value * 1e3
    achieved = decode_bytes(nums, BATCH, ctx_mid) / (ms_per_step * 1e-3) / 1e9

    if not args.no_points:
        for b in (1, 64):
            decode_point(points, f"decode_b{b}", engine, nums, pk, b, CONTEXT, few, warmup, rng, genuine=(b == 1))
        for b in (1, 8, 64):
            decode_point(points, f"decode_b{b}_prompt16", engine, nums, pk, b, 16 + RUNS * few + warmup + 2, few, warmup,
                         rng, genuine=True)
        prefill_point(points, "prefill_4x512", runner, cfg, nums, pk, rng, PREFILL_TOKENS, 512)
        del engine, runner
        torch.cuda.empty_cache()

        wide = SHAPES["lfm2.5-1.2b-f8192"]
        _, wide_nums = model_numbers(wide)
        eng = make_engine(wide, CONTEXT, 1)
        decode_point(points, "f8192_decode_b1", eng, wide_nums, pk, 1, CONTEXT, few, warmup, rng, genuine=True)
        points["f8192_mb_per_token"] = round(wide_nums["weight_bytes"] / 1e6, 1)
        del eng
        torch.cuda.empty_cache()

        small = SHAPES["lfm2-350m"]
        eng = Engine(None, dtype="bfloat16", ctx_size=CONTEXT, max_tokens=64 * 2560 + 4096, page_size=PAGE,
                     max_batched_tokens=PREFILL_TOKENS, max_running=64, config=small, weight_seed=0)
        serve_point(points, "serve_350m", eng, rng)
        del eng
        torch.cuda.empty_cache()

        big = SHAPES["lfm2-2.6b"]
        big_cfg, big_nums = model_numbers(big)
        eng = make_engine(big, 16384, 64)
        prefill_point(points, "big_prefill_8192_by_2048", eng.runner, big_cfg, big_nums, pk, rng, 8192, 2048)
        for b in (1, 8, 64):
            decode_point(points, f"big_decode_b{b}", eng, big_nums, pk, b, 16384, min(few, 16), warmup, rng, genuine=(b == 1))
        del eng
        torch.cuda.empty_cache()

    h2d = 4 * (8 * (BATCH + 4) + (BATCH * ((CONTEXT + PAGE - 1) // PAGE) + 4))
    out = {
        "metric": "decode tok/s at batch 8, context 8192 (LFM2.5-1.2B shape)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random N(0,0.02) bf16 weights, uniform random token ids)",
        "config": {"model": "LFM2.5-1.2B shape", "global_batch": BATCH, "seq_len": CONTEXT, "parallelism": "single GPU",
                   "layers": cfg.num_hidden_layers, "layers_of_config": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "ffn": cfg.ffn_dim, "vocab": cfg.vocab_size, "conv_L_cache": cfg.conv_L_cache,
                   "attn_layers": nums["n_attn"], "page_size": PAGE, "l2": "inputs larger than L2 (2.6 GB per step)",
                   "peaks": pk_src, "points_cache": "b64 contexts filled without computing them",
                   "runs": f"{RUNS} x {steps} steps, mean; half-range in value_pm"},
        "value_pm": round(value_pm, 1),
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "pm": round(e2e_pm, 1), "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * (BATCH + 1)},
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
