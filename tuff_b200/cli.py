"""Command line in the manner of the reference's `tuff` (src/main.c:45-97 usage,
769-979 flags): the same names and meanings where it has them.

    bin/tuff --model DIR --prompt-ids "1 5 9" -n 128 [--temp 0.8 --seed 2 ...]

Differences that the engine's scope makes: the model is a folder (config.json +
safetensors) instead of a GGUF file; prompts are token ids (`--prompt-ids`,
`--prompt-ids-file`; `--prompt TEXT` needs a `tokenizer.json` in the folder and
the `tokenizers` package); `--random CONFIG.json --weight-seed S` writes a
random-weights folder first.  Modes kept: timed generation with `--warmup` and
`--runs` (mean and half-range of tok/s, src/main.c:1891-1904), `--inspect`,
`--dump-tokens` (ids on stdout, all else on stderr, src/main.c:1661-1718),
`--dump-logits PATH` and `--teacher-force FILE [--tf-batch B]` (logit rows in
the reference's container: 8 bytes "CLBRLGT1", u32 rows, u32 vocab, then fp32
rows; src/main.c:1340-1351,1608-1613).  Exit codes as there: 0 ok, 1 runtime
error, 2 usage, 3 fatal I/O.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import sys
import tempfile
import time
from typing import List


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tuff", description="LFM2/LFM2.5 dense inference on one B200")
    ap.add_argument("--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--random", metavar="CONFIG.json", help="make a random-weights model from this config.json")
    ap.add_argument("--weight-seed", type=int, default=0)
    ap.add_argument("--prompt", "-p", help="prompt text (needs tokenizer.json in the model folder)")
    ap.add_argument("--prompt-file", help="read the prompt text from a UTF-8 file")
    ap.add_argument("--prompt-ids", help="prompt as token ids, separated by spaces or commas")
    ap.add_argument("--prompt-ids-file", help="prompt token ids from a file")
    ap.add_argument("-c", "--ctx-size", "--max-seq", dest="ctx", type=int, default=4096,
                    help="maximum context sequence length (default: 4096)")
    ap.add_argument("-n", dest="n_predict", type=int, default=None, help="tokens to generate (default: 128; 32 in dump modes)")
    ap.add_argument("--warmup", type=int, default=32, help="warmup tokens (default: 32)")
    ap.add_argument("--runs", type=int, default=3, help="benchmark runs (default: 3)")
    ap.add_argument("--prefill-batch", type=int, default=None,
                    help="feed the prompt in portions of at most N tokens (default: the step's token budget)")
    ap.add_argument("--tf-batch", type=int, default=1, help="with --teacher-force: feed the reference in chunks of B tokens")
    ap.add_argument("--temp", "--temperature", dest="temp", type=float, default=0.0)
    ap.add_argument("--top-p", "--top_p", dest="top_p", type=float, default=1.0)
    ap.add_argument("--top-k", "--top_k", dest="top_k", type=int, default=0)
    ap.add_argument("--min-p", "--min_p", dest="min_p", type=float, default=0.0)
    ap.add_argument("--repeat-penalty", "--repeat_penalty", dest="repeat_penalty", type=float, default=1.0)
    ap.add_argument("--repeat-last-n", "--repeat_last_n", dest="repeat_last_n", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--inspect", action="store_true", help="print model/hparam inventory and exit")
    ap.add_argument("--dump-tokens", action="store_true", help="oracle mode: print token IDs to stdout")
    ap.add_argument("--dump-logits", metavar="PATH", help="numeric-gate mode: dump final logit vectors")
    ap.add_argument("--teacher-force", metavar="FILE", help="feed reference token IDs, report per-step top-1 agreement")
    ap.add_argument("--dtype", choices=["bfloat16", "bf16", "float32", "fp32"], default="bfloat16")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--num-pages", type=int, default=None, help="cache pages (default: enough for one full context)")
    ap.add_argument("--max-batched-tokens", type=int, default=2048)
    ap.add_argument("--max-running", type=int, default=4, help="requests that may be live at once (default: 4)")
    ap.add_argument("--device", default="cuda:0")
    return ap


def _prompt_ids(args, model_dir) -> List[int]:
    if args.prompt_ids is not None:
        return _ids(args.prompt_ids)
    if args.prompt_ids_file:
        with open(args.prompt_ids_file) as f:
            return _ids(f.read())
    text = args.prompt
    if args.prompt_file:
        with open(args.prompt_file, encoding="utf-8") as f:
            text = f.read()
    if text is None:
        return []
    tok_path = os.path.join(model_dir, "tokenizer.json")
    try:
        from tokenizers import Tokenizer
        return Tokenizer.from_file(tok_path).encode(text).ids
    except Exception as e:  # noqa: BLE001
        raise SystemExit(f"Error: --prompt needs {tok_path} and the tokenizers package ({e}); use --prompt-ids") from None


def inspect(model_dir: str) -> None:
    from .config.registry import load_config
    from .models.model import Model
    arch, cfg = load_config(model_dir)
    model = Model(arch.model_spec(cfg))
    exp = model.expected_tensors()
    n_params = 0
    for d in exp.values():
        n = 1
        for s in d.shape:
            n *= s
        n_params += n
    print(f"architecture: {arch.name}")
    for k, v in cfg.describe().items():
        print(f"  {k}: {v}")
    print(f"tensors: {len(exp)}   parameters: {n_params:,}")
    for i, need in enumerate(model.storage_needs()):
        print(f"  cache storage {i}: {need}")


def write_logit_file(path: str, rows) -> None:
    import numpy as np
    rows = np.asarray(rows, dtype="<f4")
    with open(path, "wb") as f:
        f.write(b"CLBRLGT1")
        f.write(struct.pack("<II", rows.shape[0], rows.shape[1]))
        f.write(rows.tobytes())


def main(argv=None) -> int:
    ap = build_parser()
    try:
        args = ap.parse_args(argv)
    except SystemExit as e:
        return 2 if e.code not in (0, None) else 0
    if not args.model and not args.random:
        print("Error: --model <dir> (or --random <config.json>) is required", file=sys.stderr)
        return 2
    tmp = None
    model_dir = args.model
    try:
        if args.random:
            from .weights.random_init import write_random_model
            with open(args.random) as f:
                raw = json.load(f)
            if not model_dir:
                tmp = tempfile.TemporaryDirectory(prefix="tuff-random-")
                model_dir = tmp.name
            write_random_model(model_dir, raw, args.weight_seed)
            print(f"[tuff] random weights (seed {args.weight_seed}) written to {model_dir}", file=sys.stderr)
        if args.inspect:
            inspect(model_dir)
            return 0
        return run(args, model_dir)
    except (OSError, IOError) as e:
        print(f"[tuff] FATAL: {e}", file=sys.stderr)
        return 3
    except (ValueError, RuntimeError, KeyError) as e:
        print(f"[tuff] Error: {e}", file=sys.stderr)
        return 1
    finally:
        if tmp is not None:
            tmp.cleanup()


def run(args, model_dir: str) -> int:
    import numpy as np
    import torch

    from .engine.batch import StepEntry
    from .engine.engine import Engine
    from .sampling.params import SamplingParams
    from .sampling.sampler import SampleRow
    dump_mode = args.dump_tokens or args.dump_logits or args.teacher_force
    n_predict = args.n_predict if args.n_predict is not None else (32 if dump_mode else 128)
    prompt = _prompt_ids(args, model_dir)
    if not prompt:
        print("Error: a prompt is required (--prompt-ids, --prompt-ids-file, --prompt, --prompt-file)", file=sys.stderr)
        return 2
    budget = args.prefill_batch or args.max_batched_tokens
    max_tokens = args.num_pages * args.page_size if args.num_pages else args.ctx
    engine = Engine(model_dir, dtype=args.dtype, device=args.device, ctx_size=args.ctx, max_tokens=max_tokens,
                    page_size=args.page_size, max_batched_tokens=budget, max_running=max(1, args.max_running))
    print(f"[tuff] prompt: {len(prompt)} tokens: {' '.join(map(str, prompt[:32]))}{' ...' if len(prompt) > 32 else ''}",
          file=sys.stderr)
    sp = SamplingParams(temp=args.temp, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                        repeat_penalty=args.repeat_penalty, repeat_last_n=args.repeat_last_n, seed=args.seed,
                        max_new_tokens=n_predict)

    if args.teacher_force:
        with open(args.teacher_force) as f:
            ref = _ids(f.read())[:n_predict]
        stream = prompt + ref
        runner = engine.runner
        rc = runner.open("teacher")
        rows, agree, pos = [], 0, 0
        first = len(prompt) - 1                       # the row after the last prompt token predicts ref[0]
        while pos < len(stream) - 1 or (pos == 0 and len(stream) == 1):
            if pos < first:
                n = min(budget, first - pos)
                runner.step([StepEntry(rc, stream[pos:pos + n], [])])
            else:
                n = min(args.tf_batch, len(stream) - 1 - pos)
                lg = runner.step([StepEntry(rc, stream[pos:pos + n], list(range(n)))]).cpu().numpy()
                for j in range(n):
                    i = pos + j - first
                    agree += int(lg[j].argmax() == ref[i])
                    rows.append(lg[j])
            pos += n
        runner.close(rc)
        print(f"[tuff] teacher-forced top-1 agreement: {agree}/{len(rows)}", file=sys.stderr)
        if args.dump_logits:
            write_logit_file(args.dump_logits, rows)
        return 0

    if args.dump_tokens or args.dump_logits:
        if args.dump_logits:
            runner = engine.runner
            rc = runner.open("dump")
            toks, rows = list(prompt), []
            lg = runner.step([StepEntry(rc, toks, [len(toks) - 1])])
            for _ in range(n_predict):
                rows.append(lg[0].cpu().numpy())
                nxt = int(engine.sampler.sample(lg, [SampleRow(sp, 0, len(toks) - len(prompt), toks)])[0])
                toks.append(nxt)
                lg = runner.step([StepEntry(rc, [nxt], [0])])
            runner.close(rc)
            write_logit_file(args.dump_logits, rows)
            out = toks[len(prompt):]
        else:
            out = engine.generate([prompt], sp)[0]
        if args.dump_tokens:
            print("\n".join(str(t) for t in out))
        return 0

    # timed generation: warm-up tokens, then n timed tokens, several runs
    speeds = []
    out: List[int] = []
    for run_i in range(max(1, args.runs)):
        req = engine.add_request(("run", run_i), prompt, SamplingParams(**{**sp.__dict__,
                                                                          "max_new_tokens": args.warmup + n_predict}))
        t0 = None
        while engine.scheduler.has_work():
            if t0 is None and len(req.output) >= args.warmup:
                torch.cuda.synchronize()
                t0, base = time.perf_counter(), len(req.output)
            engine.step()
        torch.cuda.synchronize()
        if t0 is not None and len(req.output) > base:
            speeds.append((len(req.output) - base) / (time.perf_counter() - t0))
        out = req.output[args.warmup:]
        print(f"[tuff] run {run_i}: {speeds[-1] if speeds else float('nan'):.2f} tok/s", file=sys.stderr)
    print(" ".join(str(t) for t in out))
    if speeds:
        mean = float(np.mean(speeds))
        spread = (max(speeds) - min(speeds)) / 2.0
        print("\n========================================================================", file=sys.stderr)
        print(f" Pipeline Generation Speed: {mean:.2f} +/- {spread:.2f} tok/s (mean of {len(speeds)} runs, "
              f"{args.warmup} warmup + {n_predict} timed)", file=sys.stderr)
        print(f" VRAM: {torch.cuda.max_memory_allocated() / 2**20:.1f} MiB used", file=sys.stderr)
        print("========================================================================", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
