"""Trace replay: feeds given token ids through the model step by step and writes
logits; it samples nothing.

It drives the same `ModelRunner.step`, cache manager and kernels as generation.
The reference's counterpart is `--teacher-force <ids> --dump-logits <file>` for
its single sequence (src/main.c:1277-1546); here a trace holds several requests
and says for every step which tokens of which request run together.

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step that wants logits, `<out>/<step>.f32` receives them as little-endian
float32 [wanted, vocab], in the order of the entries and of `want`.  After every
step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

from ..cache.manager import RequestCache
from ..kernels import ops
from .batch import StepEntry
from .runner import ModelRunner


class TraceError(ValueError):
    pass


def replay(runner: ModelRunner, lines: IO[str], out_dir: str, report: IO[str] = sys.stdout) -> int:
    os.makedirs(out_dir, exist_ok=True)
    live: Dict[str, RequestCache] = {}
    n_steps = 0
    for raw in lines:
        raw = raw.strip()
        if not raw:
            continue
        try:
            rec = json.loads(raw)
            step = rec["step"]
            entries_in = rec.get("entries", [])
            ends = rec.get("end", [])
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            raise TraceError(f"bad trace line {raw[:80]!r}: {e}") from None
        entries = []
        for e in entries_in:
            rid = str(e["id"])
            if rid not in live:
                live[rid] = runner.open(rid)
            entries.append(StepEntry(live[rid], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                ops.check_tc_status()          # the copy has waited for the step: a wait that ran out shows here
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for rid in ends:
            rid = str(rid)
            if rid not in live:
                raise TraceError(f"step {step}: request {rid!r} ends but is not live")
            runner.close(live.pop(rid))
        n_steps += 1
        print(f"done {step}", file=report, flush=True)
    return n_steps
