"""Trace replay on the GPU against the plain implementation: the same requests
whole, with the last 32 tokens decoded one by one, in portions of changing size,
and mixed with other requests in a pool so small that pages are used again; in
32-bit and in bfloat16."""
import io
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_lfm2 as plain
import traces
from tiny import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Logits of these models are of order 1.  The 32-bit engine differs from the float64 plain
# implementation by rounding of fp32 sums; the bfloat16 engine by bf16 rounding of weights'
# products' inputs (activations, keys and values), layer after layer.
TOL = {"float32": dict(atol=1e-4, rtol=1e-4), "bfloat16": dict(atol=4e-2, rtol=4e-2)}

LENGTHS = {"tiny_a": (70, 45, 97, 130, 66), "tiny_b": (83, 40, 129, 65, 100), "tiny_c": (64, 33, 90, 47, 128),
           "tiny_d": (150, 64, 37, 193, 129)}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    out = {}
    for name in CONFIGS:
        folder = make_folder(base, name)
        cfg = CONFIGS[name][0]
        reqs = {f"r{i}": random_tokens(cfg["vocab_size"], n, 10 * i + len(name)) for i, n in enumerate(LENGTHS[name])}
        expect = {rid: plain.PlainLfm2(folder).forward(t) for rid, t in reqs.items()}
        out[name] = (folder, reqs, expect)
    return out


def run_trace(folder, dtype, steps, tmp_path, page_size=16, max_tokens=None):
    from tuff_b200.engine.replay import replay
    from tuff_b200.engine.runner import ModelRunner
    n = max_tokens or traces.tokens_needed(steps)
    runner = ModelRunner(folder, dtype=dtype, max_tokens=n, page_size=page_size, max_requests=4)
    runner.cache.owners = {}                      # log every hand-out of a page
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    log = io.StringIO()
    replay(runner, io.StringIO(text), str(tmp_path), report=log)
    assert log.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
    runner.cache.check()
    assert not runner.cache.live
    return runner


def compare(out_dir, wanted, expect, vocab, dtype, what):
    worst = 0.0
    for step, rows in wanted.items():
        got = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for i, (rid, pos) in enumerate(rows):
            ref = expect[rid][pos]
            err = np.abs(got[i] - ref)
            worst = max(worst, float(err.max()))
            bad = err > TOL[dtype]["atol"] + TOL[dtype]["rtol"] * np.abs(ref)
            assert not bad.any(), (f"{what} {dtype}: request {rid} position {pos} (step {step}): "
                                   f"max error {err.max():.3g} at token {int(err.argmax())}")
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("mode", ["whole", "tail_decoded", "portions", "mixed"])
def test_replay_modes(models, tmp_path, name, dtype, mode):
    folder, reqs, expect = models[name]
    vocab = CONFIGS[name][0]["vocab_size"]
    steps, wanted = getattr(traces, mode)(reqs)
    page = {"tiny_a": 16, "tiny_b": 4, "tiny_c": 8, "tiny_d": 8}[name]
    runner = run_trace(folder, dtype, steps, tmp_path, page_size=page)
    compare(str(tmp_path), wanted, expect, vocab, dtype, f"{name} {mode}")
    if mode == "mixed":
        # pages were used again: the pool's own log shows pages that two different requests held
        reused = [k for k, who in runner.cache.owners.items() if len(set(who)) > 1]
        assert len(reused) >= 2, runner.cache.owners


def logits_by_place(out_dir, wanted, vocab):
    out = {}
    for step, rows in wanted.items():
        got = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for i, place in enumerate(rows):
            out[place] = got[i].copy()
    return out


@pytest.mark.parametrize("name", list(CONFIGS))
def test_float32_logits_are_bitwise_equal_in_every_mode(models, tmp_path, name):
    """The 32-bit path adds in an order that depends on sizes only: the logits of a (request, position)
    are the same bits whether the request ran whole, with its tail decoded, in portions, or mixed with
    others in reused pages (the reference's gate: tests/verify_lfm25_prefill.sh:28-54 compares its batched
    and its one-by-one prefill with `cmp`, tests/verify_lfm25_golden.sh:247-272 hashes every logits row
    under every execution mode)."""
    folder, reqs, _ = models[name]
    vocab = CONFIGS[name][0]["vocab_size"]
    page = {"tiny_a": 16, "tiny_b": 4, "tiny_c": 8, "tiny_d": 8}[name]
    seen = {}
    for mode in ("whole", "tail_decoded", "portions", "mixed"):
        steps, wanted = getattr(traces, mode)(reqs)
        out = tmp_path / mode
        run_trace(folder, "float32", steps, out, page_size=page)
        for place, row in logits_by_place(str(out), wanted, vocab).items():
            if place in seen:
                same = np.array_equal(seen[place][1].view(np.uint32), row.view(np.uint32))
                assert same, (f"{name}: request {place[0]} position {place[1]} differs between {seen[place][0]} and {mode}: "
                              f"max difference {np.abs(seen[place][1] - row).max():.3g}")
            else:
                seen[place] = (mode, row)
    assert len(seen) == sum(len(t) for t in reqs.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    """bin/trace_run as a program: reads the trace from standard input, answers `done <step>`."""
    folder, reqs, expect = models["tiny_b"]
    steps, wanted = traces.mixed(reqs, seed=3)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(traces.tokens_needed(steps))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True, capture_output=True,
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    compare(str(out), wanted, expect, CONFIGS["tiny_b"][0]["vocab_size"], dtype, "trace_run mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_range_checking_build_finds_nothing_on_a_mixed_trace(models, tmp_path, dtype):
    """The build whose kernels range-check every table row, page id and state slot they are given
    (TUFF_DEBUG_BOUNDS=1), as a program over a mixed trace with reused pages: it ends without a code in the
    status word (trace_run reads it after every step) and writes the very logits of the normal build."""
    folder, reqs, expect = models["tiny_d"]
    steps, wanted = traces.mixed(reqs, seed=5)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    outs = {}
    for name, env in (("normal", {}), ("checked", {"TUFF_DEBUG_BOUNDS": "1"})):
        out = tmp_path / name
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                               "--out", str(out), "--max-tokens", str(traces.tokens_needed(steps))],
                              input=text, text=True, capture_output=True, timeout=1500, env={**os.environ, **env})
        assert proc.returncode == 0, proc.stderr[-2000:]
        outs[name] = logits_by_place(str(out), wanted, CONFIGS["tiny_d"][0]["vocab_size"])
    compare(str(tmp_path / "checked"), wanted, expect, CONFIGS["tiny_d"][0]["vocab_size"], dtype, "checked build")
    for place, row in outs["normal"].items():
        assert np.array_equal(row.view(np.uint32), outs["checked"][place].view(np.uint32)), place
