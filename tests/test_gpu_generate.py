"""Generation through the Python entry point and the command line, the scheduler on
the GPU (preemption does not change outputs), long decoding, and the first tokens of
a sequence."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from tiny import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MARGIN = {"float32": 1e-4, "bfloat16": 6e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("gen")
    return {n: make_folder(base, n) for n in CONFIGS}


def check_greedy(folder, prompt, out, dtype):
    """Every generated token is the plain implementation's greedy choice given the tokens before
    it, or within the dtype's margin of it (a near-tie)."""
    ref = plain.PlainLfm2(folder).forward(prompt + out)
    for i, tok in enumerate(out):
        row = ref[len(prompt) + i - 1]
        assert row.max() - row[tok] <= MARGIN[dtype], (i, tok, int(row.argmax()), row.max() - row[tok])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from tuff_b200 import Engine, SamplingParams
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 40 + n) for n in (7, 13, 1, 30)]
    eng = Engine(folders[name], dtype=dtype, ctx_size=128, max_tokens=256, page_size=8, max_batched_tokens=16)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=8))
    assert [len(o) for o in outs] == [8] * 4
    for p, o in zip(prompts, outs):
        check_greedy(folders[name], p, o, dtype)
    eng.runner.cache.check()
    assert not eng.runner.cache.live and eng.stats()["decode_tokens"] == 32


def test_batching_and_preemption_do_not_change_outputs(folders):
    """The same requests alone, batched, and in a pool so small that requests are preempted and
    recomputed: the same tokens every time, greedy and sampled (fp32, where runs are comparable)."""
    from tuff_b200 import Engine, SamplingParams
    name = "tiny_b"
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 70 + n) for n in (5, 17, 31)]
    params = [SamplingParams(max_new_tokens=12), SamplingParams(temp=0.8, seed=2, max_new_tokens=12),
              SamplingParams(temp=1.1, top_k=20, top_p=0.9, seed=5, max_new_tokens=12)]

    def run(max_tokens, budget, together):
        eng = Engine(folders[name], dtype="float32", ctx_size=64, max_tokens=max_tokens, page_size=4,
                     max_batched_tokens=budget, max_running=4)
        if together:
            reqs = [eng.add_request(i, p, sp) for i, (p, sp) in enumerate(zip(prompts, params))]
            while eng.scheduler.has_work():
                eng.step()
            outs = [r.output for r in reqs]
        else:
            outs = []
            for i, (p, sp) in enumerate(zip(prompts, params)):
                eng.scheduler._next_key = i          # the same request number as in the batched run
                r = eng.add_request(i, p, sp)
                while eng.scheduler.has_work():
                    eng.step()
                outs.append(r.output)
        eng.runner.cache.check()
        return outs, eng.stats()

    alone, _ = run(256, 64, together=False)
    batched, s1 = run(256, 4, together=True)          # chunks of 4 mixed with decode tokens
    tight, s2 = run(64, 64, together=True)            # 16 pages for 3 requests that need 5+8+11
    assert s1["preemptions"] == 0 and s2["preemptions"] >= 1
    assert alone == batched == tight
    check_greedy(folders[name], prompts[0], alone[0], "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_of_the_sampled_ids_changes_nothing(folders, dtype):
    """Decoding steps launched before the ids of the step before them were read (their input ids
    stay on the device) give the same tokens as the plain loop: greedy and sampled, requests of
    different lengths that leave the batch one by one, a stop token met in mid-flight (its
    request has then run one step too many), and a request that arrives while others decode."""
    from tuff_b200 import Engine, SamplingParams
    name = "tiny_d"
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 90 + n) for n in (6, 19, 33, 11)]

    def make(run_ahead):
        return Engine(folders[name], dtype=dtype, ctx_size=160, max_tokens=1024, page_size=8, max_batched_tokens=32,
                      max_running=8, run_ahead=run_ahead)

    # a first run finds tokens that requests 0 and 2 will emit in mid-flight: they become their stop tokens
    probe = make(False).generate(prompts, [SamplingParams(max_new_tokens=40), SamplingParams(temp=0.9, seed=3, max_new_tokens=25),
                                           SamplingParams(max_new_tokens=33), SamplingParams(temp=1.2, top_k=12, seed=8, max_new_tokens=17)])
    stop0, stop2 = probe[0][13], probe[2][20]
    params = [SamplingParams(max_new_tokens=40, stop_token_ids=(stop0,)), SamplingParams(temp=0.9, seed=3, max_new_tokens=25),
              SamplingParams(max_new_tokens=33, stop_token_ids=(stop2,)), SamplingParams(temp=1.2, top_k=12, seed=8, max_new_tokens=17)]
    late_prompt = random_tokens(vocab, 9, 5)

    def run(run_ahead):
        eng = make(run_ahead)
        reqs = [eng.add_request(i, p, sp) for i, (p, sp) in enumerate(zip(prompts, params))]
        steps, late = 0, None
        while eng.scheduler.has_work():
            eng.step()
            steps += 1
            if steps == 9:
                late = eng.add_request("late", late_prompt, SamplingParams(max_new_tokens=14))
        eng.runner.cache.check()
        assert not eng.runner.cache.live and eng._ahead is None
        return [r.output for r in reqs] + [late.output], [r.finish_reason for r in reqs], eng

    plain_outs, plain_why, _ = run(False)
    ahead_outs, ahead_why, eng = run(True)
    assert ahead_outs == plain_outs and ahead_why == plain_why
    assert plain_why[0] == "stop" and plain_why[2] == "stop" and plain_why[1] == "length"
    assert len(plain_outs[0]) <= 14 and plain_outs[0][-1] == stop0
    assert eng.run_ahead and eng.timing["steps"] >= len(plain_outs[1])


def test_running_ahead_under_pressure(folders):
    """Twelve requests of random lengths arriving over time into a pool that cannot hold them all
    (requests are preempted and recomputed), greedy and sampled: with and without steps launched
    ahead, the same tokens, and the cache manager's books stay right."""
    from tuff_b200 import Engine, SamplingParams
    name = "tiny_a"
    vocab = CONFIGS[name][0]["vocab_size"]
    rng = np.random.default_rng(77)
    jobs = []
    for i in range(12):
        n_p, n_new = int(rng.integers(1, 40)), int(rng.integers(5, 30))
        sp = SamplingParams(max_new_tokens=n_new) if i % 3 else SamplingParams(temp=0.9, top_p=0.95, seed=10 + i, max_new_tokens=n_new)
        jobs.append((int(rng.integers(0, 25)), random_tokens(vocab, n_p, 300 + i), sp))

    def run(run_ahead):
        eng = Engine(folders[name], dtype="float32", ctx_size=80, max_tokens=200, page_size=4, max_batched_tokens=24,
                     max_running=6, run_ahead=run_ahead)
        reqs, step = {}, 0
        while len(reqs) < len(jobs) or eng.scheduler.has_work():
            for i, (at, prompt, sp) in enumerate(jobs):
                if at == step:
                    eng.scheduler._next_key = i
                    reqs[i] = eng.add_request(i, prompt, sp)
            eng.step()
            step += 1
            if step % 7 == 0:
                eng.runner.cache.check()
        eng.runner.cache.check()
        assert not eng.runner.cache.live
        return [reqs[i].output for i in range(len(jobs))], eng.stats()

    plain_outs, s0 = run(False)
    ahead_outs, s1 = run(True)
    assert plain_outs == ahead_outs
    assert s0["preemptions"] >= 1 and all(len(o) == j[2].max_new_tokens for o, j in zip(plain_outs, jobs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_plain_logits(folders, dtype):
    """300 tokens decoded one by one (pages fill up, many pages per request): the logits still
    match the whole-sequence computation at the end."""
    from tuff_b200.engine import ModelRunner, StepEntry
    folder = folders["tiny_a"]
    toks = random_tokens(256, 300, 5)
    ref = plain.PlainLfm2(folder).forward(toks)
    runner = ModelRunner(folder, dtype=dtype, max_tokens=320, page_size=16, max_requests=2)
    rc = runner.open("long")
    rows = {}
    for p, t in enumerate(toks):
        lg = runner.step([StepEntry(rc, [t], [0] if p % 37 == 0 or p >= 290 else [])])
        if lg.shape[0]:
            rows[p] = lg[0].double().cpu().numpy()
    tol = 1e-4 if dtype == "float32" else 4e-2
    for p, row in rows.items():
        assert np.abs(row - ref[p]).max() <= tol * max(1, np.abs(ref[p]).max()), p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_c"])
def test_first_tokens_of_a_sequence(folders, name, dtype):
    """Positions 0, 1, 2 (no history, less history than convolution taps) alone and as one portion."""
    from tuff_b200.engine import ModelRunner, StepEntry
    vocab = CONFIGS[name][0]["vocab_size"]
    toks = random_tokens(vocab, 3, 9)
    ref = plain.PlainLfm2(folders[name]).forward(toks)
    runner = ModelRunner(folders[name], dtype=dtype, max_tokens=64, page_size=2, max_requests=2)
    a, b = runner.open("a"), runner.open("b")
    one = torch.cat([runner.step([StepEntry(a, [t], [0])]) for t in toks]).double().cpu().numpy()
    whole = runner.step([StepEntry(b, toks, [0, 1, 2])]).double().cpu().numpy()
    tol = 1e-4 if dtype == "float32" else 4e-2
    assert np.abs(one - ref).max() <= tol and np.abs(whole - ref).max() <= tol


def test_step_refuses_bad_batches(folders):
    from tuff_b200.cache import OutOfPages
    from tuff_b200.engine import BatchError, ModelRunner, StepEntry
    runner = ModelRunner(folders["tiny_a"], dtype="float32", max_tokens=16, page_size=4, max_requests=2,
                         max_context=12)
    a = runner.open("a")
    for bad in ([StepEntry(a, [], [])], [StepEntry(a, [256], [0])], [StepEntry(a, [1, 2], [2])],
                [StepEntry(a, [1], [0]), StepEntry(a, [2], [0])], [StepEntry(a, list(range(13)), [])], []):
        with pytest.raises(BatchError):
            runner.step(bad)
    b = runner.open("b")
    runner.step([StepEntry(a, list(range(10)), [])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry(a, [1], [0]), StepEntry(b, list(range(9)), [])])   # 3 pages held, 1 + 3 wanted
    assert a.n_tokens == 10 and b.n_tokens == 0 and a.reserved == 0 and b.reserved == 0
    runner.cache.check()
    assert runner.step([StepEntry(a, [1], [0])]).shape == (1, 256)      # nothing was lost by the refusal


def test_command_line(folders, tmp_path):
    import json
    tuff = os.path.join(ROOT, "bin", "tuff")
    folder = folders["tiny_a"]
    prompt = random_tokens(256, 9, 3)
    ids = " ".join(map(str, prompt))
    r = subprocess.run([sys.executable, tuff, "--model", folder, "--prompt-ids", ids, "-n", "6", "--dump-tokens",
                        "--dtype", "float32", "-c", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-1500:]
    out = [int(t) for t in r.stdout.split()]
    assert len(out) == 6
    check_greedy(folder, prompt, out, "float32")
    # teacher-forced logits in the reference's container format
    (tmp_path / "ref.txt").write_text("\n".join(map(str, out)))
    dump = tmp_path / "logits.bin"
    r = subprocess.run([sys.executable, tuff, "--model", folder, "--prompt-ids", ids, "-n", "6", "--teacher-force",
                        str(tmp_path / "ref.txt"), "--tf-batch", "4", "--dump-logits", str(dump), "--dtype", "float32",
                        "-c", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "agreement: 6/6" in r.stderr, r.stderr[-1500:]
    raw = dump.read_bytes()
    assert raw[:8] == b"CLBRLGT1" and np.frombuffer(raw[8:16], "<u4").tolist() == [6, 256]
    rows = np.frombuffer(raw[16:], "<f4").reshape(6, 256)
    ref = plain.PlainLfm2(folder).forward(prompt + out)
    assert np.abs(rows - ref[len(prompt) - 1:len(prompt) + 5]).max() < 1e-4
    # timed mode with sampling options, a random model written on the fly, usage errors
    cfgp = tmp_path / "cfg.json"
    cfgp.write_text(json.dumps(CONFIGS["tiny_c"][0]))
    r = subprocess.run([sys.executable, tuff, "--random", str(cfgp), "--weight-seed", "2", "--prompt-ids", "1,2,3", "-n", "5",
                        "--warmup", "2", "--runs", "2", "--temp", "0.8", "--top-k", "10", "--seed", "4", "-c", "64"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "Pipeline Generation Speed" in r.stderr and len(r.stdout.split()) == 5, r.stderr[-1500:]
    assert subprocess.run([sys.executable, tuff, "--prompt-ids", "1"], capture_output=True).returncode == 2
    r = subprocess.run([sys.executable, tuff, "--model", str(tmp_path / "nothing"), "--prompt-ids", "1"], capture_output=True)
    assert r.returncode in (1, 3)
