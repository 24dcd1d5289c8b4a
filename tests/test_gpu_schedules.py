"""Schedules that the measurements run and the other tests do not reach: decoding steps with
many live rows (17, 33, 64: CUDA graphs of that many rows, the swapped split-K tensor-core
products, the sliced attention over many rows), long contexts in the sliced attention, one step
of 2,048 tokens at the real layer sizes, CUDA graphs replayed after other steps have run between,
and the kernels' status word read by generation."""
import io
import json

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from tiny import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu
MARGIN = {"float32": 1e-4, "bfloat16": 6e-2}

REAL_WIDTH = dict(
    architectures=["Lfm2ForCausalLM"], hidden_size=2048, num_hidden_layers=4, num_attention_heads=32,
    num_key_value_heads=8, intermediate_size=8192, block_auto_adjust_ff_dim=True, block_multiple_of=256,
    vocab_size=65536, rope_theta=1e6, norm_eps=1e-5, conv_L_cache=3, full_attn_idxs=[1, 3], tie_embedding=True)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from tuff_b200.weights import write_random_model
    base = tmp_path_factory.mktemp("sched")
    out = {"tiny_d": make_folder(base, "tiny_d")}
    out["real_width"] = write_random_model(str(base / "real_width"), REAL_WIDTH, 11)
    return out


def greedy_ok(model, prompt, out, dtype):
    ref = model.forward(prompt + out, rows=[len(prompt) + i - 1 for i in range(len(out))])
    for i, tok in enumerate(out):
        assert ref[i].max() - ref[i][tok] <= MARGIN[dtype], (i, tok, int(ref[i].argmax()), ref[i].max() - ref[i][tok])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,rows,checked", [("tiny_d", 9, 9), ("tiny_d", 17, 17), ("tiny_d", 33, 33), ("tiny_d", 64, 64),
                                              ("real_width", 12, 4), ("real_width", 17, 5), ("real_width", 64, 6)])
def test_decoding_with_many_live_rows(folders, name, rows, checked, dtype):
    """`rows` requests decode together (graphs on, steps launched ahead); every token of the checked
    requests is the plain implementation's greedy choice or a near-tie of it."""
    from tuff_b200 import Engine, SamplingParams
    from tuff_b200.kernels import ops
    cfg = CONFIGS[name][0] if name in CONFIGS else REAL_WIDTH
    vocab = cfg["vocab_size"]
    prompts = [random_tokens(vocab, 3 + (i * 7) % 11, 500 + i) for i in range(rows)]
    n_new = 7
    eng = Engine(folders[name], dtype=dtype, ctx_size=64, max_tokens=rows * 64, page_size=64 if name == "real_width" else 8,
                 max_batched_tokens=2048, max_running=rows)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=n_new))
    ops.check_tc_status()
    assert [len(o) for o in outs] == [n_new] * rows
    assert eng.runner.graph_replays > 0 and rows in eng.runner._graphs        # the captured step of `rows` rows ran
    model = plain.PlainLfm2(folders[name])
    step = max(1, rows // checked)
    for i in range(0, rows, step):
        greedy_ok(model, prompts[i], outs[i], dtype)
    eng.runner.cache.check()


@pytest.mark.parametrize("context,rows,bound", [(4097, 2, 8192), (8192, 1, 8192), (100, 2, 8192), (700, 3, 1024)])
def test_sliced_attention_at_long_contexts(context, rows, bound):
    """The sliced decode attention (32 heads in 8 groups of 64, pages of 64) over contexts of thousands
    of keys, and a short context inside a launch that is sized for a long one, against fp64.  One
    far key carries a large score, so a slice that is skipped or merged wrongly shows."""
    from tuff_b200.kernels import ops
    H, G, hd, ps = 32, 8, 64, 64
    rng = np.random.default_rng(31)
    blocks = -(-context // ps)
    n_pages = rows * blocks + 3
    k = rng.normal(size=(n_pages, G, ps, hd)) * 0.3
    v = rng.normal(size=(n_pages, G, ps, hd))
    perm = rng.permutation(n_pages)[: rows * blocks].reshape(rows, blocks)
    q = rng.normal(size=(rows, H, hd)) * 0.3
    far = [min(context - 1, 5 + 37 * r) for r in range(rows)]
    for r in range(rows):                                   # key `far[r]` of row r matches its queries
        page, off = perm[r, far[r] // ps], far[r] % ps
        for g in range(G):
            k[page, g, off] = q[r, g * (H // G)] * 8
    kp = torch.as_tensor(k).to(torch.bfloat16).cuda()
    vp = torch.as_tensor(v).to(torch.bfloat16).cuda()
    qd = torch.as_tensor(q.reshape(rows, H * hd)).to(torch.bfloat16).cuda()
    out = torch.full((rows, H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    table = torch.as_tensor(perm.astype(np.int32)).cuda()
    pos = torch.full((rows,), context - 1, dtype=torch.int32, device="cuda")
    row_of = torch.arange(rows, dtype=torch.int32, device="cuda")
    ops.attention_decode(qd, kp, vp, table, pos, row_of, out, H, G, hd, hd ** -0.5, 0, bound)
    ops.check_tc_status()
    k64, v64, q64 = kp.double().cpu().numpy(), vp.double().cpu().numpy(), qd.double().cpu().numpy().reshape(rows, H, hd)
    got = out.double().cpu().numpy().reshape(rows, H, hd)
    for r in range(rows):
        keys = np.concatenate([k64[p] for p in perm[r]], axis=1)[:, :context]        # [G, context, hd]
        vals = np.concatenate([v64[p] for p in perm[r]], axis=1)[:, :context]
        for h in range(H):
            g = h // (H // G)
            s = keys[g] @ q64[r, h] * hd ** -0.5
            w = np.exp(s - s.max()); w /= w.sum()
            ref = w @ vals[g]
            assert np.abs(got[r, h] - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max()), (r, h)


@pytest.mark.parametrize("dtype,tol", [("bfloat16", 5e-2), ("float32", 2e-4)])
def test_one_step_of_2048_tokens_at_real_width(folders, dtype, tol):
    """A whole 2,048-token prompt in one step (16 query blocks of the tensor-core attention, 128 x 256
    tiles of the products at 2,048 rows) against the plain implementation at sampled positions."""
    from tuff_b200.engine import ModelRunner, StepEntry
    from tuff_b200.kernels import ops
    T = 2048
    toks = random_tokens(65536, T, 77)
    want = [0, 1, 63, 64, 127, 128, 129, 255, 256, 1023, 1024, 1500, 1919, 1920, 2046, 2047]
    runner = ModelRunner(folders["real_width"], dtype=dtype, max_tokens=T + 64, page_size=64, max_requests=2)
    rc = runner.open("long")
    logits = runner.step([StepEntry(rc, toks, want)]).cpu().numpy()
    ops.check_tc_status()
    ref = plain.PlainLfm2(folders["real_width"]).forward(toks, rows=want)
    for i, p in enumerate(want):
        err = np.abs(logits[i] - ref[i]).max()
        assert err <= tol * max(1.0, np.abs(ref[i]).max()), (dtype, p, err)
    runner.close(rc)
    runner.cache.check()


def test_captured_steps_survive_other_steps_between(folders):
    """Graphs captured at 8..1 rows, then a prompt portion of 100 tokens (which needs the split-K and
    attention workspaces at other sizes), then the same 8 requests again: the replayed graphs still
    write where the kernels read (the workspaces never move), so the tokens equal those of plain launches."""
    from tuff_b200 import Engine, SamplingParams
    name = "tiny_d"
    vocab = CONFIGS[name][0]["vocab_size"]
    prompts = [random_tokens(vocab, 4 + i, 900 + i) for i in range(8)]
    lens = [SamplingParams(max_new_tokens=5 + 2 * i) for i in range(8)]       # the rows shrink from 8 to 1
    long_prompt = random_tokens(vocab, 100, 990)

    def run(graphs):
        eng = Engine(folders[name], dtype="bfloat16", ctx_size=160, max_tokens=2048, page_size=8,
                     max_batched_tokens=128, max_running=8, cuda_graphs=graphs, run_ahead=graphs)
        first = eng.generate(prompts, lens)
        mid = eng.generate([long_prompt], SamplingParams(max_new_tokens=4))
        again = eng.generate(prompts, lens)
        eng.runner.cache.check()
        return first, mid, again, eng.runner.graph_replays

    f1, m1, a1, replays = run(True)
    f0, m0, a0, none = run(False)
    assert replays > 0 and none == 0
    assert f1 == f0 and m1 == m0 and a1 == a0 and f1 == a1


def test_generation_reads_the_status_word(folders):
    """A kernel whose bounded wait ran out leaves a code in the status word; the step that reads its
    sampled ids raises, and the engine has given back every page and slot."""
    from tuff_b200 import Engine, SamplingParams
    from tuff_b200.kernels import ops
    name = "tiny_d"
    vocab = CONFIGS[name][0]["vocab_size"]
    eng = Engine(folders[name], dtype="bfloat16", ctx_size=64, max_tokens=256, page_size=8, max_running=4)
    eng.add_request("r", random_tokens(vocab, 9, 1), SamplingParams(max_new_tokens=4))
    eng.step()
    word = ops.status_word(eng.runner.device)
    word.fill_(63)                                           # as a consumer's wait that ran out would
    try:
        with pytest.raises(ops.KernelError):
            while eng.scheduler.has_work():
                eng.step()
    finally:
        word.zero_()
    assert not eng.scheduler.has_work() and not eng.runner.cache.live
    eng.runner.cache.check()
    # trace replay checks the word after it has copied the logits
    from tuff_b200.engine.replay import replay
    word.fill_(2)
    try:
        with pytest.raises(ops.KernelError):
            replay(eng.runner, io.StringIO(json.dumps(dict(step=0, entries=[dict(id="a", tokens=[1, 2], want=[1])], end=["a"])) + "\n"),
                   str(folders[name]) + "_out", report=io.StringIO())
    finally:
        word.zero_()
