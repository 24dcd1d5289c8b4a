"""The parts alone (each against the plain implementation's function), schedules
that name a layer twice or let a layer read another layer's cache, and a toy
mixer with state of its own that is registered, built and stepped from this
file alone."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from tuff_b200.cache import CacheManager
from tuff_b200.engine.batch import StepEntry, layout_entries, to_device

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(dtype).cuda()


def f64(t):
    return t.double().cpu().numpy()


def close(got, ref, dtype, scale=1.0):
    err = np.abs(f64(got) - ref).max()
    assert err <= TOL[dtype] * scale * max(1.0, np.abs(ref).max()), f"max error {err:.3g}"


def bind_random(part, dtype, rng, std=0.05):
    w = {}
    for n, d in part.weight_decls().items():
        a = 1 + 0.1 * rng.normal(size=d.shape) if d.init == "norm" else std * rng.normal(size=d.shape)
        w[n] = dev(a, torch.float32 if d.role == "vector" else DT[dtype])
    part.bind(dict(w), DT[dtype])
    return {n: f64(t) for n, t in w.items()}


def make_ctx(cm, dtype, portions, vocab=100):
    """portions: list of (request cache, n tokens); reserves pages and lays the step out."""
    entries = [StepEntry(rc, [1] * n, []) for rc, n in portions]
    for e in entries:
        cm.reserve(e.cache, len(e.tokens))
    return to_device(layout_entries(entries, cm), torch.device("cuda:0"), DT[dtype]), entries


def run_part_in_portions(part, cm, storage, dtype, hs, cuts):
    """Feeds each sequence of `hs` through `part` (a mixer) cut at `cuts`, several requests per step."""
    rcs = [cm.open(i) for i in range(len(hs))]
    outs = [[] for _ in hs]
    pos = [0] * len(hs)
    while any(p < len(h) for p, h in zip(pos, hs)):
        step = []
        for i, h in enumerate(hs):
            if pos[i] < len(h):
                n = min(cuts[(pos[i] + i) % len(cuts)], len(h) - pos[i])
                step.append((i, n))
        ctx, entries = make_ctx(cm, dtype, [(rcs[i], n) for i, n in step])
        x = torch.cat([dev(hs[i][pos[i]:pos[i] + n], DT[dtype]) for i, n in step])
        res = torch.zeros(x.shape[0], x.shape[1], device="cuda")
        part.forward(ctx, storage, x, res)
        o = 0
        for (i, n), e in zip(step, entries):
            outs[i].append(f64(res[o:o + n]))
            cm.commit(e.cache, n)
            pos[i] += n
            o += n
    for rc in rcs:
        cm.close(rc)
    return [np.concatenate(o) for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,K", [(80, 3), (48, 4), (112, 2)])
def test_gated_short_conv_part(dtype, d, K):
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(0)
    part = MIXERS.build(PartSpec("gated_short_conv", dict(d_model=d, kernel_size=K)))
    w = bind_random(part, dtype, rng, std=0.2)
    cm = CacheManager([part.cache_need()], page_size=4, max_tokens=64, max_requests=3, dtype=DT[dtype], device="cuda:0")
    hs = [f64(dev(rng.normal(size=(n, d)), DT[dtype])) for n in (23, 9, 14)]
    got = run_part_in_portions(part, cm, cm.storages[0], dtype, hs, cuts=(1, 5, 2, 3, 1, 1, 8))
    for g, h in zip(got, hs):
        ref = plain.short_conv_mixer(h, w["in_proj"], w["conv"].reshape(d, K), w["out_proj"])
        err = np.abs(g - ref).max()
        assert err <= TOL[dtype] * 2 * max(1, np.abs(ref).max()), err


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,H,G,hd,page,window", [(64, 4, 2, 16, 4, None), (80, 6, 3, 48, 8, None), (96, 4, 1, 32, 2, 7),
                                                  (72, 2, 2, 64, 16, None)])
def test_gqa_attention_part(dtype, d, H, G, hd, page, window):
    from tuff_b200.parts import MIXERS, PartSpec
    rng = np.random.default_rng(1)
    theta, eps = 5e4, 1e-6
    part = MIXERS.build(PartSpec("gqa_attention", dict(
        d_model=d, num_heads=H, num_kv_heads=G, head_dim=hd, qk_norm_eps=eps, window=window,
        position_encoding=PartSpec("rope_neox", dict(head_dim=hd, theta=theta)))))
    w = bind_random(part, dtype, rng, std=0.3)
    cm = CacheManager([part.cache_need()], page_size=page, max_tokens=128, max_requests=3, dtype=DT[dtype],
                      device="cuda:0")
    hs = [f64(dev(rng.normal(size=(n, d)), DT[dtype])) for n in (41, 6, 30)]
    got = run_part_in_portions(part, cm, cm.storages[0], dtype, hs, cuts=(3, 1, 7, 2, 1, 12))
    for g, h in zip(got, hs):
        ref = plain.gqa_attention_mixer(h, w["q_proj"], w["k_proj"], w["v_proj"], w["out_proj"], w["q_layernorm"],
                                        w["k_layernorm"], H, G, hd, eps, theta, window=window)
        err = np.abs(g - ref).max()
        assert err <= TOL[dtype] * 4 * max(1, np.abs(ref).max()), err
    cm.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_norm_embedding_head_parts(dtype):
    from tuff_b200.parts import EMBEDDINGS, FEED_FORWARDS, HEADS, NORMS, PartSpec
    rng = np.random.default_rng(2)
    d, F, V, T = 80, 200, 301, 11
    ffn = FEED_FORWARDS.build(PartSpec("swiglu", dict(d_model=d, ffn_dim=F)))
    wf = bind_random(ffn, dtype, rng, std=0.2)
    norm = NORMS.build(PartSpec("rmsnorm", dict(dim=d, eps=1e-5)))
    wn = bind_random(norm, dtype, rng)
    emb = EMBEDDINGS.build(PartSpec("token_embedding", dict(vocab_size=V, d_model=d)))
    we = bind_random(emb, dtype, rng, std=1.0)
    head = HEADS.build(PartSpec("lm_head", dict(vocab_size=V, d_model=d)))
    wh = bind_random(head, dtype, rng, std=0.2)
    cm = CacheManager([], page_size=4, max_tokens=64, max_requests=2, device="cuda:0")
    rc = cm.open("a")
    toks = rng.integers(0, V, T).tolist()
    e = StepEntry(rc, toks, [0, 4, T - 1])
    cm.reserve(rc, T)
    ctx = to_device(layout_entries([e], cm), torch.device("cuda:0"), DT[dtype])
    x = emb.forward(ctx)
    np.testing.assert_array_equal(f64(x), we["weight"][toks])
    h = norm.forward(ctx, x)
    close(h, plain.rms_norm(f64(x), wn["weight"], 1e-5), dtype)
    res = x.clone()
    ffn.forward(ctx, h, res)
    close(res, f64(x) + plain.swiglu_ffn(f64(h), wf["w1"], wf["w3"], wf["w2"]), dtype, scale=2)
    logits = head.forward(ctx, res, norm)
    assert logits.dtype == torch.float32 and logits.shape == (3, V)
    close(logits, plain.lm_head(f64(res)[[0, 4, T - 1]], wn["weight"], 1e-5, wh["weight"]), dtype, scale=2)


# ------------------------------------------------------------------ toy parts
def register_toy_parts():
    """A mixer with state of its own (an exponential moving average per channel, with a
    learned decay), defined here and nowhere in the package."""
    from tuff_b200.parts import Mixer, StateNeed, WeightDecl, register_mixer, MIXERS
    if "toy_ema" in MIXERS.kinds():
        return

    @register_mixer("toy_ema")
    class ToyEma(Mixer):
        replayable = False                  # walks the rows on the host

        def __init__(self, d_model):
            self.d = d_model

        def weight_decls(self):
            return {"decay": WeightDecl((self.d,), role="vector", init="norm"),
                    "proj": WeightDecl((self.d, self.d))}

        def cache_need(self):
            return StateNeed(shape=(self.d,), dtype="float32")

        def forward(self, ctx, cache, h, residual, reads_only=False):
            a = torch.sigmoid(self.w["decay"])
            cu, slots = ctx.host["cu_q"], ctx.host["slot_of_row"]
            y = torch.empty_like(h, dtype=torch.float32)
            for r in range(ctx.n_rows):
                s = cache.state[int(slots[r])]
                for t in range(int(cu[r]), int(cu[r + 1])):
                    s = a * s + (1 - a) * h[t].float()
                    y[t] = s
                cache.state[int(slots[r])] = s
            residual += (y.to(h.dtype) @ self.w["proj"].T).float()


def toy_architecture():
    """A whole toy architecture around the toy mixer, registered from the test."""
    from tuff_b200.config import Architecture, register_architecture
    from tuff_b200.models import LayerSpec, ModelSpec
    from tuff_b200.parts import PartSpec
    register_toy_parts()

    def spec(cfg):
        d, V = cfg["d"], cfg["vocab"]
        layers = []
        for i, kind in enumerate(cfg["kinds"]):
            p = f"l{i}."
            if kind == "ema":
                mixer = PartSpec("toy_ema", dict(d_model=d), {"decay": p + "decay", "proj": p + "proj"})
            else:
                mixer = PartSpec("gqa_attention", dict(d_model=d, num_heads=2, num_kv_heads=1, head_dim=16,
                                                       qk_norm_eps=None, position_encoding=None),
                                 {n: p + n for n in ("q_proj", "k_proj", "v_proj", "out_proj")})
            layers.append(LayerSpec(
                mixer=mixer, ffn=PartSpec("swiglu", dict(d_model=d, ffn_dim=cfg["ffn"]),
                                          {n: p + n for n in ("w1", "w2", "w3")}),
                mixer_norm=PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": p + "n1"}),
                ffn_norm=PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": p + "n2"})))
        return ModelSpec("ToyEmaLM", d, V, PartSpec("token_embedding", dict(vocab_size=V, d_model=d), {"weight": "emb"}),
                         layers, PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": "nf"}),
                         PartSpec("lm_head", dict(vocab_size=V, d_model=d), {"weight": "emb"}))

    register_architecture(Architecture("ToyEmaLM", lambda raw, where: raw, spec, lambda c: dict(c)))


def toy_plain_forward(folder, tokens):
    cfg = plain.read_config(folder)
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    x = w["emb"][tokens]
    d = cfg["d"]
    for i, kind in enumerate(cfg["kinds"]):
        p = f"l{i}."
        h = plain.rms_norm(x, w[p + "n1"], 1e-5)
        if kind == "ema":
            a = 1 / (1 + np.exp(-w[p + "decay"]))
            s, y = np.zeros(d), np.zeros_like(h)
            for t in range(len(tokens)):
                s = a * s + (1 - a) * h[t]
                y[t] = s
            o = y @ w[p + "proj"].T
        else:
            o = plain.gqa_attention_mixer(h, w[p + "q_proj"], w[p + "k_proj"], w[p + "v_proj"], w[p + "out_proj"],
                                          None, None, 2, 1, 16, 0.0, None)
        x = x + o
        x = x + plain.swiglu_ffn(plain.rms_norm(x, w[p + "n2"], 1e-5), w[p + "w1"], w[p + "w3"], w[p + "w2"])
    return plain.lm_head(x, w["nf"], 1e-5, w["emb"])


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from tuff_b200.engine import ModelRunner
    from tuff_b200.weights import write_random_model
    toy_architecture()
    cfg = dict(architectures=["ToyEmaLM"], d=48, vocab=97, ffn=64, kinds=["ema", "attention", "ema"])
    folder = write_random_model(str(tmp_path / "toy"), cfg, 5, store_dtype=torch.float32)
    runner = ModelRunner(folder, dtype="float32", max_tokens=64, page_size=4, max_requests=2)
    assert [type(s).__name__ for s in runner.cache.storages] == ["StateStorage", "PagedStorage", "StateStorage"]
    rng = np.random.default_rng(3)
    seqs = {"a": rng.integers(0, 97, 19).tolist(), "b": rng.integers(0, 97, 11).tolist()}
    refs = {k: toy_plain_forward(folder, v) for k, v in seqs.items()}
    rcs = {k: runner.open(k) for k in seqs}
    pos = {k: 0 for k in seqs}
    cuts = {"a": [4, 1, 1, 6, 2, 5], "b": [2, 3, 1, 1, 4]}
    while any(pos[k] < len(seqs[k]) for k in seqs):
        entries, keys = [], []
        for k in seqs:
            if pos[k] < len(seqs[k]):
                n = cuts[k].pop(0)
                entries.append(StepEntry(rcs[k], seqs[k][pos[k]:pos[k] + n], list(range(n))))
                keys.append((k, n))
        logits = f64(runner.step(entries))
        o = 0
        for k, n in keys:
            np.testing.assert_allclose(logits[o:o + n], refs[k][pos[k]:pos[k] + n], atol=2e-4, rtol=2e-4)
            pos[k] += n
            o += n
    # a slot that is used again starts from zero state
    runner.close(rcs["a"])
    rc = runner.open("again")
    logits = f64(runner.step([StepEntry(rc, seqs["a"], [len(seqs["a"]) - 1])]))
    np.testing.assert_allclose(logits[0], refs["a"][-1], atol=2e-4, rtol=2e-4)


def register_toy_routed_ffn_and_position_encoding():
    """A feed-forward with routing (each token goes to the one of E small experts whose router
    logit is largest, its output scaled by the softmax weight of that logit) and a position
    encoding with pairing of neighbours (element 2j with 2j+1) and its own angle law, both defined
    here and nowhere in the package."""
    from tuff_b200.kernels import ops
    from tuff_b200.parts import (FEED_FORWARDS, FeedForward, PositionEncoding, WeightDecl, register_feed_forward,
                                 register_position_encoding)
    if "toy_top1_experts" in FEED_FORWARDS.kinds():
        return

    @register_feed_forward("toy_top1_experts")
    class ToyTop1(FeedForward):
        replayable = False                  # the rows of an expert are gathered on the host's say

        def __init__(self, d_model, ffn_dim, n_experts):
            self.d, self.F, self.E = d_model, ffn_dim, n_experts

        def weight_decls(self):
            decls = {"router": WeightDecl((self.E, self.d))}
            for e in range(self.E):
                decls[f"up{e}"] = WeightDecl((self.F, self.d))
                decls[f"down{e}"] = WeightDecl((self.d, self.F))
            return decls

        def forward(self, ctx, h, residual):
            T = h.shape[0]
            logits = torch.empty((T, self.E), dtype=torch.float32, device=h.device)
            ops.linear(h, self.w["router"], logits)                 # router logits in fp32
            weight, expert = torch.softmax(logits, -1).max(-1)
            for e in range(self.E):
                idx = torch.nonzero(expert == e).flatten()
                if idx.numel() == 0:
                    continue
                he = h[idx].contiguous()
                mid = torch.empty((idx.numel(), self.F), dtype=h.dtype, device=h.device)
                ops.linear(he, self.w[f"up{e}"], mid)
                mid = torch.relu(mid)
                out = torch.zeros((idx.numel(), self.d), dtype=torch.float32, device=h.device)
                ops.linear(mid, self.w[f"down{e}"], out, accumulate=True)
                residual[idx] += out * weight[idx, None]

    @register_position_encoding("toy_pairs")
    class ToyPairs(PositionEncoding):
        """Rotates (x[2j], x[2j+1]) by pos / (j + 1): no table for the fused kernel, so the
        attention mixer calls `rotate` between its norm and its cache write."""

        def __init__(self, head_dim):
            self.hd = head_dim

        def rotate(self, ctx, q, k):
            j = torch.arange(self.hd // 2, device=q.device, dtype=torch.float32)
            ang = ctx.positions.float()[:, None] / (j + 1)[None]
            c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            for x in (q, k):
                if x is None:
                    continue
                x0, x1 = x[..., 0::2].float().clone(), x[..., 1::2].float().clone()
                x[..., 0::2] = (x0 * c - x1 * s_).to(x.dtype)
                x[..., 1::2] = (x0 * s_ + x1 * c).to(x.dtype)


def test_toy_routed_feed_forward_and_position_encoding(tmp_path):
    """Layers that differ in feed-forward and position encoding within one model: layer 0 has the
    toy position encoding and the toy routed feed-forward, layer 1 the package's rotary encoding and
    SwiGLU.  Stepped in portions and compared with a plain forward over the whole sequence."""
    from tuff_b200.config import Architecture, register_architecture
    from tuff_b200.engine import ModelRunner
    from tuff_b200.models import LayerSpec, ModelSpec
    from tuff_b200.parts import PartSpec
    from tuff_b200.weights import write_random_model
    register_toy_routed_ffn_and_position_encoding()
    d, V, F, E, H, G, hd = 40, 61, 24, 3, 4, 2, 8

    def spec(cfg):
        layers = []
        for i in range(2):
            p = f"l{i}."
            pe = PartSpec("toy_pairs", dict(head_dim=hd)) if i == 0 else PartSpec("rope_neox", dict(head_dim=hd, theta=500.0))
            mixer = PartSpec("gqa_attention", dict(d_model=d, num_heads=H, num_kv_heads=G, head_dim=hd, qk_norm_eps=None,
                                                   position_encoding=pe),
                             {n: p + n for n in ("q_proj", "k_proj", "v_proj", "out_proj")})
            if i == 0:
                names = {"router": p + "router"}
                for e in range(E):
                    names[f"up{e}"], names[f"down{e}"] = p + f"up{e}", p + f"down{e}"
                ffn = PartSpec("toy_top1_experts", dict(d_model=d, ffn_dim=F, n_experts=E), names)
            else:
                ffn = PartSpec("swiglu", dict(d_model=d, ffn_dim=F), {n: p + n for n in ("w1", "w2", "w3")})
            layers.append(LayerSpec(mixer=mixer, ffn=ffn,
                                    mixer_norm=PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": p + "n1"}),
                                    ffn_norm=PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": p + "n2"})))
        return ModelSpec("ToyRoutedLM", d, V, PartSpec("token_embedding", dict(vocab_size=V, d_model=d), {"weight": "emb"}),
                         layers, PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": "nf"}),
                         PartSpec("lm_head", dict(vocab_size=V, d_model=d), {"weight": "emb"}))

    register_architecture(Architecture("ToyRoutedLM", lambda raw, where: raw, spec, lambda c: dict(c)))
    folder = write_random_model(str(tmp_path / "routed"), dict(architectures=["ToyRoutedLM"]), 9, store_dtype=torch.float32)
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    # the router's rows far apart, so that the choice of expert does not hang on rounding
    w = {k: np.asarray(v, np.float64) for k, v in w.items()}

    def attention(h, p, toy):
        T = h.shape[0]
        q = (h @ w[p + "q_proj"].T).reshape(T, H, hd)
        k = (h @ w[p + "k_proj"].T).reshape(T, G, hd)
        v = (h @ w[p + "v_proj"].T).reshape(T, G, hd)
        pos = np.arange(T)
        if toy:
            ang = pos[:, None] / (np.arange(hd // 2) + 1)[None]
            c, s_ = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
            def rot(x):
                y = x.copy()
                y[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s_
                y[..., 1::2] = x[..., 0::2] * s_ + x[..., 1::2] * c
                return y
            q, k = rot(q), rot(k)
        else:
            q, k = plain.rope_neox(q, pos, 500.0), plain.rope_neox(k, pos, 500.0)
        out = np.zeros((T, H, hd))
        for hh in range(H):
            g = hh // (H // G)
            sc = np.where(pos[None] > pos[:, None], -np.inf, q[:, hh] @ k[:, g].T / np.sqrt(hd))
            pr = np.exp(sc - sc.max(-1, keepdims=True))
            out[:, hh] = (pr / pr.sum(-1, keepdims=True)) @ v[:, g]
        return out.reshape(T, H * hd) @ w[p + "out_proj"].T

    def forward(tokens):
        x = w["emb"][tokens]
        margins = []
        for i in range(2):
            p = f"l{i}."
            x = x + attention(plain.rms_norm(x, w[p + "n1"], 1e-5), p, i == 0)
            h = plain.rms_norm(x, w[p + "n2"], 1e-5)
            if i == 0:
                lg = h @ w[p + "router"].T
                pr = np.exp(lg - lg.max(-1, keepdims=True)); pr /= pr.sum(-1, keepdims=True)
                srt = np.sort(lg, -1)
                margins.append(srt[:, -1] - srt[:, -2])
                o = np.zeros_like(x)
                for t in range(len(tokens)):
                    e = int(lg[t].argmax())
                    o[t] = (np.maximum(h[t] @ w[p + f"up{e}"].T, 0) @ w[p + f"down{e}"].T) * pr[t, e]
                x = x + o
            else:
                x = x + plain.swiglu_ffn(h, w[p + "w1"], w[p + "w3"], w[p + "w2"])
        return plain.lm_head(x, w["nf"], 1e-5, w["emb"]), np.concatenate(margins)

    rng = np.random.default_rng(12)
    tokens = rng.integers(0, V, 37).tolist()
    ref, margin = forward(tokens)
    decided = margin > 1e-4                        # tokens whose expert does not hang on rounding
    assert decided.mean() > 0.9
    runner = ModelRunner(folder, dtype="float32", max_tokens=64, page_size=4, max_requests=2)
    assert not runner.cuda_graphs                  # a part said it cannot be replayed
    rc = runner.open("r")
    pos = 0
    for n in (5, 1, 1, 1, 2, 12, 1, 8, 6):
        logits = f64(runner.step([StepEntry(rc, tokens[pos:pos + n], list(range(n)))]))
        # a token routed differently would change every later position of the sequence
        if decided[:pos + n].all():
            np.testing.assert_allclose(logits, ref[pos:pos + n], atol=3e-4, rtol=3e-4)
        pos += n
    assert decided.all() or pos == len(tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_names_a_layer_twice_and_shares_a_cache(tmp_path, dtype):
    """The order of layers is data: layer 1 runs twice (with storage of its own each time) and
    the last run of an attention layer reads the keys and values that an earlier one wrote."""
    from tuff_b200.config import Architecture, register_architecture
    from tuff_b200.engine import ModelRunner
    from tuff_b200.models import ScheduleEntry
    from tuff_b200.models.lfm2 import lfm2_spec
    from tuff_b200.config import Lfm2Config
    from tuff_b200.weights import write_random_model
    from tiny import TINY_A

    def spec(cfg):
        s = lfm2_spec(cfg)
        s.architecture = "Lfm2Looped"
        # layers: 0 conv, 1 attention, 2 conv, 3 attention
        s.schedule = [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2), ScheduleEntry(1, 3),
                      ScheduleEntry(3, 1, reads_only=True)]
        return s
    register_architecture(Architecture("Lfm2Looped", Lfm2Config.from_dict, spec, lambda c: c.to_dict()))
    raw = dict(TINY_A, architectures=["Lfm2Looped"])
    folder = write_random_model(str(tmp_path / "looped"), raw, 3)
    m = plain.PlainLfm2(folder)
    w, d, eps = m.w, m.d, m.eps

    def plain_forward(tokens):
        x = plain.embed(w["model.embed_tokens.weight"], tokens)
        kv_from = {}

        def attn(i, h, shared_h=None):
            a = f"model.layers.{i}.self_attn."
            src = f"model.layers.{1 if shared_h is not None else i}.self_attn."
            hk = h if shared_h is None else shared_h
            T = len(tokens)
            pos = np.arange(T)
            q = plain.rope_neox(plain.rms_norm((h @ w[a + "q_proj.weight"].T).reshape(T, m.H, m.hd),
                                               w[a + "q_layernorm.weight"], eps), pos, m.theta)
            k = plain.rope_neox(plain.rms_norm((hk @ w[src + "k_proj.weight"].T).reshape(T, m.G, m.hd),
                                               w[src + "k_layernorm.weight"], eps), pos, m.theta)
            v = (hk @ w[src + "v_proj.weight"].T).reshape(T, m.G, m.hd)
            out = np.zeros((T, m.H, m.hd))
            for hh in range(m.H):
                g = hh // (m.H // m.G)
                s = q[:, hh] @ k[:, g].T / math.sqrt(m.hd)
                s = np.where(np.triu(np.ones((T, T), bool), 1), -np.inf, s)
                p = np.exp(s - s.max(-1, keepdims=True))
                out[:, hh] = (p / p.sum(-1, keepdims=True)) @ v[:, g]
            return out.reshape(T, -1) @ w[a + "out_proj.weight"].T

        first_h1 = None
        for layer, shared in ((0, False), (1, False), (2, False), (1, False), (3, True)):
            p = f"model.layers.{layer}."
            h = plain.rms_norm(x, w[p + "operator_norm.weight"], eps)
            if layer in (0, 2):
                o = plain.short_conv_mixer(h, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"].reshape(d, 3),
                                           w[p + "conv.out_proj.weight"])
            elif shared:
                o = attn(3, h, shared_h=first_h1)
            else:
                if first_h1 is None:
                    first_h1 = h
                o = attn(1, h)
            x = x + o
            f = p + "feed_forward."
            x = x + plain.swiglu_ffn(plain.rms_norm(x, w[p + "ffn_norm.weight"], eps), w[f + "w1.weight"],
                                     w[f + "w3.weight"], w[f + "w2.weight"])
        return plain.lm_head(x, w["model.embedding_norm.weight"], eps, w["model.embed_tokens.weight"])

    runner = ModelRunner(folder, dtype=dtype, max_tokens=64, page_size=4, max_requests=2)
    assert len(runner.cache.storages) == 4
    toks = np.random.default_rng(4).integers(0, 256, 29).tolist()
    ref = plain_forward(toks)
    rc = runner.open("x")
    got = []
    for lo, hi in ((0, 9), (9, 10), (10, 12), (12, 29)):
        got.append(f64(runner.step([StepEntry(rc, toks[lo:hi], list(range(hi - lo)))])))
    got = np.concatenate(got)
    tol = 2e-4 if dtype == "float32" else 5e-2
    assert np.abs(got - ref).max() < tol, np.abs(got - ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_windows_have_pages_of_their_own(tmp_path, dtype):
    """An architecture whose attention layers differ in what they keep (a window of 40 keys, all
    keys, a window of 24): three groups of pages, each with its own block table; pages that a
    window has passed go back to their group's pool while the request runs and are taken again by
    the other request.  Portions, decoding and both requests in one batch, against a plain forward
    with the same windows (head size 64: the tensor-core attention kernels in bf16)."""
    from tuff_b200.config import Architecture, Lfm2Config, register_architecture
    from tuff_b200.engine import ModelRunner
    from tuff_b200.models.lfm2 import lfm2_spec
    from tuff_b200.weights import write_random_model
    from tiny import TINY_D
    windows = {0: 40, 2: None, 4: 24}              # layer -> window (TINY_D: attention in layers 0, 2, 4)

    def spec(cfg):
        s = lfm2_spec(cfg)
        s.architecture = "Lfm2Windowed"
        for i, wdw in windows.items():
            s.layers[i].mixer.params["window"] = wdw
        return s
    register_architecture(Architecture("Lfm2Windowed", Lfm2Config.from_dict, spec, lambda c: c.to_dict()))
    folder = write_random_model(str(tmp_path / "windowed"), dict(TINY_D, architectures=["Lfm2Windowed"]), 8)
    m = plain.PlainLfm2(folder)
    w, d, eps = m.w, m.d, m.eps

    def plain_forward(tokens):
        x = plain.embed(w["model.embed_tokens.weight"], tokens)
        for i in range(5):
            p = f"model.layers.{i}."
            h = plain.rms_norm(x, w[p + "operator_norm.weight"], eps)
            if i in windows:
                a = p + "self_attn."
                o = plain.gqa_attention_mixer(h, w[a + "q_proj.weight"], w[a + "k_proj.weight"], w[a + "v_proj.weight"],
                                              w[a + "out_proj.weight"], w[a + "q_layernorm.weight"], w[a + "k_layernorm.weight"],
                                              m.H, m.G, m.hd, eps, m.theta, window=windows[i])
            else:
                o = plain.short_conv_mixer(h, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"].reshape(d, 3),
                                           w[p + "conv.out_proj.weight"])
            x = x + o
            f = p + "feed_forward."
            x = x + plain.swiglu_ffn(plain.rms_norm(x, w[p + "ffn_norm.weight"], eps), w[f + "w1.weight"],
                                     w[f + "w3.weight"], w[f + "w2.weight"])
        return plain.lm_head(x, w["model.embedding_norm.weight"], eps, w["model.embed_tokens.weight"])

    runner = ModelRunner(folder, dtype=dtype, max_tokens=256, page_size=8, max_requests=2)
    cm = runner.cache
    assert sorted(str(g.need.window) for g in cm.groups) == ["24", "40", "None"]
    rng = np.random.default_rng(6)
    seqs = {"a": rng.integers(0, 500, 150).tolist(), "b": rng.integers(0, 500, 90).tolist()}
    refs = {k: plain_forward(v) for k, v in seqs.items()}
    rcs = {"a": runner.open("a")}
    tol = 3e-4 if dtype == "float32" else 6e-2
    worst = 0.0

    def run(entries):
        nonlocal worst
        logits = f64(runner.step([StepEntry(rcs[k], seqs[k][lo:hi], list(range(hi - lo))) for k, lo, hi in entries]))
        o = 0
        for k, lo, hi in entries:
            worst = max(worst, np.abs(logits[o:o + hi - lo] - refs[k][lo:hi]).max())
            o += hi - lo
        cm.check()

    run([("a", 0, 33)])
    run([("a", 33, 97)])                            # the window of 40 has passed the first pages: they are free again
    free_after_prompt = {str(g.need.window): g.pool.n_free for g in cm.groups}
    assert free_after_prompt["40"] > free_after_prompt["None"] and free_after_prompt["24"] > free_after_prompt["40"]
    rcs["b"] = runner.open("b")
    run([("a", 97, 98), ("b", 0, 50)])              # a decoding row beside a portion
    pos = {"a": 98, "b": 50}
    while pos["a"] < 150 or pos["b"] < 90:
        entries = [(k, pos[k], pos[k] + 1) for k in ("a", "b") if pos[k] < len(seqs[k])]
        run(entries)
        for k, lo, hi in entries:
            pos[k] = hi
    assert worst < tol, worst
    held = {str(g.need.window): sum(p != -1 for p in rcs["a"].tables[i]) for i, g in enumerate(cm.groups)}
    assert held["None"] == 19 and held["40"] <= 6 and held["24"] <= 4        # 150 tokens in pages of 8; windows keep a few
    runner.close(rcs["a"]); runner.close(rcs["b"])
    cm.check()


# ---- state whose neutral element is not zero; values wider than keys ---------------------------
def register_toy_max_and_wide_values():
    """Two more mixers defined here and nowhere in the package: a running maximum per channel (its
    state starts at the lowest float, `StateNeed(fill=...)`), and single-head attention whose values are
    three times as wide as its keys (`PagedKVNeed(v_head_dim=...)`), written to and read from the pages
    on the host's say."""
    from tuff_b200.parts import MIXERS, Mixer, PagedKVNeed, StateNeed, WeightDecl, register_mixer
    if "toy_running_max" in MIXERS.kinds():
        return

    @register_mixer("toy_running_max")
    class ToyMax(Mixer):
        replayable = False

        def __init__(self, d_model):
            self.d = d_model

        def weight_decls(self):
            return {"proj": WeightDecl((self.d, self.d))}

        def cache_need(self):
            return StateNeed(shape=(self.d,), dtype="float32", fill=LOWEST)

        def forward(self, ctx, cache, h, residual, reads_only=False):
            cu, slots = ctx.host["cu_q"], ctx.host["slot_of_row"]
            y = torch.empty_like(h, dtype=torch.float32)
            for r in range(ctx.n_rows):
                s = cache.state[int(slots[r])]
                for t in range(int(cu[r]), int(cu[r + 1])):
                    s = torch.maximum(s, h[t].float())
                    y[t] = s
                cache.state[int(slots[r])] = s
            residual += (y.to(h.dtype) @ self.w["proj"].T).float()

    @register_mixer("toy_wide_values")
    class ToyWideValues(Mixer):
        replayable = False

        def __init__(self, d_model, key_dim, value_dim):
            self.d, self.dk, self.dv = d_model, key_dim, value_dim

        def weight_decls(self):
            return {"q": WeightDecl((self.dk, self.d)), "k": WeightDecl((self.dk, self.d)),
                    "v": WeightDecl((self.dv, self.d)), "o": WeightDecl((self.d, self.dv))}

        def cache_need(self):
            return PagedKVNeed(kv_heads=1, head_dim=self.dk, v_head_dim=self.dv)

        def forward(self, ctx, cache, h, residual, reads_only=False):
            q, k, v = (h @ self.w[n].T for n in "qkv")
            table = ctx.host["block_tables"][cache.group]
            cu, pos, page = ctx.host["cu_q"], ctx.host["positions"], cache.page_size
            out = torch.empty((h.shape[0], self.dv), dtype=h.dtype, device=h.device)
            for r in range(ctx.n_rows):
                for t in range(int(cu[r]), int(cu[r + 1])):
                    p = int(pos[t])
                    cache.k_pages[int(table[r][p // page]), 0, p % page] = k[t]
                    cache.v_pages[int(table[r][p // page]), 0, p % page] = v[t]
                    keys = torch.stack([cache.k_pages[int(table[r][j // page]), 0, j % page] for j in range(p + 1)])
                    vals = torch.stack([cache.v_pages[int(table[r][j // page]), 0, j % page] for j in range(p + 1)])
                    w = torch.softmax((keys.float() @ q[t].float()) / math.sqrt(self.dk), 0)
                    out[t] = (w @ vals.float()).to(h.dtype)
            residual += (out @ self.w["o"].T).float()


LOWEST = float(np.finfo(np.float32).min)


def test_state_with_its_own_neutral_element_and_values_wider_than_keys(tmp_path):
    """What another architecture might bring without a change to the cache manager: a state that does not
    start at zero, and pages whose values have another width than their keys.  Stepped in portions of
    changing size, two requests at once, a slot and pages used again; against a plain restatement."""
    from tuff_b200.config import Architecture, register_architecture
    from tuff_b200.engine import ModelRunner
    from tuff_b200.models import LayerSpec, ModelSpec
    from tuff_b200.parts import PartSpec
    from tuff_b200.weights import write_random_model
    register_toy_max_and_wide_values()
    d, V, F, dk, dv = 40, 61, 48, 8, 24

    def spec(cfg):
        layers = []
        for i, kind in enumerate(("max", "wide")):
            p = f"l{i}."
            mixer = (PartSpec("toy_running_max", dict(d_model=d), {"proj": p + "proj"}) if kind == "max" else
                     PartSpec("toy_wide_values", dict(d_model=d, key_dim=dk, value_dim=dv), {n: p + n for n in "qkvo"}))
            layers.append(LayerSpec(mixer=mixer, ffn=PartSpec("swiglu", dict(d_model=d, ffn_dim=F), {n: p + n for n in ("w1", "w2", "w3")}),
                                    mixer_norm=PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": p + "n1"}),
                                    ffn_norm=PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": p + "n2"})))
        return ModelSpec("ToyMaxLM", d, V, PartSpec("token_embedding", dict(vocab_size=V, d_model=d), {"weight": "emb"}),
                         layers, PartSpec("rmsnorm", dict(dim=d, eps=1e-5), {"weight": "nf"}),
                         PartSpec("lm_head", dict(vocab_size=V, d_model=d), {"weight": "emb"}))

    register_architecture(Architecture("ToyMaxLM", lambda raw, where: raw, spec, lambda c: dict(c)))
    folder = write_random_model(str(tmp_path / "toymax"), dict(architectures=["ToyMaxLM"]), 9, store_dtype=torch.float32)
    runner = ModelRunner(folder, dtype="float32", max_tokens=48, page_size=4, max_requests=2)
    paged = [s for s in runner.cache.storages if type(s).__name__ == "PagedStorage"][0]
    assert paged.k_pages.shape[-1] == dk and paged.v_pages.shape[-1] == dv
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))

    def reference(tokens):
        x = w["emb"][tokens]
        h = plain.rms_norm(x, w["l0.n1"], 1e-5)
        x = x + np.maximum.accumulate(h, axis=0) @ w["l0.proj"].T
        x = x + plain.swiglu_ffn(plain.rms_norm(x, w["l0.n2"], 1e-5), w["l0.w1"], w["l0.w3"], w["l0.w2"])
        h = plain.rms_norm(x, w["l1.n1"], 1e-5)
        q, k, v = h @ w["l1.q"].T, h @ w["l1.k"].T, h @ w["l1.v"].T
        s = q @ k.T / math.sqrt(dk)
        s = np.where(np.triu(np.ones_like(s, dtype=bool), 1), -np.inf, s)
        p = np.exp(s - s.max(-1, keepdims=True))
        x = x + (p / p.sum(-1, keepdims=True)) @ v @ w["l1.o"].T
        x = x + plain.swiglu_ffn(plain.rms_norm(x, w["l1.n2"], 1e-5), w["l1.w1"], w["l1.w3"], w["l1.w2"])
        return plain.lm_head(x, w["nf"], 1e-5, w["emb"])

    rng = np.random.default_rng(4)
    seqs = {"a": rng.integers(0, V, 17).tolist(), "b": rng.integers(0, V, 9).tolist()}
    refs = {k: reference(v) for k, v in seqs.items()}
    rcs = {k: runner.open(k) for k in seqs}
    pos = {k: 0 for k in seqs}
    cuts = {"a": [3, 1, 6, 2, 5], "b": [2, 1, 1, 5]}
    while any(pos[k] < len(seqs[k]) for k in seqs):
        entries, keys = [], []
        for k in seqs:
            if pos[k] < len(seqs[k]):
                n = cuts[k].pop(0)
                entries.append(StepEntry(rcs[k], seqs[k][pos[k]:pos[k] + n], list(range(n))))
                keys.append((k, n))
        logits = f64(runner.step(entries))
        o = 0
        for k, n in keys:
            np.testing.assert_allclose(logits[o:o + n], refs[k][pos[k]:pos[k] + n], atol=2e-4, rtol=2e-4)
            pos[k] += n
            o += n
    # the slot and the pages of a finished request, taken again: the state starts at its own neutral element
    runner.close(rcs["a"])
    rc = runner.open("again")
    logits = f64(runner.step([StepEntry(rc, seqs["b"], [len(seqs["b"]) - 1])]))
    np.testing.assert_allclose(logits[0], refs["b"][-1], atol=2e-4, rtol=2e-4)
    runner.close(rc); runner.close(rcs["b"])
    runner.cache.check()
