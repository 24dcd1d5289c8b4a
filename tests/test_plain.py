"""The plain implementation against the reference's own float64 forward (golden
file made by tests/golden/make_golden.py), and its parts against each other."""
import json
import os

import numpy as np
import pytest

import plain_lfm2 as plain
from golden.make_golden import weights_checksum

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "lfm2_fp64_ref.npz")


@pytest.mark.parametrize("case", ["tiny_a", "tiny_b_k3"])
def test_plain_equals_reference_fp64(tmp_path, case):
    g = np.load(GOLDEN)
    folder = tmp_path / case
    folder.mkdir()
    (folder / "config.json").write_bytes(bytes(g[case + ".config"]))
    (folder / "model.safetensors").write_bytes(bytes(g[case + ".safetensors"]))     # the very weights the reference ran on
    model = plain.PlainLfm2(str(folder))
    assert weights_checksum(model.w) == bytes(g[case + ".checksum"]).decode()
    logits = model.forward(g[case + ".tokens"].tolist())
    ref = g[case + ".logits"].astype(np.float64)
    assert logits.shape == ref.shape
    assert np.abs(logits - ref).max() < 2e-6        # the golden rows are stored as float32


def test_conv_is_causal_and_matches_stepwise(tmp_path):
    rng = np.random.default_rng(0)
    d, K, T = 8, 4, 11
    h = rng.normal(size=(T, d))
    w_in, taps, w_out = rng.normal(size=(3 * d, d)), rng.normal(size=(d, K)), rng.normal(size=(d, d))
    full = plain.short_conv_mixer(h, w_in, taps, w_out)
    # token-by-token recurrence with an explicit state (src/lfm25_gpu.cu:287-337, generalised to K taps)
    state = np.zeros((K - 1, d))
    for t in range(T):
        bcx = w_in @ h[t]
        u = bcx[:d] * bcx[2 * d:]
        y = sum(state[j] * taps[:, j] for j in range(K - 1)) + u * taps[:, K - 1]
        state = np.concatenate([state[1:], u[None]], 0)
        np.testing.assert_allclose(w_out @ (bcx[d:2 * d] * y), full[t], rtol=1e-12, atol=1e-12)


def test_attention_prefix_independence():
    rng = np.random.default_rng(1)
    d, H, G, hd, T = 12, 4, 2, 6, 9
    h = rng.normal(size=(T, d))
    ws = [rng.normal(size=s) for s in ((H * hd, d), (G * hd, d), (G * hd, d), (d, H * hd))]
    qn, kn = 1 + 0.1 * rng.normal(size=hd), 1 + 0.1 * rng.normal(size=hd)
    full = plain.gqa_attention_mixer(h, *ws, qn, kn, H, G, hd, 1e-5, 1e4)
    part = plain.gqa_attention_mixer(h[:5], *ws, qn, kn, H, G, hd, 1e-5, 1e4)
    np.testing.assert_allclose(full[:5], part, rtol=1e-12, atol=1e-12)


def test_sample_token_rules():
    l = np.array([1.0, 3.0, 3.0, -2.0, 0.5])
    assert plain.sample_token(l) == 1                       # greedy: first maximum
    assert plain.sample_token(l, temp=1.0, top_k=1, u=0.99) == 1
    assert plain.sample_token(l, temp=1.0, top_k=2, u=0.99) == 2
    assert plain.sample_token(l, temp=1.0, min_p=0.5, u=0.0) == 1
    # top-p 0.5: the two equal leaders hold ~0.44 each, so the nucleus needs both
    assert plain.sample_token(l, temp=1.0, top_p=0.5, u=0.999) == 2
    # penalty per occurrence
    assert plain.sample_token(l, temp=1e-3, repeat_penalty=2.0, recent=[1, 2, 1, 2], u=0.5) == 0
    us = [plain.uniform_draw(7, 3, i) for i in range(1000)]
    assert 0.0 <= min(us) and max(us) < 1.0 and 0.45 < np.mean(us) < 0.55
