"""Layers of the real size (LFM2.5-1.2B widths: hidden 2048, 32/8 heads of 64, feed-forward 5632, vocabulary
65536, pages of 64) but only four of them: the kernels that the tiny configurations never reach at these shapes
(tensor-core products with 256-wide tiles and the SwiGLU epilogue over blocked gate/up rows, split-K, the fused
norm at 2048 columns, the tensor-core attention at 32 heads in 8 groups) against the plain implementation."""
import io
import json

import numpy as np
import pytest

import plain_lfm2 as plain
import traces

pytestmark = pytest.mark.gpu

CONFIG = dict(
    architectures=["Lfm2ForCausalLM"], hidden_size=2048, num_hidden_layers=4, num_attention_heads=32,
    num_key_value_heads=8, intermediate_size=8192, block_auto_adjust_ff_dim=True, block_multiple_of=256,
    vocab_size=65536, rope_theta=1e6, norm_eps=1e-5, conv_L_cache=3, full_attn_idxs=[1, 3], tie_embedding=True)


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    from tuff_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("big") / "m"), CONFIG, 7)
    rng = np.random.default_rng(1)
    reqs = {"a": rng.integers(0, 65536, 300).tolist(), "b": rng.integers(0, 65536, 70).tolist(),
            "c": rng.integers(0, 65536, 131).tolist()}
    model = plain.PlainLfm2(folder)
    return folder, reqs, {k: model.forward(v) for k, v in reqs.items()}


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", 5e-2)])
@pytest.mark.parametrize("mode", ["whole", "tail_decoded", "mixed"])
def test_full_size_layers(big, tmp_path, dtype, tol, mode):
    from tuff_b200.engine.replay import replay
    from tuff_b200.engine.runner import ModelRunner
    from tuff_b200.kernels import ops
    folder, reqs, ref = big
    steps, wanted = getattr(traces, mode)(reqs)
    runner = ModelRunner(folder, dtype=dtype, max_tokens=traces.tokens_needed(steps), page_size=64, max_requests=4)
    replay(runner, io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), str(tmp_path), report=io.StringIO())
    ops.check_tc_status()
    for step, rows in wanted.items():
        got = np.fromfile(tmp_path / f"{step}.f32", dtype="<f4").reshape(len(rows), 65536)
        for i, (rid, pos) in enumerate(rows):
            r = ref[rid][pos]
            err = np.abs(got[i] - r).max()
            assert err <= tol * max(1.0, np.abs(r).max()), (mode, dtype, rid, pos, err)
    runner.cache.check()
