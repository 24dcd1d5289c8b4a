#!/usr/bin/env python3
"""Makes tests/golden/lfm2_fp64_ref.npz: logits of the reference's own float64
forward (tools/lfm25_fp64_ref.py of niihelium/tuff, run unmodified on the CPU)
for two tiny random models, against which tests/test_plain.py checks the plain
implementation.

    python tests/golden/make_golden.py /path/to/tuff

For each case it writes a random model folder with this package's seeded
random-weights mode, converts the tensors to an F32 GGUF under the names the
reference binds (src/lfm25_model.c:120-216), and lets the reference script run
teacher-forced over a token sequence (a 1-token prompt, the rest as the stream,
which yields one logits row per position).  The reference script fixes the
convolution at 3 taps and the head size at hidden/heads, so both cases have
conv_L_cache = 3; sizes with 4 taps rest on the formulas alone.

Stored per case: the configuration, the weight seed, the model.safetensors file
itself (the test needs no random generator to have the same weights), a checksum
of the weights, the tokens, and the logits as float32 [T, vocab].
"""
import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

CASES = {
    "tiny_a": dict(
        seed=0, n_tokens=21,
        config=dict(architectures=["Lfm2ForCausalLM"], hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                    num_key_value_heads=2, intermediate_size=192, block_auto_adjust_ff_dim=False, vocab_size=256,
                    rope_theta=10000.0, norm_eps=1e-5, conv_L_cache=3,
                    layer_types=["conv", "full_attention", "conv", "full_attention"], tie_embedding=True)),
    "tiny_b_k3": dict(
        seed=1, n_tokens=37,
        config=dict(architectures=["Lfm2ForCausalLM"], hidden_size=96, num_hidden_layers=6, num_attention_heads=4,
                    num_key_value_heads=1, intermediate_size=384, block_auto_adjust_ff_dim=True,
                    ffn_dim_multiplier=1.0, block_multiple_of=32, vocab_size=384, rope_theta=1e6, norm_eps=1e-6,
                    conv_L_cache=3, full_attn_idxs=[0, 3], tie_embedding=False)),
}

GGUF_NAMES = {
    "operator_norm.weight": "attn_norm.weight", "ffn_norm.weight": "ffn_norm.weight",
    "conv.in_proj.weight": "shortconv.in_proj.weight", "conv.conv.weight": "shortconv.conv.weight",
    "conv.out_proj.weight": "shortconv.out_proj.weight", "self_attn.q_proj.weight": "attn_q.weight",
    "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
    "self_attn.out_proj.weight": "attn_output.weight", "self_attn.q_layernorm.weight": "attn_q_norm.weight",
    "self_attn.k_layernorm.weight": "attn_k_norm.weight", "feed_forward.w1.weight": "ffn_gate.weight",
    "feed_forward.w3.weight": "ffn_up.weight", "feed_forward.w2.weight": "ffn_down.weight",
}


def weights_checksum(tensors):
    h = hashlib.sha256()
    for n in sorted(tensors):
        h.update(n.encode())
        h.update(np.ascontiguousarray(tensors[n], dtype=np.float32).tobytes())
    return h.hexdigest()


def case_tokens(name, case):
    rng = np.random.default_rng(case["seed"] + 100)
    return rng.integers(0, case["config"]["vocab_size"], case["n_tokens"]).tolist()


def main():
    import gguf
    from plain_lfm2 import read_safetensors
    from tuff_b200.weights import write_random_model
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/a/checkout/of/niihelium/tuff")
    ref_root = sys.argv[1]
    script = os.path.join(ref_root, "tools", "lfm25_fp64_ref.py")
    out = {}
    for name, case in CASES.items():
        cfg = case["config"]
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_random_model(os.path.join(tmp, name), cfg, case["seed"])
            w = read_safetensors(os.path.join(folder, "model.safetensors"))
            path = os.path.join(tmp, name + ".gguf")
            gw = gguf.GGUFWriter(path, "lfm2")
            gw.add_uint32("lfm2.block_count", cfg["num_hidden_layers"])
            gw.add_float32("lfm2.attention.layer_norm_rms_epsilon", cfg["norm_eps"])
            gw.add_float32("lfm2.rope.freq_base", cfg["rope_theta"])
            gw.add_uint32("lfm2.attention.head_count", cfg["num_attention_heads"])
            gw.add_uint32("lfm2.embedding_length", cfg["hidden_size"])
            for n, a in w.items():
                a = a.astype(np.float32)
                if n == "model.embed_tokens.weight":
                    g = "token_embd.weight"
                elif n == "model.embedding_norm.weight":
                    g = "token_embd_norm.weight"
                elif n == "lm_head.weight":
                    g = "output.weight"
                else:
                    _, _, i, rest = n.split(".", 3)
                    g = f"blk.{i}.{GGUF_NAMES[rest]}"
                    if rest == "conv.conv.weight":
                        a = a.reshape(a.shape[0], a.shape[2])
                gw.add_tensor(g, np.ascontiguousarray(a))
            gw.write_header_to_file(); gw.write_kv_data_to_file(); gw.write_tensors_to_file(); gw.close()
            toks = case_tokens(name, case)
            stream = os.path.join(tmp, "stream.txt")
            with open(stream, "w") as f:
                f.write("\n".join(str(t) for t in toks[1:] + [0]) + "\n")
            binf = os.path.join(tmp, "logits.bin")
            env = dict(os.environ, LLAMA_GGUF_PY="/nonexistent")
            subprocess.run([sys.executable, script, "--model", path, "--prompt-tokens", str(toks[0]),
                            "--tokens", stream, "-n", str(len(toks)), "--out", binf], check=True, env=env)
            logits = np.fromfile(binf, dtype=np.float32).reshape(len(toks), cfg["vocab_size"])
            out[name + ".config"] = np.frombuffer(json.dumps(cfg).encode(), dtype=np.uint8)
            out[name + ".seed"] = np.int64(case["seed"])
            out[name + ".checksum"] = np.frombuffer(weights_checksum(w).encode(), dtype=np.uint8)
            with open(os.path.join(folder, "model.safetensors"), "rb") as f:
                out[name + ".safetensors"] = np.frombuffer(f.read(), dtype=np.uint8)      # the weights themselves
            out[name + ".tokens"] = np.asarray(toks, np.int32)
            out[name + ".logits"] = logits
            print(name, logits.shape, float(np.abs(logits).max()))
    np.savez_compressed(os.path.join(HERE, "lfm2_fp64_ref.npz"), **out)


if __name__ == "__main__":
    main()
