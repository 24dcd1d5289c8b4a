"""The tests' own small configurations of the architecture and helpers to make
model folders from them.  The two differ in every size and option: layer count
and kinds (given by `layer_types` in one and `full_attn_idxs` in the other),
width, head counts and groups, head size (24 is no power of two), feed-forward
width (given directly / auto-adjusted), vocabulary, rope base, eps, number of
convolution taps, tied and untied head."""
import numpy as np

TINY_A = dict(
    architectures=["Lfm2ForCausalLM"], hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
    num_key_value_heads=2, intermediate_size=192, block_auto_adjust_ff_dim=False, vocab_size=256,
    rope_theta=10000.0, norm_eps=1e-5, conv_L_cache=3,
    layer_types=["conv", "full_attention", "conv", "full_attention"], tie_embedding=True)

TINY_B = dict(
    architectures=["Lfm2ForCausalLM"], hidden_size=96, num_hidden_layers=6, num_attention_heads=4,
    num_key_value_heads=1, intermediate_size=384, block_auto_adjust_ff_dim=True, ffn_dim_multiplier=1.0,
    block_multiple_of=32, vocab_size=384, rope_theta=1e6, norm_eps=1e-6, conv_L_cache=4,
    full_attn_idxs=[0, 3], tie_embedding=False)

# a third one with head size 48 (a step of 16 that is no power of two), 3 groups of 2 heads,
# a width and a vocabulary that are no multiple of 16 anywhere else
TINY_C = dict(
    architectures=["Lfm2ForCausalLM"], hidden_size=80, num_hidden_layers=3, num_attention_heads=6,
    num_key_value_heads=3, head_dim=48, intermediate_size=200, block_auto_adjust_ff_dim=False, vocab_size=301,
    rope_theta=5e5, norm_eps=1e-5, conv_L_cache=2,
    layer_types=["full_attention", "conv", "full_attention"], tie_embedding=True)

# head size 64 (the tensor-core attention kernels' size) with 4 x 64 != hidden, 2 query heads per group
TINY_D = dict(
    architectures=["Lfm2ForCausalLM"], hidden_size=128, num_hidden_layers=5, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, intermediate_size=320, block_auto_adjust_ff_dim=False, vocab_size=500,
    rope_theta=1e6, norm_eps=1e-5, conv_L_cache=3,
    layer_types=["full_attention", "conv", "full_attention", "conv", "full_attention"], tie_embedding=True)

CONFIGS = {"tiny_a": (TINY_A, 0), "tiny_b": (TINY_B, 1), "tiny_c": (TINY_C, 2), "tiny_d": (TINY_D, 3)}


def make_folder(tmp_path, name, store_dtype=None):
    import torch
    from tuff_b200.weights import write_random_model
    cfg, seed = CONFIGS[name]
    return write_random_model(str(tmp_path / name), cfg, seed,
                              store_dtype=store_dtype or torch.bfloat16)


def random_tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()
