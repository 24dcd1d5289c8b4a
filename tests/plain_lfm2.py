"""A plain, slow implementation of the LFM2 / LFM2.5 dense decoder in NumPy:
whole sequences, no cache, one function for each part.

It is written from the reference's formulas (each function cites the place) and
shares no code with `tuff_b200`: it reads config.json and the safetensors file
with the standard library and NumPy alone.  It rests on the formulas; it is
compared once with the reference's own float64 forward
(tools/lfm25_fp64_ref.py) in tests/golden/ (see make_golden.py there).

Everything is float64 unless `dtype` says otherwise.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# ------------------------------------------------------------------ file reading
def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path):
    """name -> float64 array (BF16 and F32 tensors)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        if info["dtype"] == "BF16":
            a = _bf16_to_f32(np.frombuffer(data[b:e], dtype=np.uint16))
        elif info["dtype"] == "F32":
            a = np.frombuffer(data[b:e], dtype=np.float32)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = a.astype(np.float64).reshape(info["shape"])
    return out


def ffn_width(cfg):
    """Feed-forward width from the configuration (two thirds of intermediate_size when
    block_auto_adjust_ff_dim, times the multiplier, rounded up to block_multiple_of).
    The reference reads the final width from the model file (src/lfm25_model.c:99-100)."""
    f = cfg["intermediate_size"]
    if cfg.get("block_auto_adjust_ff_dim", False):
        f = int(2 * f / 3)
        if cfg.get("ffn_dim_multiplier") is not None:
            f = int(cfg["ffn_dim_multiplier"] * f)
        m = cfg.get("block_multiple_of", 256)
        f = m * ((f + m - 1) // m)
    return f


def layer_kinds(cfg):
    L = cfg["num_hidden_layers"]
    if cfg.get("layer_types") is not None:
        return ["attention" if t in ("full_attention", "attention") else "conv" for t in cfg["layer_types"]]
    idx = set(cfg["full_attn_idxs"])
    return ["attention" if i in idx else "conv" for i in range(L)]


# ------------------------------------------------------------------------ parts
def embed(E, tokens):
    """x = E[token]: a row gather, no scale (src/lfm25_engine.c:360, src/lfm25_gpu.cu:725-741)."""
    return E[np.asarray(tokens)]


def rms_norm(x, w, eps):
    """x * rsqrt(mean(x^2) + eps) * w over the last axis (src/lfm25_gpu.cu:207-262;
    tools/lfm25_fp64_ref.py:81-82)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def rope_neox(x, positions, theta, rotary_dim=None):
    """NeoX rotation of x [T, heads, hd] at absolute positions: element j pairs with
    j + hd/2, angle pos * theta^(-2j/hd) (src/lfm25_gpu.cu:459-474;
    tools/lfm25_fp64_ref.py:93-100)."""
    hd = x.shape[-1]
    rd = hd if rotary_dim is None else rotary_dim
    half = rd // 2
    inv_freq = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / rd)
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * inv_freq[None, None, :]
    c, s = np.cos(a), np.sin(a)
    x0, x1 = x[..., :half], x[..., half:rd]
    return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c, x[..., rd:]], axis=-1)


def short_conv_mixer(h, w_in, taps, w_out):
    """Gated short convolution over a whole sequence h [T, d]
    (src/lfm25_gpu.cu:344-415: order b, c, x at :378-380, taps at :387-391, gate at :396;
    recurrence over tokens src/lfm25_gpu.cu:1046-1099; tools/lfm25_fp64_ref.py:118-126).
    taps [d, K]: tap K-1 multiplies the current token; before the sequence u is 0."""
    T, d = h.shape
    K = taps.shape[1]
    bcx = h @ w_in.T
    B, C, xg = bcx[:, :d], bcx[:, d:2 * d], bcx[:, 2 * d:]
    u = B * xg
    up = np.concatenate([np.zeros((K - 1, d)), u], axis=0)
    y = np.zeros_like(u)
    for j in range(K):
        y += taps[:, j][None, :] * up[j:j + T]
    return (C * y) @ w_out.T


def gqa_attention_mixer(h, wq, wk, wv, wo, qn_w, kn_w, n_heads, n_kv, hd, eps, theta, positions=None,
                        window=None):
    """Grouped-query attention over a whole sequence h [T, d], causal
    (projections src/lfm25_engine.c:386-390; q/k norm and rotation src/lfm25_gpu.cu:420-485;
    scores scaled by 1/sqrt(hd) :520, head h uses key head h // (H/G) :518, token at p
    sees keys 0..p :531, softmax :546-553; tools/lfm25_fp64_ref.py:128-143)."""
    T = h.shape[0]
    pos = np.arange(T) if positions is None else np.asarray(positions)
    q = (h @ wq.T).reshape(T, n_heads, hd)
    k = (h @ wk.T).reshape(T, n_kv, hd)
    v = (h @ wv.T).reshape(T, n_kv, hd)
    if qn_w is not None:
        q = rms_norm(q, qn_w, eps)
        k = rms_norm(k, kn_w, eps)
    if theta is not None:
        q = rope_neox(q, pos, theta)
        k = rope_neox(k, pos, theta)
    rep = n_heads // n_kv
    out = np.zeros((T, n_heads, hd))
    for hh in range(n_heads):
        g = hh // rep
        s = (q[:, hh, :] @ k[:, g, :].T) / np.sqrt(hd)          # [T, T]
        mask = pos[None, :] > pos[:, None]
        if window:
            mask |= pos[None, :] < (pos[:, None] - window + 1)
        s = np.where(mask, -np.inf, s)
        s = np.exp(s - s.max(-1, keepdims=True))
        s /= s.sum(-1, keepdims=True)
        out[:, hh, :] = s @ v[:, g, :]
    return out.reshape(T, n_heads * hd) @ wo.T


def swiglu_ffn(h, w1, w3, w2):
    """(silu(h W1^T) * (h W3^T)) W2^T with silu(g) = g / (1 + exp(-g))
    (src/lfm25_gpu.cu:583-618, silu at :615-616; tools/lfm25_fp64_ref.py:159-161)."""
    g = h @ w1.T
    u = h @ w3.T
    return (g / (1.0 + np.exp(-g)) * u) @ w2.T


def lm_head(x, norm_w, eps, out_w):
    """Final RMSNorm then the output matrix (src/lfm25_gpu.cu:1216-1237;
    tools/lfm25_fp64_ref.py:163)."""
    return rms_norm(x, norm_w, eps) @ out_w.T


# ------------------------------------------------------------------------ model
class PlainLfm2:
    def __init__(self, model_dir):
        self.cfg = cfg = read_config(model_dir)
        self.w = read_safetensors(os.path.join(model_dir, "model.safetensors"))
        self.d = cfg["hidden_size"]
        self.H = cfg["num_attention_heads"]
        self.G = cfg.get("num_key_value_heads", self.H)
        self.hd = cfg.get("head_dim") or self.d // self.H
        self.eps = cfg["norm_eps"]
        self.theta = cfg["rope_theta"]
        self.kinds = layer_kinds(cfg)
        self.tied = cfg.get("tie_embedding", True)

    def forward(self, tokens, rows=None):
        """Logits [T, vocab] (float64) for a whole sequence; layer order and residuals
        as in src/lfm25_engine.c:365-423.  `rows`: positions whose logits are wanted (all if None);
        the sequence runs whole either way."""
        w = self.w
        x = embed(w["model.embed_tokens.weight"], tokens)
        for i, kind in enumerate(self.kinds):
            p = f"model.layers.{i}."
            h = rms_norm(x, w[p + "operator_norm.weight"], self.eps)
            if kind == "conv":
                K = self.cfg["conv_L_cache"]
                o = short_conv_mixer(h, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"].reshape(self.d, K),
                                     w[p + "conv.out_proj.weight"])
            else:
                a = p + "self_attn."
                o = gqa_attention_mixer(h, w[a + "q_proj.weight"], w[a + "k_proj.weight"], w[a + "v_proj.weight"],
                                        w[a + "out_proj.weight"], w[a + "q_layernorm.weight"],
                                        w[a + "k_layernorm.weight"], self.H, self.G, self.hd, self.eps, self.theta)
            x = x + o
            h = rms_norm(x, w[p + "ffn_norm.weight"], self.eps)
            f = p + "feed_forward."
            x = x + swiglu_ffn(h, w[f + "w1.weight"], w[f + "w3.weight"], w[f + "w2.weight"])
        out_w = w["model.embed_tokens.weight"] if self.tied else w["lm_head.weight"]
        if rows is not None:
            x = x[np.asarray(rows)]
        return lm_head(x, w["model.embedding_norm.weight"], self.eps, out_w)


# --------------------------------------------------------------------- sampling
_M64 = (1 << 64) - 1


def _mix64(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_draw(seed, request_key, token_index):
    """The engine's counter-based uniform number (its own definition; the reference
    uses a sequential xorshift128+ stream, src/sampler.c:20-45)."""
    z = _mix64((seed + 0x9E3779B97F4A7C15 * (request_key + 1)) & _M64)
    z = _mix64(z ^ ((token_index * 0xD1B54A32D192ED03 + 0x8CB92BA72F3D8DD7) & _M64))
    return (z >> 40) / 16777216.0


def sample_token(logits, temp=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, recent=(), u=0.0):
    """The reference's sampling chain (src/sampler.c:99-230): greedy when temp <= 0 (first
    maximum); else repetition penalty per occurrence -> max -> min-p on scaled logits ->
    descending order -> top-k -> softmax -> top-p + renormalise -> one draw.  Equal values
    are ordered lowest index first, and the draw `u` walks the kept tokens in vocabulary
    order (the reference walks its sorted list; the distribution is the same)."""
    l = np.asarray(logits, dtype=np.float64).copy()
    if temp <= 0:
        return int(np.argmax(l))
    if repeat_penalty > 1.0:
        for t in recent:
            if 0 <= t < l.size:
                l[t] = l[t] / repeat_penalty if l[t] > 0 else l[t] * repeat_penalty
    s = (l - l.max()) / temp
    keep = np.ones(l.size, bool)
    if 0.0 < min_p < 1.0:
        keep &= s >= np.log(min_p)
    order = np.argsort(-s, kind="stable")
    order = order[keep[order]]
    if top_k > 0 and order.size > top_k:
        order = order[:top_k]
    p = np.exp(s[order])
    p /= p.sum()
    if 0.0 < top_p < 1.0:
        cum = np.cumsum(p)
        n = int(np.searchsorted(cum, top_p, side="left")) + 1
        n = min(n, order.size)
        order, p = order[:n], p[:n] / p[:n].sum()
    idx = np.sort(order)
    w = np.zeros(l.size)
    w[order] = p
    cum = np.cumsum(w[idx])
    j = int(np.searchsorted(cum, u * cum[-1], side="left"))
    return int(idx[min(j, idx.size - 1)])
