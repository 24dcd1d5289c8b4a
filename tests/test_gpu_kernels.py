"""Each CUDA kernel alone against a plain fp32/fp64 reference of the same
operation, at sizes other than the engine's tests use (head sizes in steps of
16, widths and vocabularies that are no power of two, odd row counts)."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as plain

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a)).to(dtype).cuda()


def close(got, ref, dtype, scale=1.0):
    got = got.float().cpu().numpy().astype(np.float64)
    tol = 2e-5 if dtype == "float32" else 2e-2
    err = np.abs(got - ref).max()
    assert err <= tol * scale * max(1.0, np.abs(ref).max()), f"max error {err:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,V,n", [(80, 301, 7), (2048, 1000, 3), (17, 5, 33)])
def test_embed(dtype, d, V, n):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(0)
    table = dev(rng.normal(size=(V, d)), DT[dtype])
    toks = rng.integers(0, V, n)
    out = torch.empty(n, d, device="cuda")
    ops.embed(dev(toks, torch.int32), table, out)
    assert torch.equal(out, table.float()[torch.as_tensor(toks).cuda()])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,n,eps", [(80, 5, 1e-5), (2048, 3, 1e-6), (333, 9, 1e-3), (4096 + 16, 2, 1e-5)])
def test_rmsnorm(dtype, d, n, eps):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(1)
    x = rng.normal(size=(n, d)) * 3
    w = 1 + 0.1 * rng.normal(size=d)
    xd, wd = dev(x), dev(w)
    out = torch.empty(n, d, dtype=DT[dtype], device="cuda")
    ops.rmsnorm(xd, wd, eps, out)
    close(out, plain.rms_norm(xd.cpu().numpy().astype(np.float64), wd.cpu().numpy().astype(np.float64), eps), dtype)
    idx = dev([n - 1, 0, n - 1], torch.int32)
    out2 = torch.empty(3, d, dtype=DT[dtype], device="cuda")
    ops.rmsnorm(xd, wd, eps, out2, idx)
    assert torch.equal(out2, out[[n - 1, 0, n - 1]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 301, 80), (7, 130, 200), (65, 64, 48), (130, 257, 1000), (3, 2048, 5632),
                                   (300, 520, 136), (512, 2048, 192), (257, 129, 72), (1100, 777, 2048), (2048, 3080, 136),
                                   (260, 2048, 8192), (40, 2048, 8192)])
def test_linear(dtype, M, N, K):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(2)
    a = dev(rng.normal(size=(M, K)), DT[dtype])
    w = dev(rng.normal(size=(N, K)) * 0.05, DT[dtype])
    ref = a.double().cpu().numpy() @ w.double().cpu().numpy().T
    out = torch.empty(M, N, dtype=DT[dtype], device="cuda")
    ops.linear(a, w, out)
    close(out, ref, dtype, scale=2.0)
    res = dev(rng.normal(size=(M, N)))
    acc = res.clone()
    ops.linear(a, w, acc, accumulate=True)                 # the residual stream takes the product in fp32
    close(acc, res.double().cpu().numpy() + ref, "float32" if dtype == "float32" else dtype, scale=2.0)
    logits = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.linear(a, w, logits)
    close(logits, ref, "float32", scale=4.0 if dtype == "float32" else 1.0)   # fp32 out even from bf16 operands


def test_linear_is_batch_invariant():
    """A row's fp32 result does not depend on how many rows run with it."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(3)
    a = dev(rng.normal(size=(70, 333)))
    w = dev(rng.normal(size=(129, 333)))
    full = torch.empty(70, 129, device="cuda")
    ops.linear(a, w, full)
    for lo, hi in ((0, 1), (5, 7), (63, 70)):
        part = torch.empty(hi - lo, 129, device="cuda")
        ops.linear(a[lo:hi].contiguous(), w, part)
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("F,n", [(200, 5), (5632, 3), (33, 17)])
def test_swiglu(dtype, F, n):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(4)
    gu = dev(rng.normal(size=(n, 2 * F)) * 2, DT[dtype])
    out = torch.empty(n, F, dtype=DT[dtype], device="cuda")
    ops.swiglu(gu, out)
    g, u = gu.double().cpu().numpy()[:, :F], gu.double().cpu().numpy()[:, F:]
    close(out, g / (1 + np.exp(-g)) * u, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,K,lens", [(80, 3, (5, 1, 2, 9)), (96, 4, (1, 1, 1)), (200, 2, (7, 2)), (64, 5, (3, 2, 1, 11)),
                                      (80, 3, (40, 1, 13, 50, 2)), (96, 4, (33, 2, 31)), (200, 2, (70, 9)), (64, 5, (30, 41))])
def test_shortconv_continues_state(dtype, d, K, lens):
    """Portions of any length (also shorter than K-1) continue each row's state; slots are not
    in row order; the rolled state equals the last K-1 values of u."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(5)
    R, T = len(lens), sum(lens)
    taps = rng.normal(size=(d, K))
    n_slots = R + 2
    slots = rng.permutation(n_slots)[:R]
    state0 = rng.normal(size=(n_slots, K - 1, d))
    bcx = dev(rng.normal(size=(T, 3 * d)), DT[dtype])
    b64 = bcx.double().cpu().numpy()
    state = dev(state0)
    cu = np.concatenate([[0], np.cumsum(lens)])
    out = torch.empty(T, d, dtype=DT[dtype], device="cuda")
    ops.shortconv(bcx, dev(taps), state, dev(slots, torch.int32),
                  dev(np.repeat(np.arange(R), lens), torch.int32), dev(cu, torch.int32), out)
    taps32 = dev(taps).double().cpu().numpy()
    st32 = dev(state0).double().cpu().numpy()
    new_state = state.double().cpu().numpy()
    for r in range(R):
        seg = b64[cu[r]:cu[r + 1]]
        u = np.concatenate([st32[slots[r]], seg[:, :d] * seg[:, 2 * d:]], 0)
        y = sum(taps32[:, j][None] * u[j:j + lens[r]] for j in range(K))
        close(out[cu[r]:cu[r + 1]], seg[:, d:2 * d] * y, dtype)
        np.testing.assert_allclose(new_state[slots[r]], u[-(K - 1):], rtol=1e-6, atol=1e-6)
    untouched = [s for s in range(n_slots) if s not in slots]
    np.testing.assert_array_equal(new_state[untouched], st32[untouched])


def paged_setup(rng, seqs, G, hd, page, dtype, n_pages=None):
    """Scatters each sequence's keys/values over shuffled pages; returns pages and block tables."""
    blocks = [math.ceil(s / page) for s in seqs]
    n_pages = n_pages or sum(blocks) + 3
    perm = rng.permutation(n_pages)
    kp = torch.zeros(n_pages, G, page, hd, dtype=DT[dtype], device="cuda")
    vp = torch.zeros_like(kp)
    kp.fill_(float("nan")); vp.fill_(float("nan"))          # a read outside a request's keys would show
    table = np.full((len(seqs), max(blocks)), -1, np.int32)
    o = 0
    for r, b in enumerate(blocks):
        table[r, :b] = perm[o:o + b]
        o += b
    return kp, vp, table


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("blocked", [False, True])
@pytest.mark.parametrize("H,G,hd,page,rot", [(4, 2, 16, 4, 16), (6, 3, 48, 8, 48), (8, 1, 80, 16, 32), (2, 2, 128, 2, 0),
                                             (5, 5, 256, 64, 256), (8, 2, 64, 16, 64), (6, 2, 64, 8, 64), (4, 4, 128, 32, 128),
                                             (8, 1, 128, 64, 64), (2, 1, 64, 16, 0)])
def test_qk_norm_rope_write_and_attention(dtype, H, G, hd, page, rot, blocked):
    """The fused q/k kernel and the paged attention together against the plain attention, for
    rows that continue at different positions; pages are scattered and other pages hold NaN."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(6)
    theta, eps = 12345.0, 1e-5
    starts, lens = (0, 137, 5), (9, 1, 75)       # a fresh row, a decode row deep in its context, a long portion
    seqs = [s + n for s, n in zip(starts, lens)]
    kp, vp, table = paged_setup(rng, seqs, G, hd, page, dtype)
    qn, kn = 1 + 0.1 * rng.normal(size=hd), 1 + 0.1 * rng.normal(size=hd)
    inv_freq = (theta ** (-2.0 * np.arange(rot // 2) / rot)).astype(np.float32) if rot else None
    full = [rng.normal(size=(s, (H + 2 * G) * hd)) for s in seqs]
    tb = dev(table, torch.int32)

    def run(rows_tokens):      # rows_tokens: list of (row, first position, count)
        pos = np.concatenate([np.arange(p0, p0 + n) for _, p0, n in rows_tokens])
        rot_ = np.concatenate([np.full(n, r) for r, _, n in rows_tokens])
        qkv = dev(np.concatenate([full[r][p0:p0 + n] for r, p0, n in rows_tokens]), DT[dtype])
        ops.qk_norm_rope_write(qkv, dev(qn), dev(kn), None if inv_freq is None else dev(inv_freq),
                               dev(pos, torch.int32), dev(rot_, torch.int32), tb, kp, vp, H, G, hd, rot, eps)
        out = torch.empty(len(pos), H * hd, dtype=DT[dtype], device="cuda")
        per_row = [0, 0, 0]
        for r, _, n in rows_tokens:
            per_row[r] = n
        cu = np.concatenate([[0], np.cumsum(per_row)])
        # blocked: the kernel for prompt portions (rows of several tokens); else the one that takes
        # every token by itself
        ops.paged_attention(qkv, kp, vp, tb, dev(pos, torch.int32), dev(rot_, torch.int32), out, H, G, hd,
                            1 / math.sqrt(hd), cu_q=dev(cu, torch.int32) if blocked else None, all_single=not blocked,
                            max_seq_len=max(seqs))
        return out

    # first the earlier parts of rows 1 and 2 (their "cache"), then the step under test
    run([(1, 0, starts[1]), (2, 0, starts[2])])
    out = run([(r, starts[r], lens[r]) for r in range(3)])
    o = 0
    for r in range(3):
        x = dev(full[r], DT[dtype]).double().cpu().numpy().reshape(seqs[r], H + 2 * G, hd)
        q, k, v = x[:, :H], x[:, H:H + G], x[:, H + G:]
        q, k = plain.rms_norm(q, qn.astype(np.float32), eps), plain.rms_norm(k, kn.astype(np.float32), eps)
        if rot:
            q = plain.rope_neox(q, np.arange(seqs[r]), theta, rot)
            k = plain.rope_neox(k, np.arange(seqs[r]), theta, rot)
        ref = np.zeros((seqs[r], H, hd))
        for h in range(H):
            g = h // (H // G)
            s = q[:, h] @ k[:, g].T / math.sqrt(hd)
            s = np.where(np.triu(np.ones((seqs[r], seqs[r]), bool), 1), -np.inf, s)
            p = np.exp(s - s.max(-1, keepdims=True))
            ref[:, h] = (p / p.sum(-1, keepdims=True)) @ v[:, g]
        close(out[o:o + lens[r]], ref[starts[r]:].reshape(lens[r], H * hd), dtype, scale=3.0)
        o += lens[r]
        # the keys in the pages carry the rotation of their absolute positions (the scores above see only
        # differences of positions, so they cannot tell), and the values lie where the table says
        kd, vd = kp.double().cpu().numpy(), vp.double().cpu().numpy()
        for pos in sorted({0, seqs[r] // 2, seqs[r] - 1}):
            pg, off = table[r][pos // page], pos % page
            close(torch.as_tensor(kd[pg, :, off]), k[pos], dtype, scale=2.0)
            close(torch.as_tensor(vd[pg, :, off]), v[pos], dtype, scale=2.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,blocked", [(32, False), (64, False), (64, True), (128, False)])
def test_attention_finds_a_far_key_and_respects_the_window(dtype, hd, blocked):
    """One key among hundreds matches the query (score far above the rest): the output must be
    that key's value, wherever its page lies; with a window that ends just after it, it must not."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(7)
    H = G = 1
    page, n = 8, 700
    kp, vp, table = paged_setup(rng, [n], G, hd, page, dtype)
    keys = rng.normal(size=(n, hd)) * 0.1
    vals = rng.normal(size=(n, hd))
    q = rng.normal(size=hd)
    for far in (0, 7, 8, 333, 698):
        k2 = keys.copy()
        k2[far] = q * 4.0                       # q.k = 4 |q|^2 ~ 128, every other score ~ 0.5
        for p in range(n):
            pg, off = table[0, p // page], p % page
            kp[pg, 0, off] = dev(k2[p], DT[dtype]); vp[pg, 0, off] = dev(vals[p], DT[dtype])
        qd = dev(q[None], DT[dtype])
        out = torch.empty(1, hd, dtype=DT[dtype], device="cuda")
        args = (qd, kp, vp, dev(table, torch.int32), dev([n - 1], torch.int32), dev([0], torch.int32), out, 1, 1, hd, 1.0)
        kw = dict(cu_q=dev([0, 1], torch.int32) if blocked else None, all_single=not blocked, max_seq_len=n)
        ops.paged_attention(*args, **kw)
        close(out, dev(vals[far], DT[dtype]).double().cpu().numpy()[None], dtype)
        w_in, w_out = n - far, n - far - 1       # the window that just holds the key / just misses it
        ops.paged_attention(*args, window=w_in, **kw)
        close(out, dev(vals[far], DT[dtype]).double().cpu().numpy()[None], dtype)
        if w_out >= 1:
            ops.paged_attention(*args, window=w_out, **kw)
            assert (out.float().cpu().numpy() - vals[far]).std() > 0.3


@pytest.mark.parametrize("H,G,page,window", [(4, 2, 16, 0), (3, 1, 64, 0), (12, 2, 8, 100), (2, 2, 64, 129), (9, 3, 32, 0)])
def test_attention_prefill_tc_long_portions(H, G, page, window):
    """The tcgen05 kernel for prompt portions (head size 64): requests whose portions span several
    128-token blocks and many 64-key tiles, start inside a page and inside a tile, with and without
    a window, beside a single-token request; never-written cache slots hold NaN.  Against fp64."""
    portions_case(H, G, page, window, (0, 70, 513, 5, 200), (300, 200, 129, 1, 128), 0)


@pytest.mark.parametrize("H,G,page,window", [(4, 2, 16, 0), (12, 2, 8, 100), (8, 8, 64, 0)])
def test_attention_of_decoding_rows_beside_portions(H, G, page, window):
    """A batch as the scheduler makes it, decoding rows first and portions of prompts after them:
    the decoding rows go to the sliced kernel and the portions to the blocked one, each with its
    own part of the tables.  Against fp64."""
    portions_case(H, G, page, window, (300, 70, 513, 5, 200, 64), (1, 1, 1, 140, 128, 2), 3)
    # head size 128: the sliced kernel beside the blocked mma.sync kernel
    portions_case(H, G, page, window, (300, 70, 513, 5, 200, 64), (1, 1, 1, 140, 128, 2), 3, hd=128)


def portions_case(H, G, page, window, starts, lens, single_prefix, hd=64):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(31)
    seqs = [a + n for a, n in zip(starts, lens)]
    kp, vp, table = paged_setup(rng, seqs, G, hd, page, "bfloat16")
    ks = [rng.normal(size=(n, G, hd)) for n in seqs]
    vs = [rng.normal(size=(n, G, hd)) for n in seqs]
    for r, n in enumerate(seqs):
        ks[r][n // 3] *= 12.0                      # one key that stands out: a lost tile shows, and rows raise their reference late
        for b in range(math.ceil(n / page)):
            a, e = b * page, min(n, (b + 1) * page)
            kp[table[r, b], :, :e - a] = dev(ks[r][a:e], torch.bfloat16).transpose(0, 1)
            vp[table[r, b], :, :e - a] = dev(vs[r][a:e], torch.bfloat16).transpose(0, 1)
    qs = [rng.normal(size=(n, H, hd)) for n in lens]
    # q as a slice of a wider matrix, as the fused q/k/v product leaves it
    wide = torch.zeros(sum(lens), (H + 2 * G) * hd, dtype=torch.bfloat16, device="cuda")
    wide[:, :H * hd] = dev(np.concatenate(qs).reshape(-1, H * hd), torch.bfloat16)
    q = wide[:, :H * hd]
    pos = np.concatenate([np.arange(a, a + n) for a, n in zip(starts, lens)])
    row_of = np.repeat(np.arange(len(lens)), lens)
    cu = np.concatenate([[0], np.cumsum(lens)])
    assert ops.attention_prefill_tc_supported(q, kp, H, G, hd) == (hd == 64)
    out = torch.full((sum(lens), H * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.paged_attention(q, kp, vp, dev(table, torch.int32), dev(pos, torch.int32), dev(row_of, torch.int32), out, H, G, hd,
                        1 / math.sqrt(hd), window=window, cu_q=dev(cu, torch.int32), all_single=False, max_seq_len=max(seqs),
                        single_prefix=single_prefix)
    ops.check_tc_status()
    o = 0
    for r, n in enumerate(lens):
        qq = q[o:o + n].double().cpu().numpy().reshape(n, H, hd)
        kk = dev(ks[r], torch.bfloat16).double().cpu().numpy()
        vv = dev(vs[r], torch.bfloat16).double().cpu().numpy()
        ref = np.zeros((n, H, hd))
        kpos, qpos = np.arange(seqs[r])[None], (starts[r] + np.arange(n))[:, None]
        hidden = (kpos > qpos) | ((kpos < qpos - window + 1) if window else False)
        for h in range(H):
            g = h // (H // G)
            sc = np.where(hidden, -np.inf, qq[:, h] @ kk[:, g].T / math.sqrt(hd))
            pr = np.exp(sc - sc.max(-1, keepdims=True))
            ref[:, h] = (pr / pr.sum(-1, keepdims=True)) @ vv[:, g]
        close(out[o:o + n], ref.reshape(n, H * hd), "bfloat16", scale=3.0)
        o += n


@pytest.mark.parametrize("V", [301, 65536, 5, 1025])
def test_argmax_first_maximum(V):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(8)
    l = rng.normal(size=(6, V)).astype(np.float32)
    l[1, [V // 2, V - 1]] = 9.0                     # a tie: the lower index wins
    l[2, :] = -1.0                                  # all equal: index 0
    l[3, V - 1] = 50.0
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.argmax(dev(l), out)
    ref = [int(r.argmax()) for r in l]
    assert out.tolist() == ref and ref[1] == V // 2 and ref[2] == 0 and ref[3] == V - 1


@pytest.mark.parametrize("V", [301, 4096, 65536])
def test_sampling_chain_matches_plain(V):
    from tuff_b200.sampling import Sampler, SamplingParams, SampleRow
    rng = np.random.default_rng(9)
    cases = [
        SamplingParams(temp=0.8, seed=2),
        SamplingParams(temp=1.5, top_k=5, seed=3),
        SamplingParams(temp=0.7, top_p=0.6, seed=4),
        SamplingParams(temp=1.0, min_p=0.2, seed=5),
        SamplingParams(temp=0.9, top_k=40, top_p=0.9, min_p=0.02, repeat_penalty=1.3, repeat_last_n=8, seed=6),
        SamplingParams(temp=0.0),
        SamplingParams(temp=2.0, top_k=1, seed=7),
        SamplingParams(temp=1.0, top_p=0.3, seed=8),
    ]
    logits = (rng.normal(size=(len(cases), V)) * 3).astype(np.float32)
    logits[1, :10] = 7.0                           # ties across the top-k edge
    logits[7, [3, 9]] = 12.0                       # two equal leaders at the nucleus edge
    recent = [list(rng.integers(0, V, 12)) for _ in cases]
    sampler = Sampler(V, "cuda:0")
    ld = dev(logits)
    hits = 0
    for tok_index in range(24):
        rows = [SampleRow(p, 100 + i, tok_index, recent[i]) for i, p in enumerate(cases)]
        got = sampler.sample(ld, rows).tolist()
        for i, p in enumerate(cases):
            u = plain.uniform_draw(p.seed, 100 + i, tok_index)
            rec = recent[i][-p.repeat_last_n:] if p.repeat_penalty > 1 else ()
            want = plain.sample_token(logits[i], p.temp, p.top_k, p.top_p, p.min_p, p.repeat_penalty, rec, u)
            hits += got[i] == want
            if got[i] != want:       # only a draw that lands on a boundary within fp32 rounding may differ
                w64 = np.exp((logits[i].astype(np.float64) - logits[i].max()) / p.temp)
                cum = np.cumsum(w64 / w64.sum())
                assert p.temp > 0 and min(abs(cum - u)) < 1e-4, (i, tok_index, got[i], want)
    assert hits >= 24 * len(cases) - 2
    # the draw of a row does not depend on the rows beside it
    solo = sampler.sample(ld[4:5], [SampleRow(cases[4], 104, 5, recent[4])]).tolist()
    both = sampler.sample(ld, [SampleRow(p, 100 + i, 5, recent[i]) for i, p in enumerate(cases)]).tolist()
    assert solo[0] == both[4]


def test_temperature_sampling_follows_the_distribution():
    from tuff_b200.sampling import Sampler, SamplingParams, SampleRow
    V = 50
    rng = np.random.default_rng(10)
    l = rng.normal(size=V).astype(np.float32) * 2
    p = np.exp(l.astype(np.float64) / 0.7); p /= p.sum()
    sampler = Sampler(V, "cuda:0")
    n = 4000
    ld = dev(np.tile(l, (n, 1)))
    sp = SamplingParams(temp=0.7, seed=11)
    toks = np.array(sampler.sample(ld, [SampleRow(sp, 1, i) for i in range(n)]).tolist())
    freq = np.bincount(toks, minlength=V) / n
    assert np.abs(freq - p).max() < 4 * np.sqrt(p.max() / n) + 0.01


@pytest.mark.parametrize("M,N,K", [(1, 301, 80), (8, 2048, 2048), (7, 264, 96), (8, 2048, 5632), (5, 6144, 2048), (3, 40, 4096), (6, 520, 1000)])
def test_gemm_decode_epilogues_and_fused_norm(M, N, K):
    """The decode products: store / accumulate, with and without the RMSNorm done by the product
    itself, against fp64 (the normed rows rounded to bf16 as the separate norm kernel stores them)."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(20)
    w = dev(rng.normal(size=(N, K)) * 0.05, torch.bfloat16)
    x = dev(rng.normal(size=(M, K)) * 2)
    nw = dev(1 + 0.1 * rng.normal(size=K))
    h = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    ops.rmsnorm(x, nw, 1e-5, h)
    ref = h.double().cpu().numpy() @ w.double().cpu().numpy().T
    lazy = ops.NormedRows(x, nw, 1e-5, torch.bfloat16)
    assert lazy.fusable(w) == (K <= ops.FUSED_NORM_MAX_K)
    for a in (h, lazy) if lazy.fusable(w) else (h,):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.gemm_decode(a, w, out)
        close(out, ref, "bfloat16")
        o32 = torch.full((M, N), float("nan"), device="cuda")
        ops.gemm_decode(a, w, o32)
        close(o32, ref, "float32", scale=4.0)
        res = dev(rng.normal(size=(M, N)))
        acc = res.clone()
        ops.gemm_decode(a, w, acc, ops.EPI_ACCUM)
        close(acc, res.double().cpu().numpy() + ref, "float32", scale=4.0)
    # linear() routes few-token bf16 products here, with the lazy norm too
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.linear(ops.NormedRows(x, nw, 1e-5, torch.bfloat16), w, out)
    close(out, ref, "bfloat16")


@pytest.mark.parametrize("M,d,K,N2", [(8, 2048, 2048, 6144), (1, 2048, 5632, 2048), (7, 264, 96, 520), (5, 1000, 80, 301),
                                     (8, 2048, 8192, 2048)])
def test_gemm_decode_norm_split_over_two_products(M, d, K, N2):
    """A product that adds into the residual prepares the RMSNorm that follows (bf16(x * w) and sums of
    squares per CTA), and the product that consumes the norm scales its rows: against fp64, with
    epilogues store and swiglu; the preparation is dropped when x is written again."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(24)
    a = dev(rng.normal(size=(M, K)), torch.bfloat16)
    w1 = dev(rng.normal(size=(d, K)) * 0.05, torch.bfloat16)
    x0 = dev(rng.normal(size=(M, d)) * 2)
    nw = dev(1 + 0.1 * rng.normal(size=d))
    w2 = dev(rng.normal(size=(N2, d)) * 0.05, torch.bfloat16)
    eps = 1e-5
    x = x0.clone()
    ops.announce_norm(x, nw, eps)
    ops.linear(a, w1, x, accumulate=True)
    x_ref = x0.double().cpu().numpy() + a.double().cpu().numpy() @ w1.double().cpu().numpy().T
    close(x, x_ref, "float32", scale=4.0)
    lazy = ops.NormedRows(x, nw, eps, torch.bfloat16)
    assert lazy.pre is not None and lazy.fusable(w2)
    x64 = x.double().cpu().numpy()
    h = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + eps) * nw.double().cpu().numpy()
    ref = h @ w2.double().cpu().numpy().T
    out = torch.full((M, N2), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear(lazy, w2, out)
    close(out, ref, "bfloat16", scale=1.5)
    if N2 % 2 == 0:
        F = N2 // 2
        act = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.linear_swiglu(lazy, w2, act)
        gu = torch.as_tensor(ref).to(torch.bfloat16).double().numpy()
        close(act, gu[:, :F] / (1 + np.exp(-gu[:, :F])) * gu[:, F:], "bfloat16", scale=2.0)
    # the same norm computed by the product itself (nothing prepared) agrees
    if K <= ops.FUSED_NORM_MAX_K or True:
        plain_h = torch.empty(M, d, dtype=torch.bfloat16, device="cuda")
        ops.rmsnorm(x, nw, eps, plain_h)
        out2 = torch.empty(M, N2, dtype=torch.bfloat16, device="cuda")
        ops.linear(plain_h, w2, out2)
        close(out2, ref, "bfloat16", scale=1.5)
    # written again by a kernel of this module, or in place by torch: the preparation is void
    ops.linear(a, w1, x, accumulate=True)
    assert ops.NormedRows(x, nw, eps, torch.bfloat16).pre is None
    ops.announce_norm(x, nw, eps)
    ops.linear(a, w1, x, accumulate=True)
    assert ops.NormedRows(x, nw, eps, torch.bfloat16).pre is not None
    x.add_(1.0)
    assert ops.NormedRows(x, nw, eps, torch.bfloat16).pre is None
    ops.check_tc_status()


@pytest.mark.parametrize("M,F,K", [(1, 100, 80), (8, 5632, 2048), (8, 264, 96), (7, 40, 64), (4, 8192, 2048)])
def test_gemm_decode_swiglu(M, F, K):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(21)
    w13 = dev(rng.normal(size=(2 * F, K)) * 0.05, torch.bfloat16)
    a = dev(rng.normal(size=(M, K)), torch.bfloat16)
    gu = (a.double() @ w13.double().T).to(torch.bfloat16).double().cpu().numpy()
    ref = gu[:, :F] / (1 + np.exp(-gu[:, :F])) * gu[:, F:]
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear_swiglu(a, w13, out)
    close(out, ref, "bfloat16")


@pytest.mark.parametrize("M,d,L", [(1, 80, 3), (8, 2048, 3), (8, 96, 4), (5, 200, 2)])
def test_gemm_decode_shortconv(M, d, L):
    """The input projection with the gated convolution and the state roll fused on, one token per
    row, against the projection followed by the stand-alone convolution kernel's definition."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(22)
    w_in = dev(rng.normal(size=(3 * d, d)) * 0.1, torch.bfloat16)
    a = dev(rng.normal(size=(M, d)), torch.bfloat16)
    taps = dev(rng.normal(size=(d, L)))
    n_slots = M + 3
    slots = rng.permutation(n_slots)[:M]
    state0 = dev(rng.normal(size=(n_slots, L - 1, d)))
    state = state0.clone()
    out = torch.full((M, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops.linear_shortconv(a, w_in, taps, state, dev(slots, torch.int32), out)
    bcx = (a.double() @ w_in.double().T).to(torch.bfloat16).double().cpu().numpy()
    t64, s64 = taps.double().cpu().numpy(), state0.double().cpu().numpy()
    new = state.double().cpu().numpy()
    for m in range(M):
        u = bcx[m, :d] * bcx[m, 2 * d:]
        hist = np.concatenate([s64[slots[m]], u[None]], 0)          # [L, d]
        y = (t64.T * hist).sum(0)
        close(out[m:m + 1], (bcx[m, d:2 * d] * y)[None], "bfloat16", scale=2.0)
        # u = B * x from values rounded to bf16: where the kernel's fp32 sum and the fp64 product
        # fall on different sides of a rounding boundary, u differs by a bf16 step
        np.testing.assert_allclose(new[slots[m], -1], hist[-1], rtol=2e-2, atol=2e-2 * np.abs(hist[-1]).max())
        np.testing.assert_array_equal(new[slots[m], :-1], s64[slots[m], 1:])       # the older entries only move
    other = [s for s in range(n_slots) if s not in slots]
    np.testing.assert_array_equal(new[other], s64[other])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,F,K", [(3, 256, 64), (16, 640, 96), (64, 384, 128), (200, 256, 80), (2048, 5632, 256), (129, 128, 64),
                                   (300, 8192, 128)])
def test_linear_swiglu_blocked_layout(dtype, M, F, K):
    """Gate and up stacked in blocks of 128 rows: the few-token product, the tensor-core product with
    the activation in its epilogue (more than 128 tokens) and the unfused path all give silu(g) * u."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(23)
    w1 = dev(rng.normal(size=(F, K)) * 0.1, DT[dtype])
    w3 = dev(rng.normal(size=(F, K)) * 0.1, DT[dtype])
    a = dev(rng.normal(size=(M, K)), DT[dtype])
    w13, block = ops.stack_gate_up(w1, w3)
    assert block == 128 and w13.shape == (2 * F, K)
    assert torch.equal(w13[:128], w1[:128]) and torch.equal(w13[128:256], w3[:128])
    g = a.double() @ w1.double().T
    u = a.double() @ w3.double().T
    if dtype == "bfloat16":
        g, u = g.to(torch.bfloat16).double(), u.to(torch.bfloat16).double()
    ref = (g / (1 + torch.exp(-g)) * u).cpu().numpy()
    out = torch.full((M, F), float("nan"), dtype=DT[dtype], device="cuda")
    ops.linear_swiglu(a, w13, out, block)
    close(out, ref, dtype, scale=2.0)
    ops.check_tc_status()


# ---- the product of 17 to 128 tokens: K split over a thread-block cluster, sums met in distributed shared memory
@pytest.mark.parametrize("M,N,K", [(17, 2048, 2048), (64, 2048, 5632), (33, 384, 200), (128, 6144, 2048), (100, 520, 1000),
                                   (40, 130, 264), (64, 2048, 8192), (96, 3072, 2048), (20, 128, 64), (9, 2048, 2048),
                                   (16, 6144, 2048), (12, 264, 96)])
def test_gemm_cluster_store_and_accumulate(M, N, K):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(31)
    a = dev(rng.normal(size=(M, K)), torch.bfloat16)
    w = dev(rng.normal(size=(N, K)) * 0.05, torch.bfloat16)
    assert ops._cluster_eligible(a, w, torch.empty(M, N, dtype=torch.bfloat16, device="cuda"), ops.EPI_STORE)
    ref = a.double().cpu().numpy() @ w.double().cpu().numpy().T
    for dt in ("bfloat16", "float32"):
        out = torch.full((M, N), float("nan"), dtype=DT[dt], device="cuda")
        ops.gemm_cluster(a, w, out, ops.EPI_STORE)
        close(out, ref, "bfloat16" if dt == "bfloat16" else "float32", scale=8.0 if dt == "float32" else 1.0)
    x0 = dev(rng.normal(size=(M, N)) * 2)
    x = x0.clone()
    ops.gemm_cluster(a, w, x, ops.EPI_ACCUM)
    close(x, x0.double().cpu().numpy() + ref, "float32", scale=8.0)
    # the sums are added in a fixed order: the same bits every time
    y = x0.clone()
    ops.gemm_cluster(a, w, y, ops.EPI_ACCUM)
    assert torch.equal(x, y)
    # a view with a row stride of its own
    wide = torch.full((M, N + 24), float("nan"), dtype=torch.float32, device="cuda")
    ops.linear(a, w, wide[:, 8:8 + N])
    close(wide[:, 8:8 + N], ref, "float32", scale=8.0)
    assert torch.isnan(wide[:, :8]).all() and torch.isnan(wide[:, 8 + N:]).all()
    ops.check_tc_status()


@pytest.mark.parametrize("M,F,K", [(17, 256, 96), (64, 5632, 2048), (128, 8192, 2048), (50, 1280, 264), (9, 5632, 2048), (16, 8192, 2048)])
def test_gemm_cluster_swiglu(M, F, K):
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(32)
    w1 = dev(rng.normal(size=(F, K)) * 0.05, torch.bfloat16)
    w3 = dev(rng.normal(size=(F, K)) * 0.05, torch.bfloat16)
    a = dev(rng.normal(size=(M, K)), torch.bfloat16)
    w13, block = ops.stack_gate_up(w1, w3)
    assert block == 128
    g = (a.double() @ w1.double().T).to(torch.bfloat16).double().cpu().numpy()
    u = (a.double() @ w3.double().T).to(torch.bfloat16).double().cpu().numpy()
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops._cluster_eligible(a, w13, out, ops.EPI_SWIGLU) == (M <= 64)     # beyond 64 tokens: product, then activation
    ops.linear_swiglu(a, w13, out, block)
    close(out, g / (1 + np.exp(-g)) * u, "bfloat16")
    ops.check_tc_status()


@pytest.mark.parametrize("M,d,K,F", [(64, 2048, 2048, 5632), (17, 264, 96, 256), (128, 2048, 5632, 1024), (37, 1000, 80, 384),
                                     (9, 2048, 8192, 256), (16, 264, 96, 128)])
def test_gemm_cluster_norm_split_over_two_products(M, d, K, F):
    """The product that adds into the residual prepares the RMSNorm that follows (bf16(x * w), sums of squares per
    CTA and token); the products that consume the norm scale their tokens' results: against fp64."""
    from tuff_b200.kernels import ops
    rng = np.random.default_rng(33)
    a = dev(rng.normal(size=(M, K)), torch.bfloat16)
    w1 = dev(rng.normal(size=(d, K)) * 0.05, torch.bfloat16)
    x0 = dev(rng.normal(size=(M, d)) * 2)
    nw = dev(1 + 0.1 * rng.normal(size=d))
    wg, wu = dev(rng.normal(size=(F, d)) * 0.05, torch.bfloat16), dev(rng.normal(size=(F, d)) * 0.05, torch.bfloat16)
    eps = 1e-5
    x = x0.clone()
    ops.announce_norm(x, nw, eps)
    ops.linear(a, w1, x, accumulate=True)
    x_ref = x0.double().cpu().numpy() + a.double().cpu().numpy() @ w1.double().cpu().numpy().T
    close(x, x_ref, "float32", scale=8.0)
    lazy = ops.NormedRows(x, nw, eps, torch.bfloat16)
    assert lazy.pre is not None and lazy.pre["part"].shape[1] == M
    x64 = x.double().cpu().numpy()
    h = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + eps) * nw.double().cpu().numpy()
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear(lazy, wg, out)
    close(out, h @ wg.double().cpu().numpy().T, "bfloat16", scale=1.5)
    w13, block = ops.stack_gate_up(wg, wu)
    act = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear_swiglu(lazy, w13, act, block)
    g = torch.as_tensor(h @ wg.double().cpu().numpy().T).to(torch.bfloat16).double().numpy()
    u = torch.as_tensor(h @ wu.double().cpu().numpy().T).to(torch.bfloat16).double().numpy()
    close(act, g / (1 + np.exp(-g)) * u, "bfloat16", scale=2.0)
    x.add_(1.0)
    assert ops.NormedRows(x, nw, eps, torch.bfloat16).pre is None
    ops.check_tc_status()
