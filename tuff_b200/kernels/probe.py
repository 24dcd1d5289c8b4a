"""Runs one kernel alone on synthetic data and times it: a quick check of a kernel's bandwidth or
throughput, and a small program to put under a profiler.

    python -m tuff_b200.kernels.probe gemm_tc --m 2048 --n 11264 --k 2048
    python -m tuff_b200.kernels.probe gemm_decode --m 8 --n 5632 --k 2048 --epilogue swiglu --norm
    python -m tuff_b200.kernels.probe gemm_cluster --m 64 --n 2048 --k 5632 --epilogue accum
    python -m tuff_b200.kernels.probe decode_chain --m 8 --layers 16
    python -m tuff_b200.kernels.probe attention_decode --batch 8 --context 8192
    python -m tuff_b200.kernels.probe attention_prefill --tokens 2048

    python -m tuff_b200.kernels.probe decode_step --config C.json --batch 8 --context 8192 --steps 6 --no-graphs
    python -m tuff_b200.kernels.probe prefill_step --config C.json --tokens 2048 --steps 3
    python -m tuff_b200.kernels.probe mixed_step --config C.json --batch 32 --context 4096 --tokens 512 --steps 5
    python -m tuff_b200.kernels.probe product_phases --config C.json --batch 64 --context 256

Timing: CUDA events around each launch, after warm-up, with a buffer larger than L2 written
between launches.  Prints the median time and the achieved rate against the bytes or flops the
kernel has to move or do.  The `*_step` forms run whole steps of the engine on a random-weights
model of the sizes in the given config.json (contexts filled without computing them) and print the
wall time a step; under a profiler they give the list of a step's launches.  `product_phases` runs one
decode step (a CUDA graph replay) with the decode products' own time stamps switched on and prints, per
product, when its CTAs started, when they were allowed to read activations, when their first weights
had arrived, when the sums were complete and when the result was written.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import ops


FLUSH_L2 = [True]      # --warm-l2: leave what a launch read in L2 for the next one


def timed(fn, reps: int, warmup: int = 3):
    flush = torch.empty(256 * 1024 * 1024 if FLUSH_L2[0] else 16, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(reps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2] * 1e-3


def run_steps(a) -> int:
    """Whole steps of the engine on a random-weights model of the sizes in `--config`."""
    import json
    import time

    import numpy as np

    if not a.config:
        print("the *_step forms need --config CONFIG.json: the sizes of the model to build", file=sys.stderr)
        return 2
    with open(a.config) as f:
        shape = json.load(f)
    from ..engine import ModelRunner, StepEntry
    from ..engine.engine import Engine
    from ..engine.scheduler import RequestStatus
    from ..sampling import SamplingParams
    rng = np.random.default_rng(0)
    vocab = shape["vocab_size"]
    if a.kernel == "product_phases":
        return product_phases(a, shape)
    if a.kernel == "decode_step":
        n_new = a.steps + 8
        eng = Engine(None, dtype="bfloat16", ctx_size=a.context, max_tokens=a.batch * a.context + 4096, page_size=a.page_size,
                     max_running=a.batch, config=dict(shape), cuda_graphs=not a.no_graphs)
        for i in range(a.batch):
            r = eng.scheduler.add(i, rng.integers(0, vocab, a.context - n_new).tolist(), SamplingParams(max_new_tokens=n_new))
            eng.scheduler.waiting.remove(r)
            r.cache = eng.runner.open(i)
            eng.runner.synthetic_fill(r.cache, a.context - n_new - 1)
            r.status = RequestStatus.RUNNING
            eng.scheduler.running.append(r)
        for _ in range(4):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            eng.step()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / a.steps
        print(f"decode_step batch={a.batch} context={a.context} graphs={not a.no_graphs}: {dt * 1e3:.3f} ms a step, "
              f"{a.batch / dt:.0f} tok/s")
        return 0
    if a.kernel == "prefill_step":
        runner = ModelRunner(None, dtype="bfloat16", max_tokens=a.tokens + 4096, page_size=a.page_size, max_requests=4,
                             max_context=a.tokens + 64, config=dict(shape))
        for i in range(a.steps):
            rc = runner.open(i)
            toks = rng.integers(0, vocab, a.tokens).tolist()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            runner.step([StepEntry(rc, toks, [a.tokens - 1])])
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            runner.close(rc)
            print(f"prefill_step tokens={a.tokens}: {dt * 1e3:.2f} ms, {a.tokens / dt:.0f} tok/s", flush=True)
        return 0
    # mixed_step: decoding rows first, one portion of a prompt after them, as the scheduler lays a step out
    ctx_max = a.context + a.tokens * (a.steps + 4) + 64
    runner = ModelRunner(None, dtype="bfloat16", max_tokens=a.batch * (a.context + 256) + ctx_max, page_size=a.page_size,
                         max_requests=a.batch + 1, max_context=ctx_max, config=dict(shape))
    rows = [runner.open(i) for i in range(a.batch)]
    for rc in rows:
        runner.synthetic_fill(rc, a.context)
    portion = runner.open("portion")
    runner.synthetic_fill(portion, a.context // 4)

    def step():
        return runner.step([StepEntry(rc, [5], [0]) for rc in rows] +
                           [StepEntry(portion, rng.integers(0, vocab, a.tokens).tolist(), [a.tokens - 1])])
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        step()
    torch.cuda.synchronize()
    print(f"mixed_step {a.batch} decoding rows at {a.context} + a {a.tokens}-token portion: "
          f"{(time.perf_counter() - t0) / a.steps * 1e3:.2f} ms a step")
    return 0


def product_phases(a, shape) -> int:
    """One decode step with the products' time stamps on (tuff_gemm_stream_trace up to 8 rows,
    tuff_gemm_skinny_trace beyond): medians over a product's CTAs, microseconds from the CTAs' first start."""
    import ctypes

    import numpy as np

    from ..engine.engine import Engine
    from ..engine.scheduler import RequestStatus
    from ..sampling import SamplingParams
    from .build import load_library
    rng = np.random.default_rng(0)
    n_new = 40
    eng = Engine(None, dtype="bfloat16", ctx_size=a.context, max_tokens=a.batch * a.context + 4096, page_size=a.page_size,
                 max_running=a.batch, config=dict(shape), cuda_graphs=True, run_ahead=False)
    for i in range(a.batch):
        r = eng.scheduler.add(i, rng.integers(0, shape["vocab_size"], a.context - n_new).tolist(), SamplingParams(max_new_tokens=n_new))
        eng.scheduler.waiting.remove(r)
        r.cache = eng.runner.open(i)
        eng.runner.synthetic_fill(r.cache, a.context - n_new - 1)
        r.status = RequestStatus.RUNNING
        eng.scheduler.running.append(r)
    stream_kernel = a.batch <= ops.SKINNY_MAX_TOKENS
    lib = load_library("gemm_stream" if stream_kernel else "gemm_skinny")
    set_trace = lib.tuff_gemm_stream_trace if stream_kernel else lib.tuff_gemm_skinny_trace
    n = 256
    buf = torch.zeros(n * 256 * 8, dtype=torch.int64, device="cuda")
    eng.step()                                                    # the last prompt tokens, plain launches
    set_trace(ctypes.c_void_p(buf.data_ptr()), ctypes.c_int(n))
    eng.step()                                                    # captured with the stamps on, and replayed once
    set_trace(ctypes.c_void_p(0), ctypes.c_int(0))
    torch.cuda.synchronize()
    t = buf.cpu().numpy().reshape(n, 256, 8).astype(np.float64)
    # stamps: the stream kernel 0 start, 6 ring filled, 1 predecessor done, 2 activations ready, 3 first stage, 4 sums, 5 written;
    # the cluster kernel 0 start, 1 set up, 2 predecessor done, 3 first stage, 4 sums, 5 rows exchanged, 6 written
    cols = ([("primed", 6), ("pred.done", 1), ("acts", 2), ("1st stage", 3), ("sums", 4), ("written", 5)] if stream_kernel else
            [("set up", 1), ("pred.done", 2), ("1st stage", 3), ("sums", 4), ("exchanged", 5), ("written", 6)])
    print(f"product_phases batch={a.batch} context={a.context}: us after the product's first CTA started (medians over CTAs)")
    print("  #  CTAs   start  " + "".join(f"{c:>10s}" for c, _ in cols) + "       end   since prev. end")
    t0 = prev = None
    for i in range(n):
        m = t[i][:, 0] > 0
        if not m.any():
            break
        r = t[i][m]
        if t0 is None:
            t0 = r[:, 0].min()
        r = (r - t0) / 1e3
        st = r[:, 0].min()
        last = cols[-1][1]
        end = r[:, last].max()
        print(f"{i:3d} {int(m.sum()):5d} {st:8.2f}  " + "".join(f"{np.median(r[:, k]) - st:10.2f}" for _, k in cols) +
              f" {end:9.2f} {'' if prev is None else f'{end - prev:9.2f}'}")
        prev = end
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm_tc", "gemm_decode", "gemm_cluster", "decode_chain", "attention_decode", "attention_prefill",
                                       "decode_step", "prefill_step", "mixed_step", "product_phases"])
    ap.add_argument("--config", help="*_step: a config.json with the sizes of the model")
    ap.add_argument("--layers", type=int, default=16, help="decode_chain: layers of four products each")
    ap.add_argument("--ffn", type=int, default=5632, help="decode_chain: width of the feed-forward")
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--no-graphs", action="store_true", help="decode_step: plain launches instead of CUDA graph replays")
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=11264)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--epilogue", choices=["store", "accum", "swiglu", "conv"], default="store")
    ap.add_argument("--norm", action="store_true", help="gemm_decode: RMSNorm of fp32 rows as the prologue")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warm-l2", action="store_true", help="do not flush L2 between timed launches")
    ap.add_argument("--shuffle-pages", action="store_true", help="attention: a request's pages lie scattered over the pool")
    a = ap.parse_args(argv)
    FLUSH_L2[0] = not a.warm_l2
    torch.manual_seed(0)
    dev = "cuda"
    bf = torch.bfloat16
    if a.kernel.endswith("_step") or a.kernel == "product_phases":
        return run_steps(a)

    if a.kernel == "gemm_tc":
        x = torch.randn(a.m, a.k, device=dev).to(bf)
        w = (torch.randn(a.n, a.k, device=dev) * 0.02).to(bf)
        if a.epilogue == "swiglu":
            out = torch.empty(a.m, a.n // 2, dtype=bf, device=dev)
            fn = lambda: ops.gemm_tc(x, w, out, swiglu=True)
        elif a.epilogue == "accum":
            out = torch.zeros(a.m, a.n, device=dev)
            fn = lambda: ops.gemm_tc(x, w, out, accumulate=True)
        else:
            out = torch.empty(a.m, a.n, dtype=bf, device=dev)
            fn = lambda: ops.gemm_tc(x, w, out)
        t = timed(fn, a.reps)
        flops = 2.0 * a.m * a.n * a.k
        print(f"gemm_tc m={a.m} n={a.n} k={a.k} {a.epilogue}: {t * 1e6:.1f} us, {flops / t / 1e12:.1f} TFLOP/s, "
              f"{(a.n * a.k * 2 + a.m * a.k * 2) / t / 1e9:.0f} GB/s of operands")
    elif a.kernel == "gemm_decode":
        epi = {"store": ops.EPI_STORE, "accum": ops.EPI_ACCUM, "swiglu": ops.EPI_SWIGLU, "conv": ops.EPI_CONV}[a.epilogue]
        mult = {"swiglu": 2, "conv": 3}.get(a.epilogue, 1)
        w = (torch.randn(mult * a.n, a.k, device=dev) * 0.02).to(bf)
        if a.norm:
            x = ops.NormedRows(torch.randn(a.m, a.k, device=dev), torch.ones(a.k, device=dev), 1e-5, bf)
        else:
            x = torch.randn(a.m, a.k, device=dev).to(bf)
        out = torch.zeros(a.m, a.n, dtype=torch.float32 if a.epilogue == "accum" else bf, device=dev)
        conv = None
        if a.epilogue == "conv":
            conv = (torch.randn(a.n, 3, device=dev), torch.zeros(a.m, 2, a.n, device=dev),
                    torch.arange(a.m, dtype=torch.int32, device=dev))
        fn = lambda: ops.gemm_decode(x, w, out, epi, conv=conv)
        t = timed(fn, a.reps)
        nbytes = mult * a.n * a.k * 2
        print(f"gemm_decode m={a.m} n={a.n} k={a.k} {a.epilogue}{' +norm' if a.norm else ''}: {t * 1e6:.1f} us, "
              f"{nbytes / t / 1e9:.0f} GB/s of weights ({nbytes / 1e6:.1f} MB)")
    elif a.kernel == "gemm_cluster":
        epi = {"store": ops.EPI_STORE, "accum": ops.EPI_ACCUM, "swiglu": ops.EPI_SWIGLU}[a.epilogue]
        mult = 2 if a.epilogue == "swiglu" else 1
        w = (torch.randn(mult * a.n, a.k, device=dev) * 0.02).to(bf)
        x = torch.randn(a.m, a.k, device=dev).to(bf)
        out = torch.zeros(a.m, a.n, dtype=torch.float32 if a.epilogue == "accum" else bf, device=dev)
        if not ops._cluster_eligible(x, w, out, epi):
            print("gemm_cluster: the cluster product does not take these sizes", file=sys.stderr)
            return 2
        t = timed(lambda: ops.gemm_cluster(x, w, out, epi), a.reps)
        nbytes = mult * a.n * a.k * 2
        print(f"gemm_cluster m={a.m} n={a.n} k={a.k} {a.epilogue}: {t * 1e6:.1f} us, "
              f"{nbytes / t / 1e9:.0f} GB/s of weights ({nbytes / 1e6:.1f} MB), {ops._cluster_plan(a.m, mult * a.n, a.k, epi)} CTAs")
    elif a.kernel == "decode_chain":
        # The products of `layers` short-convolution layers back to back, each with weights of its own
        # (nothing is found in L2 again), replayed from one CUDA graph: what the decode step's products
        # cost when they follow one another, per product and as bytes over time.
        d, F, M = a.k, a.ffn, a.m
        x = torch.randn(M, d, device=dev) * 0.1
        nw = torch.ones(d, device=dev)
        layers = []
        for _ in range(a.layers):
            layers.append(dict(w_in=(torch.randn(3 * d, d, device=dev) * 0.02).to(bf), w_out=(torch.randn(d, d, device=dev) * 0.02).to(bf),
                               w13=ops.stack_gate_up((torch.randn(F, d, device=dev) * 0.02).to(bf), (torch.randn(F, d, device=dev) * 0.02).to(bf)), w2=(torch.randn(d, F, device=dev) * 0.02).to(bf),
                               taps=torch.randn(d, 3, device=dev) * 0.1, state=torch.zeros(M, 2, d, device=dev)))
        slots = torch.arange(M, dtype=torch.int32, device=dev)
        g = torch.empty(M, d, dtype=bf, device=dev)
        act = torch.empty(M, F, dtype=bf, device=dev)

        def chain():
            for L in layers:
                ops.gemm_decode(ops.NormedRows(x, nw, 1e-5, bf), L["w_in"], g, ops.EPI_CONV, conv=(L["taps"], L["state"], slots))
                ops.gemm_decode(g, L["w_out"], x, ops.EPI_ACCUM)
                ops.gemm_decode(ops.NormedRows(x, nw, 1e-5, bf), L["w13"][0], act, ops.EPI_SWIGLU, set_block=L["w13"][1])
                ops.gemm_decode(act, L["w2"], x, ops.EPI_ACCUM)
        chain()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            chain()
        t = timed(graph.replay, a.reps)
        nbytes = a.layers * (3 * d * d + d * d + 3 * d * F) * 2
        print(f"decode_chain m={M} d={d} ffn={F} layers={a.layers}: {t * 1e6:.1f} us for {4 * a.layers} products, "
              f"{t * 1e6 / (4 * a.layers):.2f} us a product, {nbytes / t / 1e9:.0f} GB/s of weights ({nbytes / 1e6:.0f} MB)")
    else:
        H, G, hd, ps = a.heads, a.kv_heads, a.head_dim, a.page_size
        if a.kernel == "attention_decode":
            rows, q_len, ctx_len = a.batch, 1, a.context
        else:
            rows, q_len, ctx_len = 1, a.tokens, a.tokens
        blocks = math.ceil(ctx_len / ps)
        n_pages = rows * blocks
        kp = (torch.randn(n_pages, G, ps, hd, device=dev) * 0.5).to(bf)
        vp = (torch.randn(n_pages, G, ps, hd, device=dev) * 0.5).to(bf)
        order = torch.randperm(n_pages, device=dev) if a.shuffle_pages else torch.arange(n_pages, device=dev)
        table = order.to(torch.int32).view(rows, blocks).contiguous()
        T = rows * q_len
        q = torch.randn(T, H * hd, device=dev).to(bf)
        out = torch.empty(T, H * hd, dtype=bf, device=dev)
        row_of = torch.arange(rows, dtype=torch.int32, device=dev).repeat_interleave(q_len)
        if a.kernel == "attention_decode":
            pos = torch.full((T,), ctx_len - 1, dtype=torch.int32, device=dev)
            fn = lambda: ops.attention_decode(q, kp, vp, table, pos, row_of, out, H, G, hd, hd ** -0.5, 0, ctx_len)
            t = timed(fn, a.reps)
            nbytes = 2 * rows * ctx_len * G * hd * 2
            print(f"attention_decode batch={rows} context={ctx_len} H={H} G={G} hd={hd} page={ps}: {t * 1e6:.1f} us, "
                  f"{nbytes / t / 1e9:.0f} GB/s of keys and values ({nbytes / 1e6:.1f} MB)")
        else:
            pos = torch.arange(q_len, dtype=torch.int32, device=dev)
            cu = torch.tensor([0, q_len], dtype=torch.int32, device=dev)
            # the tcgen05 kernel where it applies (TUFF_ATTN_TC=0: the mma.sync one)
            fn = lambda: ops.paged_attention(q, kp, vp, table, pos, row_of, out, H, G, hd, hd ** -0.5, 0, cu_q=cu,
                                             all_single=False, max_seq_len=ctx_len)
            t = timed(fn, a.reps)
            flops = 2.0 * 2.0 * H * hd * q_len * (q_len + 1) / 2
            print(f"attention_prefill tokens={q_len} H={H} G={G} hd={hd} page={ps}: {t * 1e6:.1f} us, "
                  f"{flops / t / 1e12:.1f} TFLOP/s (causal)")
    ops.check_tc_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
