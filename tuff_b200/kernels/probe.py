"""Runs one kernel alone on synthetic data and times it: the command that the summaries under
`profiles/` were made with, and a quick check of a kernel's bandwidth or throughput.

    python -m tuff_b200.kernels.probe gemm_tc --m 2048 --n 11264 --k 2048
    python -m tuff_b200.kernels.probe gemm_decode --m 8 --n 5632 --k 2048 --epilogue swiglu --norm
    python -m tuff_b200.kernels.probe attention_decode --batch 8 --context 8192
    python -m tuff_b200.kernels.probe attention_prefill --tokens 2048

Timing: CUDA events around each launch, after warm-up, with a buffer larger than L2 written
between launches.  Prints the median time and the achieved rate against the bytes or flops the
kernel has to move or do.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import ops


def timed(fn, reps: int, warmup: int = 3):
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm_tc", "gemm_decode", "attention_decode", "attention_prefill"])
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
    ap.add_argument("--shuffle-pages", action="store_true", help="attention: a request's pages lie scattered over the pool")
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    dev = "cuda"
    bf = torch.bfloat16

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
