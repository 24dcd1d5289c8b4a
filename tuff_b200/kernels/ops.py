"""Python faces of the CUDA kernels: each function checks its tensors, then calls
the `extern "C"` launcher of the same name on the current CUDA stream.

Nothing here computes on the host or through a library: a tensor that is not on
a CUDA device is refused, and a launcher that cannot be compiled or loaded
raises (`tuff_b200.kernels.build.KernelBuildError`).
"""
from __future__ import annotations

import os
import struct
import weakref
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load_library

F32, BF16 = 0, 1
_ERRORS = {-2: "unsupported combination of element types", -3: "a size outside what the kernel supports",
           -4: "a pointer or stride that breaks an alignment rule", -5: "scratch memory too small"}


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"tensors must be float32 or bfloat16, found {t.dtype}")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("tuff_b200 kernels run on CUDA tensors only; there is no host path")
    return c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current CUDA stream of the current device as a raw handle (the fast path skips the
    construction of a torch.cuda.Stream object, which costs more than the launch itself)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = {"n": 0}      # kernels launched through this module (a captured graph replays its share)


def _check(status: int, what: str, kernels: int = 1) -> None:
    if status == 0:
        LAUNCHES["n"] += kernels
        return
    if status in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[status]}")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _i32(t: torch.Tensor | None, name: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, found {t.dtype}")


# ----------------------------------------------------------------- elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = table[tokens[t], :] as float32."""
    _written(out)
    _i32(tokens, "tokens")
    n, d = out.shape
    assert out.dtype == torch.float32 and table.shape[1] == d and tokens.numel() == n
    _contig(table, "table"); _contig(out, "out")
    lib = load_library("elementwise")
    _check(lib.tuff_embed(_ptr(tokens), _ptr(table), dtype_code(table), _ptr(out), c_int(n), c_int(d),
                          c_int(table.shape[0]), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            row_index: torch.Tensor | None = None) -> None:
    """out[r] = x[row_index[r] or r] * rsqrt(mean(x^2) + eps) * weight."""
    _written(out)
    d = x.shape[-1]
    n = out.shape[0]
    assert weight.dtype == torch.float32 and weight.numel() == d and out.shape[-1] == d
    _contig(x, "x"); _contig(out, "out"); _i32(row_index, "row_index")
    lib = load_library("elementwise")
    _check(lib.tuff_rmsnorm(_ptr(x), dtype_code(x), _ptr(weight), _ptr(out), dtype_code(out), _ptr(row_index),
                            c_int(n), c_int(d), c_float(eps), _stream()), "rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out = silu(gate) * up.  gate_up [n, 2F] holds, per `block` outputs, block gate columns then
    block up columns; block = 0 means all F gate columns, then all F up columns."""
    _written(out)
    n, F = out.shape
    assert gate_up.shape == (n, 2 * F) and gate_up.dtype == out.dtype
    _contig(gate_up, "gate_up"); _contig(out, "out")
    lib = load_library("elementwise")
    _check(lib.tuff_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out), c_int(n), c_int(F), c_int(block), _stream()),
           "swiglu")


def stack_gate_up(w1: torch.Tensor, w3: torch.Tensor, block: int = 128):
    """[gate; up] as one matrix for `linear_swiglu`: returns (w13, block).  When the width is a multiple
    of `block`, the rows are laid out as `block` gate rows followed by their `block` up rows, and so on,
    so that a 256-wide tile of the product holds matching gate and up columns; else they are stacked
    whole (block 0)."""
    F, K = w1.shape
    if F % block == 0:
        w13 = torch.stack([w1.view(F // block, block, K), w3.view(F // block, block, K)], dim=1).reshape(2 * F, K)
        return w13.contiguous(), block
    return torch.cat([w1, w3], dim=0).contiguous(), 0


def cast(src: torch.Tensor, out: torch.Tensor) -> None:
    assert src.numel() == out.numel()
    _written(out)
    _contig(src, "src"); _contig(out, "out")
    lib = load_library("elementwise")
    _check(lib.tuff_cast(_ptr(src), dtype_code(src), _ptr(out), dtype_code(out), c_longlong(src.numel()), _stream()),
           "cast")


# ------------------------------------------------------------------------ GEMM
def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (=|+=) a @ w.T with fp32 FFMA accumulation; a [M,K], w [N,K], out [M,N]."""
    _written(out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    lib = load_library("gemm_plain")
    _check(lib.tuff_gemm_plain(_ptr(a), dtype_code(a), _ptr(w), dtype_code(w), _ptr(out), dtype_code(out),
                               c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)), c_longlong(w.stride(0)),
                               c_longlong(out.stride(0)), c_int(1 if accumulate else 0), _stream()), "gemm_plain")


_tc_state: dict = {}


def _grow(st: dict, n_floats: int, what: str) -> None:
    """Makes st["ws"] hold at least n_floats.  A workspace that is replaced stays alive (st["retired"]):
    a CUDA graph captured earlier has its address in its kernels' arguments and goes on writing
    there when it is replayed.  Sizes at least double, so all retired ones together stay smaller
    than the current one."""
    if st["ws"] is not None and st["ws"].numel() >= n_floats:
        return
    if torch.cuda.is_current_stream_capturing():
        raise KernelError(f"the {what} workspace would have to grow inside a CUDA graph capture; "
                          "run the step once before capturing it, or reserve it (ops.reserve_workspaces)")
    if st["ws"] is not None:
        st.setdefault("retired", []).append(st["ws"])
        n_floats = max(n_floats, 2 * st["ws"].numel())
    st["ws"] = torch.empty(n_floats, dtype=torch.float32, device=st["device"])


def _tc_buffers(device: torch.device, need_bytes: int):
    """The tensor-core product's device status word and split-K workspace (grown on demand)."""
    st = _tc_state.get(device)
    if st is None:
        st = _tc_state[device] = {"status": torch.zeros(1, dtype=torch.int32, device=device), "ws": None, "device": device}
    if need_bytes:
        _grow(st, (need_bytes + 3) // 4, "split-K")
    return st


def tc_status(device=None) -> int:
    """The status word of the tensor-core kernels (synchronises); non-zero means a bounded wait
    ran out: in the tensor-core product 1 producer, 2 MMA issuer, 3 epilogue, 4 accumulator hand-back;
    in the decode product 61 producer, 63 consumers; in the cluster product 51 producer, 52 MMA issuer, 53 epilogue; in attention 11/12 decode producer/consumer, 21/22 prompt
    portions on mma.sync producer/consumer; in the tcgen05 attention 31 producer, 32-36 MMA issuer
    (query, keys, score buffer, P, -), 37-41 softmax warps (scores, last tile's values, O before a
    rescale, P buffer, final O).  A build with TUFF_DEBUG_BOUNDS=1 also leaves 71 (a position beyond a
    block table's width), 72 (a page id outside the pool), 73 (a state slot outside the slots) or 74 (a batch
    row outside the table) where a kernel was given such an index, and skips the access."""
    out = 0
    for dev, st in _tc_state.items():
        if device is None or torch.device(device) == dev:
            out = out or int(st["status"].item())
    return out


def check_tc_status() -> None:
    raise_on_status(tc_status())


def raise_on_status(code: int) -> None:
    if code:
        what = "was given an index outside its range" if 71 <= code <= 74 else "gave up waiting on a barrier"
        raise KernelError(f"a kernel {what} (code {code}, see ops.tc_status); the results of the step are invalid")


def status_word(device) -> torch.Tensor:
    """The device int32 in which a kernel whose bounded wait ran out leaves its code (0: all is well).
    Read it together with a step's results, at the point where the host waits for them anyway."""
    return _tc_buffers(torch.device(device), 0)["status"]


def gemm_tc_eligible(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool) -> bool:
    K = a.shape[1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and (out.dtype == torch.float32 or not accumulate))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False, swiglu: bool = False) -> None:
    """out (=|+=) a @ w.T on the tcgen05 tensor cores (bf16 operands, fp32 accumulation).  `swiglu`:
    w is a gate/up matrix in blocks of 128 (see stack_gate_up) and out [M, F] = silu(gate) * up."""
    _written(out)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N // 2 if swiglu else N)
    if not gemm_tc_eligible(a, w, out, accumulate):
        raise KernelError("gemm_tc needs bf16 operands with K, strides and addresses aligned for TMA")
    lib = load_library("gemm_tc")
    lib.tuff_gemm_tc_workspace_bytes.restype = c_longlong
    need = lib.tuff_gemm_tc_workspace_bytes(c_int(M), c_int(N), c_int(K))
    st = _tc_buffers(a.device, need)
    ws = st["ws"]
    _check(lib.tuff_gemm_tc(_ptr(a), _ptr(w), _ptr(out), dtype_code(out), c_int(M), c_int(N), c_int(K),
                            c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                            c_int(2 if swiglu else 1 if accumulate else 0), _ptr(ws),
                            c_longlong(0 if ws is None else ws.numel() * 4),
                            _ptr(st["status"]), _stream()), "gemm_tc")


# The decode product on mma.sync (csrc/gemm_stream.cu) takes up to 8 tokens: measured against the cluster product
# it is ahead up to there (0.74 against 0.76 ms a step at 8 rows) and behind beyond (0.94 against 0.77 ms at 12).
# TUFF_STREAM_MAX_TOKENS gives it fewer (0: none).
SKINNY_MAX_TOKENS = max(0, min(8, int(os.environ.get("TUFF_STREAM_MAX_TOKENS", "8"))))
CLUSTER_MAX_TOKENS = 128         # the product that splits K over a cluster (csrc/gemm_skinny.cu): from there up to 128 tokens
FUSED_NORM_MAX_K = 2048          # the widest row the fused RMSNorm of a decode product holds in registers


# ---- a norm split over the products around it -------------------------------------------------
# A decode product that adds into the residual x can also write what the RMSNorm that follows needs
# (csrc/gemm_stream.cu, "emit"): bf16(x * weight) and sums of squares per CTA.  The product that
# consumes the norm then reads those rows and scales its result rows, and no CTA norms x itself.
# `announce_norm` says which norm will follow the next addition into x; the product that performs
# it leaves a record here; `NormedRows` picks the record up if x has not been written since
# (every op of this module that writes a tensor drops the tensor's record, and a torch in-place
# operation changes x._version).
_norm_announced: dict = {}
_norm_ready: dict = {}


def announce_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """The next product of few tokens that adds into `x` (fp32 [M, d], M <= 128) may prepare RMSNorm(x; weight, eps)."""
    if (x.dtype == torch.float32 and x.dim() == 2 and x.shape[0] <= CLUSTER_MAX_TOKENS
            and x.is_contiguous() and weight.dtype == torch.float32 and weight.numel() == x.shape[1]):
        _norm_announced[x.data_ptr()] = (weight, float(eps))


def _written(t: torch.Tensor) -> None:
    """`t` is about to be written by a kernel of this module: what was prepared from its old values is void."""
    if _norm_announced or _norm_ready:
        ptr = t.data_ptr()
        _norm_announced.pop(ptr, None)
        _norm_ready.pop(ptr, None)


def _remember(table: dict, t: torch.Tensor, rec: dict) -> None:
    """Files `rec` under tensor `t`: valid while this very tensor object lives unchanged (a new tensor may
    get the same address)."""
    if len(table) > 64:
        for k in [k for k, r in table.items() if r["ref"]() is None]:
            del table[k]
    rec["ref"], rec["version"] = weakref.ref(t), t._version
    table[t.data_ptr()] = rec


class NormedRows:
    """An RMSNorm that has not run yet: `x` (fp32 [M, d]) to be normed with `weight` and `eps` into
    `dtype`.  The decode products take it as their input and norm the rows themselves (or, when the
    product that last added into x prepared the norm, read the prepared rows: `pre`); anything
    else calls `dense()` and gets the normed tensor (computed once)."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float, dtype: torch.dtype):
        self.x, self.weight, self.eps, self.dtype = x, weight, float(eps), dtype
        self.shape, self.device = x.shape, x.device
        self._dense = None
        rec = _norm_ready.get(x.data_ptr()) if _norm_ready else None
        self.pre = rec if (rec is not None and rec["ref"]() is x and rec["weight"].data_ptr() == weight.data_ptr() and rec["eps"] == self.eps
                           and rec["shape"] == tuple(x.shape) and rec["version"] == x._version
                           and dtype == torch.bfloat16) else None

    def dense(self) -> torch.Tensor:
        if self._dense is None:
            self._dense = torch.empty(self.x.shape, dtype=self.dtype, device=self.x.device)
            rmsnorm(self.x, self.weight, self.eps, self._dense)
        return self._dense

    def fusable(self, w: torch.Tensor) -> bool:
        M, K = self.x.shape
        if self.pre is not None:
            return (w.dtype == torch.bfloat16 and M <= SKINNY_MAX_TOKENS and K % 8 == 0 and w.stride(0) % 8 == 0
                    and w.stride(1) == 1 and w.data_ptr() % 16 == 0 and self.pre["part"].shape[1] == 16)
        return (self.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= SKINNY_MAX_TOKENS
                and K % 8 == 0 and K <= FUSED_NORM_MAX_K and w.stride(0) % 8 == 0 and w.stride(1) == 1
                and w.data_ptr() % 16 == 0 and self.x.is_contiguous() and self.x.data_ptr() % 16 == 0)


EPI_STORE, EPI_ACCUM, EPI_SWIGLU, EPI_CONV = 0, 1, 2, 3


def gemm_decode(a, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE, conv=None, set_block: int = 0) -> None:
    """A decode-step product for at most 8 tokens with its neighbours fused in (csrc/gemm_stream.cu):
    `a` is a bf16 tensor [M, K] or a `NormedRows`; epilogue EPI_SWIGLU takes w = [gate; up] stacked,
    EPI_CONV takes w = [B; C; x] stacked and conv = (taps [d, L], state [slots, L-1, d], slot_of_row)."""
    norm = a if isinstance(a, NormedRows) else None
    pre = norm.pre if norm is not None else None
    if pre is not None:
        src, norm = pre["xw"], None            # the rows times the norm weight; 1/rms is applied to the result rows
    else:
        src = norm.x if norm is not None else a
    M, K = src.shape
    N = out.shape[1]
    mult = {EPI_SWIGLU: 2, EPI_CONV: 3}.get(epilogue, 1)
    assert w.shape == (mult * N, K) and out.shape[0] == M and M <= SKINNY_MAX_TOKENS
    taps = state = slots = None
    L = 0
    if epilogue == EPI_CONV:
        taps, state, slots = conv
        L = taps.shape[1]
        assert taps.shape == (N, L) and state.shape[1:] == (L - 1, N) and taps.dtype == state.dtype == torch.float32
        _i32(slots, "slot_of_row"); _contig(state, "state"); _contig(taps, "taps")
    lib = load_library("gemm_stream")
    st = _tc_buffers(src.device, 0)
    ann = _norm_announced.pop(out.data_ptr(), None) if (epilogue == EPI_ACCUM and _norm_announced) else None
    _written(out)
    emit_w = emit_xw = emit_part = None
    if ann is not None and out.is_contiguous() and tuple(out.shape) == (M, N):
        emit_w = ann[0]
        emit_xw = torch.empty((M, N), dtype=torch.bfloat16, device=out.device)
        emit_part = torch.empty((lib.tuff_gemm_stream_grid(c_int(N)), 16), dtype=torch.float32, device=out.device)
    _check(lib.tuff_gemm_stream(_ptr(src), _ptr(norm.weight if norm is not None else None),
                                c_float(norm.eps if norm is not None else 0.0), _ptr(w), _ptr(out), dtype_code(out),
                                c_int(M), c_int(N), c_int(K), c_longlong(src.stride(0)), c_longlong(w.stride(0)),
                                c_longlong(out.stride(0)), c_int(epilogue), _ptr(taps), _ptr(state), _ptr(slots),
                                c_longlong(state.shape[0] if state is not None else 0), c_int(L), c_int(set_block), _ptr(emit_w), _ptr(emit_xw), _ptr(emit_part),
                                _ptr(pre["part"] if pre is not None else None),
                                c_int(pre["part"].shape[0] if pre is not None else 0),
                                c_float(pre["eps"] if pre is not None else 0.0),
                                _ptr(st["status"]), _stream()), "gemm_stream")
    if emit_w is not None:
        _remember(_norm_ready, out, dict(weight=ann[0], eps=ann[1], xw=emit_xw, part=emit_part, shape=(M, N)))


_cluster_ctas: dict = {}


def _cluster_plan(M: int, w_rows: int, K: int, epilogue: int) -> int:
    """CTAs that the cluster product uses for these sizes; 0: it does not take them."""
    key = (M, w_rows, K, epilogue)
    n = _cluster_ctas.get(key)
    if n is None:
        lib = load_library("gemm_skinny")
        n = _cluster_ctas[key] = int(lib.tuff_gemm_skinny_ctas(c_int(M), c_int(w_rows), c_int(K), c_int(epilogue)))
    return n


def _cluster_eligible(a, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> bool:
    M = a.shape[0]
    if not (SKINNY_MAX_TOKENS < M <= CLUSTER_MAX_TOKENS) or os.environ.get("TUFF_GEMM_CLUSTER", "1") == "0":
        return False
    if isinstance(a, NormedRows):
        if a.dtype != torch.bfloat16:
            return False
        K, a_ok = a.shape[1], True
    else:
        K = a.shape[1]
        a_ok = a.dtype == torch.bfloat16 and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
    return (a_ok and w.dtype == torch.bfloat16 and K % 8 == 0 and w.stride(0) % 8 == 0 and w.stride(1) == 1
            and w.data_ptr() % 16 == 0 and out.stride(1) == 1
            and (out.dtype == torch.float32 if epilogue == EPI_ACCUM else out.dtype in (torch.bfloat16, torch.float32))
            and _cluster_plan(M, w.shape[0], K, epilogue) > 0)


def gemm_cluster(a, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """A product for 9 to 128 tokens with its neighbours fused in (csrc/gemm_skinny.cu): the K range of
    every 128-column tile is split over a thread-block cluster and added in distributed shared memory.
    `a` is a bf16 tensor [M, K] or a `NormedRows`; EPI_SWIGLU takes w = gate and up rows in blocks of 128."""
    pre = None
    if isinstance(a, NormedRows):
        pre = a.pre
        src = pre["xw"] if pre is not None else a.dense()
    else:
        src = a
    M, K = src.shape
    w_rows = w.shape[0]
    n_out = w_rows // 2 if epilogue == EPI_SWIGLU else w_rows
    assert w.shape[1] == K and out.shape == (M, n_out)
    lib = load_library("gemm_skinny")
    st = _tc_buffers(src.device, 0)
    ann = _norm_announced.pop(out.data_ptr(), None) if (epilogue == EPI_ACCUM and _norm_announced) else None
    _written(out)
    emit_w = emit_xw = emit_part = None
    if ann is not None and out.is_contiguous():
        emit_w = ann[0]
        emit_xw = torch.empty((M, n_out), dtype=torch.bfloat16, device=out.device)
        emit_part = torch.empty((_cluster_plan(M, w_rows, K, epilogue), M), dtype=torch.float32, device=out.device)
    part = pre["part"] if pre is not None else None
    _check(lib.tuff_gemm_skinny(_ptr(src), _ptr(w), _ptr(out), dtype_code(out), c_int(M), c_int(w_rows), c_int(K),
                                c_longlong(src.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                c_int(epilogue), _ptr(emit_w), _ptr(emit_xw), _ptr(emit_part),
                                c_int(emit_part.shape[1] if emit_part is not None else 0), _ptr(part),
                                c_int(part.shape[0] if part is not None else 0),
                                c_int(part.shape[1] if part is not None else 0),
                                c_float(pre["eps"] if pre is not None else 0.0), _ptr(st["status"]), _stream()),
           "gemm_skinny")
    if emit_w is not None:
        _remember(_norm_ready, out, dict(weight=ann[0], eps=ann[1], xw=emit_xw, part=emit_part, shape=(M, n_out)))


def _decode_eligible(a, w: torch.Tensor, out: torch.Tensor, accumulate: bool) -> bool:
    if isinstance(a, NormedRows):
        return a.fusable(w) and out.stride(1) == 1 and (out.dtype == torch.float32 or not accumulate)
    return a.shape[0] <= SKINNY_MAX_TOKENS and gemm_tc_eligible(a, w, out, accumulate)


def linear_swiglu(a, w13: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out = silu(a @ w1.T) * (a @ w3.T) for (w13, block) = stack_gate_up(w1, w3); `a` may be a
    NormedRows.  Few tokens: the decode product with the activation as its epilogue; many tokens and
    the blocked layout: the tensor-core product with the activation as its epilogue; else the product,
    then the activation kernel."""
    M, F = out.shape
    if out.dtype == torch.bfloat16 and _decode_eligible(a, w13, out, False):
        gemm_decode(a, w13, out, EPI_SWIGLU, set_block=block)
        return
    if block == 128 and out.dtype == torch.bfloat16 and _cluster_eligible(a, w13, out, EPI_SWIGLU):
        gemm_cluster(a, w13, out, EPI_SWIGLU)
        return
    if isinstance(a, NormedRows):
        a = a.dense()
    if (block == 128 and M > 128 and out.dtype == torch.bfloat16 and gemm_tc_eligible(a, w13, out, False)
            and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0):
        gemm_tc(a, w13, out, swiglu=True)
        return
    gu = torch.empty((M, 2 * F), dtype=a.dtype, device=a.device)
    linear(a, w13, gu)
    swiglu(gu, out, block)


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (=|+=) a @ w.T, by the kernel that suits the element types and the shape:
    bf16 operands that meet TMA's alignment rules go to the tensor cores, everything else
    (the 32-bit path, odd sizes) to the plain FFMA kernel.  A bf16 activation against a
    matrix stored in 32-bit is raised to fp32 first.  `a` may be a NormedRows (an RMSNorm still to
    run): the decode product norms the rows itself, every other kernel gets the normed tensor."""
    if _decode_eligible(a, w, out, accumulate):
        gemm_decode(a, w, out, EPI_ACCUM if accumulate else EPI_STORE)
        return
    if _cluster_eligible(a, w, out, EPI_ACCUM if accumulate else EPI_STORE):
        gemm_cluster(a, w, out, EPI_ACCUM if accumulate else EPI_STORE)
        return
    if isinstance(a, NormedRows):
        a = a.dense()
    if a.dtype == torch.bfloat16 and w.dtype == torch.float32:
        a32 = torch.empty(a.shape, dtype=torch.float32, device=a.device)
        cast(a.contiguous(), a32)
        if out.dtype == torch.float32:
            gemm_plain(a32, w, out, accumulate)
        else:
            tmp = torch.empty(out.shape, dtype=torch.float32, device=a.device)
            gemm_plain(a32, w, tmp, False)
            cast(tmp, out)
        return
    if gemm_tc_eligible(a, w, out, accumulate):
        gemm_tc(a, w, out, accumulate)
    else:
        gemm_plain(a, w, out, accumulate)


def linear_shortconv(a, w_in: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, slot_of_row: torch.Tensor,
                     out: torch.Tensor) -> bool:
    """The gated short convolution of one token per row fused onto its input projection:
    out = C * conv(B * x) with [B | C | x] = a @ w_in.T, rolling each row's state.  Returns False
    (and does nothing) when the fused kernel does not take these tensors."""
    if out.dtype != torch.bfloat16 or not _decode_eligible(a, w_in, out, False):
        return False
    gemm_decode(a, w_in, out, EPI_CONV, conv=(taps, state, slot_of_row))
    return True


# ------------------------------------------------------------------ short conv
def shortconv(bcx: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, slot_of_row: torch.Tensor,
              row_of_token: torch.Tensor, cu_q: torch.Tensor, out: torch.Tensor, all_single: bool = False) -> None:
    """Gated short convolution of a batch of portions; rolls each row's state slot.
    `all_single`: every row brings exactly one token (one fused launch)."""
    _written(out)
    n, d = out.shape
    K = taps.shape[1]
    assert bcx.shape == (n, 3 * d) and taps.shape == (d, K) and taps.dtype == torch.float32
    assert state.dtype == torch.float32 and state.shape[1:] == (K - 1, d) and bcx.dtype == out.dtype
    for t, nm in ((slot_of_row, "slot_of_row"), (row_of_token, "row_of_token"), (cu_q, "cu_q")):
        _i32(t, nm)
    _contig(bcx, "bcx"); _contig(out, "out"); _contig(state, "state"); _contig(taps, "taps")
    n_rows = cu_q.numel() - 1
    lib = load_library("shortconv")
    _check(lib.tuff_shortconv(_ptr(bcx), _ptr(out), dtype_code(out), _ptr(taps), _ptr(state), _ptr(slot_of_row),
                              _ptr(row_of_token), _ptr(cu_q), c_int(n), c_int(n_rows), c_int(d), c_int(K),
                              c_int(1 if all_single else 0), c_longlong(state.shape[0]), _ptr(status_word(out.device)),
                              _stream()), "shortconv", kernels=1 if all_single else 2)


# ------------------------------------------------------------------- attention
def qk_norm_rope_write(qkv: torch.Tensor, q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None,
                       inv_freq: torch.Tensor | None, positions: torch.Tensor, row_of_token: torch.Tensor,
                       block_table: torch.Tensor | None, k_pages: torch.Tensor | None,
                       v_pages: torch.Tensor | None, H: int, G: int, hd: int, rot_dim: int, eps: float,
                       write_kv: bool = True) -> None:
    """Per-head RMSNorm + NeoX rotation of q and k in place; K and V stored in their pages.

    k_pages / v_pages: [num_pages, G, page_size, hd]; block_table: [rows, max_blocks] int32.
    """
    n = qkv.shape[0]
    assert qkv.shape[1] == (H + 2 * G) * hd
    _contig(qkv, "qkv"); _i32(positions, "positions"); _i32(row_of_token, "row_of_token")
    page_size, max_blocks = 1, 0
    if write_kv:
        assert k_pages is not None and v_pages is not None and block_table is not None
        assert k_pages.shape == v_pages.shape and k_pages.shape[1] == G and k_pages.shape[3] == hd
        assert k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype
        _contig(k_pages, "k_pages"); _contig(v_pages, "v_pages"); _contig(block_table, "block_table")
        _i32(block_table, "block_table")
        page_size, max_blocks = k_pages.shape[2], block_table.shape[1]
    if rot_dim:
        assert inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2
    for wv in (q_norm_w, k_norm_w):
        assert wv is None or (wv.dtype == torch.float32 and wv.numel() == hd)
    lib = load_library("attention_plain")
    _check(lib.tuff_qk_norm_rope_write(_ptr(qkv), dtype_code(qkv), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
                                       _ptr(positions), _ptr(row_of_token), _ptr(block_table), c_int(max_blocks),
                                       _ptr(k_pages), _ptr(v_pages), c_int(n), c_int(H), c_int(G), c_int(hd),
                                       c_int(rot_dim), c_int(page_size), c_float(eps), c_int(1 if write_kv else 0),
                                       c_longlong(block_table.shape[0] if write_kv else 0),
                                       c_longlong(k_pages.shape[0] if write_kv else 0), _ptr(status_word(qkv.device)),
                                       _stream()), "qk_norm_rope_write")


def paged_attention_plain(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                          positions: torch.Tensor, row_of_token: torch.Tensor, out: torch.Tensor, H: int, G: int,
                          hd: int, scale: float, window: int = 0) -> None:
    """Causal attention of each token over its request's cached keys (the last `window` if > 0).

    q: [n, >= H*hd] (row stride taken from the tensor), out: [n, H*hd].
    """
    n = q.shape[0]
    assert q.stride(1) == 1 and out.shape == (n, H * hd) and q.dtype == k_pages.dtype == out.dtype
    _contig(out, "out"); _contig(k_pages, "k_pages"); _contig(v_pages, "v_pages"); _contig(block_table, "block_table")
    _i32(block_table, "block_table"); _i32(positions, "positions"); _i32(row_of_token, "row_of_token")
    lib = load_library("attention_plain")
    _check(lib.tuff_paged_attention_plain(_ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
                                          dtype_code(q), _ptr(block_table), c_int(block_table.shape[1]),
                                          _ptr(positions), _ptr(row_of_token), _ptr(out), c_int(n), c_int(H),
                                          c_int(G), c_int(hd), c_int(k_pages.shape[2]), c_float(scale),
                                          c_int(window), c_longlong(block_table.shape[0]), c_longlong(k_pages.shape[0]),
                                          _ptr(status_word(q.device)), _stream()), "paged_attention_plain")


_attn_state: dict = {}


def _attn_workspace(device: torch.device, n_floats: int) -> torch.Tensor | None:
    st = _attn_state.setdefault(device, {"ws": None, "device": device})
    if n_floats:
        _grow(st, n_floats, "attention")
    return st["ws"] if n_floats else None


def reserve_attention_workspace(device, max_rows: int, max_context: int, heads: int, kv_heads: int, head_dim: int) -> None:
    """Sizes the sliced decode attention's workspace once for up to `max_rows` one-token rows at contexts
    up to `max_context`, so that it keeps one address (a CUDA graph captured with it may be replayed
    after steps with other row counts have run)."""
    device = torch.device(device)
    with torch.cuda.device(device):
        lib = load_library("attention_flash")
        if not lib.tuff_attention_flash_supported(c_int(heads), c_int(kv_heads), c_int(head_dim), c_int(64)):
            return
        lib.tuff_attention_decode_workspace_floats.restype = c_longlong
        need = 0
        for n in range(1, max(1, max_rows) + 1):
            splits = lib.tuff_attention_decode_splits(c_int(n), c_int(kv_heads), c_int(max(1, max_context)))
            need = max(need, lib.tuff_attention_decode_workspace_floats(c_int(n), c_int(heads), c_int(head_dim), c_int(splits)))
        _attn_workspace(device, int(need))


def reserve_product_workspace(device, widest_out: int, widest_in: int) -> None:
    """The same for the partial sums of the tensor-core product with few tokens (17..128)."""
    device = torch.device(device)
    with torch.cuda.device(device):
        lib = load_library("gemm_tc")
        lib.tuff_gemm_tc_workspace_bytes.restype = c_longlong
        _tc_buffers(device, int(lib.tuff_gemm_tc_workspace_bytes(c_int(128), c_int(max(1, widest_out)), c_int(max(8, widest_in)))))


def attention_flash_supported(q: torch.Tensor, k_pages: torch.Tensor, H: int, G: int, hd: int) -> bool:
    if q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        return False
    lib = load_library("attention_flash")
    return bool(lib.tuff_attention_flash_supported(c_int(H), c_int(G), c_int(hd), c_int(k_pages.shape[2])))


def attention_decode(q, k_pages, v_pages, block_table, positions, row_of_token, out, H, G, hd, scale,
                     window: int = 0, max_seq_len: int | None = None) -> None:
    """Attention of a few query tokens over long cached contexts (bf16), the keys of each token cut
    into slices that run in parallel; `max_seq_len` (an upper bound on the contexts) sizes the cut."""
    n = q.shape[0]
    lib = load_library("attention_flash")
    bound = int(max_seq_len) if max_seq_len else block_table.shape[1] * k_pages.shape[2]
    splits = lib.tuff_attention_decode_splits(c_int(n), c_int(G), c_int(max(1, bound)))
    lib.tuff_attention_decode_workspace_floats.restype = c_longlong
    ws = _attn_workspace(q.device, lib.tuff_attention_decode_workspace_floats(c_int(n), c_int(H), c_int(hd), c_int(splits)))
    st = _tc_buffers(q.device, 0)
    _check(lib.tuff_attention_decode(_ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
                                     c_longlong(k_pages.shape[0]), _ptr(block_table), c_int(block_table.shape[1]),
                                     _ptr(positions), _ptr(row_of_token), _ptr(out), _ptr(ws), c_int(splits),
                                     _ptr(st["status"]), c_int(n), c_int(H), c_int(G), c_int(hd),
                                     c_int(k_pages.shape[2]), c_float(scale), c_int(window), _stream()),
           "attention_decode", kernels=2 if splits > 1 else 1)


def attention_prefill(q, k_pages, v_pages, block_table, positions, row_of_token, cu_q, out, H, G, hd, scale,
                      window: int = 0, n_tokens: int | None = None) -> None:
    """Causal attention of prompt portions (bf16): blocks of query tokens against the cached keys."""
    n = q.shape[0] if n_tokens is None else n_tokens
    lib = load_library("attention_flash")
    st = _tc_buffers(q.device, 0)
    _check(lib.tuff_attention_prefill(_ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
                                      c_longlong(k_pages.shape[0]), _ptr(block_table), c_int(block_table.shape[1]),
                                      _ptr(positions), _ptr(row_of_token), _ptr(cu_q), _ptr(out), _ptr(st["status"]),
                                      c_int(n), c_int(cu_q.numel() - 1), c_int(H), c_int(G), c_int(hd),
                                      c_int(k_pages.shape[2]), c_float(scale), c_int(window), _stream()),
           "attention_prefill")


ATTN_TC_ENABLED = os.environ.get("TUFF_ATTN_TC", "1") != "0"


def attention_prefill_tc_supported(q: torch.Tensor, k_pages: torch.Tensor, H: int, G: int, hd: int) -> bool:
    """Whether the tcgen05 kernel for prompt portions takes these sizes and this query layout."""
    if not ATTN_TC_ENABLED or q.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
        return False
    if q.data_ptr() % 16 or q.stride(0) % 8:
        return False
    lib = load_library("attention_tc")
    return bool(lib.tuff_attention_prefill_tc_supported(c_int(H), c_int(G), c_int(hd), c_int(k_pages.shape[2])))


def attention_prefill_tc(q, k_pages, v_pages, block_table, positions, cu_q, out, H, G, hd, scale,
                         window: int = 0, n_tokens: int | None = None) -> None:
    """Causal attention of prompt portions (bf16, head size 64) with tcgen05.mma: 128 query tokens
    of one head per CTA, scores and weighted values accumulated in tensor memory."""
    lib = load_library("attention_tc")
    st = _tc_buffers(q.device, 0)
    _check(lib.tuff_attention_prefill_tc(_ptr(q), c_longlong(q.stride(0)), _ptr(k_pages), _ptr(v_pages),
                                         c_longlong(k_pages.shape[0]), _ptr(block_table), c_int(block_table.shape[1]),
                                         _ptr(positions), _ptr(cu_q), _ptr(out), _ptr(st["status"]),
                                         c_int(q.shape[0] if n_tokens is None else n_tokens), c_int(cu_q.numel() - 1),
                                         c_int(H), c_int(G), c_int(hd),
                                         c_int(k_pages.shape[2]), c_float(scale), c_int(window), _stream()),
           "attention_prefill_tc")


def paged_attention(q, k_pages, v_pages, block_table, positions, row_of_token, out, H, G, hd, scale,
                    window: int = 0, ctx=None, cu_q=None, all_single: bool | None = None,
                    max_seq_len: int | None = None, single_prefix: int | None = None) -> None:
    """Attention over the paged cache by the kernel that suits the batch: the tensor-core kernels
    for bf16 with head size 64 or 128 (the sliced one for rows that bring a single token, the
    blocked ones for portions of prompts), the plain kernel for everything else.  `single_prefix`:
    how many leading rows bring exactly one token; in a batch that mixes decoding rows (first) with
    portions, each kind goes to its own kernel."""
    if ctx is not None:
        cu_q = ctx.cu_q if cu_q is None else cu_q
        all_single = ctx.all_single if all_single is None else all_single
        max_seq_len = ctx.max_seq_len if max_seq_len is None else max_seq_len
        single_prefix = ctx.single_prefix if single_prefix is None else single_prefix
    assert q.stride(1) == 1 and out.shape == (q.shape[0], H * hd) and q.dtype == k_pages.dtype == out.dtype
    n_rows = 0 if cu_q is None else cu_q.numel() - 1
    sp = int(single_prefix or 0)
    if (not all_single and cu_q is not None and 0 < sp < n_rows and attention_flash_supported(q, k_pages, H, G, hd)):
        # decoding rows first, then portions: tokens 0..sp-1 are the decoding rows' (one each)
        paged_attention(q[:sp], k_pages, v_pages, block_table[:sp], positions[:sp], row_of_token[:sp], out[:sp],
                        H, G, hd, scale, window, cu_q=None, all_single=True, max_seq_len=max_seq_len, single_prefix=0)
        # the portions keep their token numbering: q, positions and out stay whole, rows and their
        # tables are counted from the first portion
        _attention_portions(q, k_pages, v_pages, block_table[sp:], positions, row_of_token, cu_q[sp:], out,
                            H, G, hd, scale, window, n_tokens=q.shape[0] - sp)
        return
    if not all_single and cu_q is not None and attention_prefill_tc_supported(q, k_pages, H, G, hd):
        _attention_portions(q, k_pages, v_pages, block_table, positions, row_of_token, cu_q, out, H, G, hd, scale, window)
        return
    if attention_flash_supported(q, k_pages, H, G, hd):
        _contig(out, "out"); _contig(k_pages, "k_pages"); _contig(v_pages, "v_pages"); _contig(block_table, "block_table")
        _i32(block_table, "block_table"); _i32(positions, "positions"); _i32(row_of_token, "row_of_token")
        if all_single or cu_q is None:
            attention_decode(q, k_pages, v_pages, block_table, positions, row_of_token, out, H, G, hd, scale, window,
                             max_seq_len)
        else:
            _i32(cu_q, "cu_q")
            attention_prefill(q, k_pages, v_pages, block_table, positions, row_of_token, cu_q, out, H, G, hd, scale,
                              window)
        return
    paged_attention_plain(q, k_pages, v_pages, block_table, positions, row_of_token, out, H, G, hd, scale, window)


def _attention_portions(q, k_pages, v_pages, block_table, positions, row_of_token, cu_q, out, H, G, hd, scale,
                        window: int = 0, n_tokens: int | None = None) -> None:
    """Rows of several tokens through the blocked kernels: tcgen05 where it applies, else mma.sync.
    `cu_q` holds token numbers into q/positions/out as they are; `block_table` starts at the first
    of these rows; `n_tokens`: how many tokens these rows bring (for sizing the launch)."""
    _contig(out, "out"); _contig(k_pages, "k_pages"); _contig(v_pages, "v_pages"); _contig(block_table, "block_table")
    _i32(block_table, "block_table"); _i32(positions, "positions"); _i32(cu_q, "cu_q")
    if attention_prefill_tc_supported(q, k_pages, H, G, hd):
        attention_prefill_tc(q, k_pages, v_pages, block_table, positions, cu_q, out, H, G, hd, scale, window,
                             n_tokens=n_tokens)
    else:
        _i32(row_of_token, "row_of_token")
        attention_prefill(q, k_pages, v_pages, block_table, positions, row_of_token, cu_q, out, H, G, hd, scale,
                          window, n_tokens=n_tokens)


# -------------------------------------------------------------------- sampling
SAMPLE_ROW_FORMAT = "<ffffiiQQQ"     # temp, top_p, min_p, repeat_penalty, top_k, n_recent, seed, request key, token index
SAMPLE_ROW_BYTES = struct.calcsize(SAMPLE_ROW_FORMAT)


_argmax_scratch: dict = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r]."""
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == n
    _contig(logits, "logits")
    lib = load_library("sampling")
    lib.tuff_argmax_scratch_bytes.restype = c_longlong
    key = (logits.device, n)
    scratch = _argmax_scratch.get(key)
    if scratch is None and not torch.cuda.is_current_stream_capturing():
        scratch = _argmax_scratch[key] = torch.zeros(lib.tuff_argmax_scratch_bytes(c_int(n)), dtype=torch.uint8,
                                                     device=logits.device)
    _check(lib.tuff_argmax(_ptr(logits), c_int(n), c_int(V), _ptr(out), _ptr(scratch), _stream()), "argmax")


def sample(logits: torch.Tensor, rows: torch.Tensor, recent: torch.Tensor | None, work: torch.Tensor,
           out: torch.Tensor) -> None:
    """Samples one token per logits row; `rows` holds packed SAMPLE_ROW_FORMAT records (uint8 tensor)."""
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == n
    assert rows.dtype == torch.uint8 and rows.numel() == n * SAMPLE_ROW_BYTES
    assert work.dtype == torch.float32 and work.numel() >= n * V
    _contig(logits, "logits"); _i32(recent, "recent")
    lib = load_library("sampling")
    assert lib.tuff_sample_row_bytes() == SAMPLE_ROW_BYTES
    max_recent = 0 if recent is None else recent.shape[1]
    _check(lib.tuff_sample(_ptr(logits), c_int(n), c_int(V), _ptr(rows), _ptr(recent), c_int(max_recent),
                           _ptr(work), _ptr(out), _stream()), "sample")
