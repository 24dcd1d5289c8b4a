"""What one step runs: entries (a request's next tokens and the places whose
logits are wanted) flattened into the device tables that the kernels read.

The reference's step takes one token, or up to eight consecutive tokens of its
single sequence, with their first position (src/lfm25_engine.h:135-145,
src/lfm25_engine.c:496-525).  Here a step is any mix of rows, each row a
request's next `n >= 1` tokens at positions `held .. held+n-1`.

Device tables (int32), all cut from one buffer that is copied once:
  tokens[T], positions[T], row_of_token[T], cu_q[R+1] (row r owns tokens
  cu_q[r]..cu_q[r+1]-1), slot_of_row[R], want_index[W] (flat token indices whose
  logits are wanted), and per paged group a block table [R, width].
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache


@dataclass
class StepEntry:
    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among `tokens` whose logits are wanted


@dataclass
class StepContext:
    device: torch.device
    act_dtype: torch.dtype
    n_tokens: int
    n_rows: int
    n_wanted: int
    tokens: torch.Tensor
    positions: torch.Tensor
    row_of_token: torch.Tensor
    cu_q: torch.Tensor
    slot_of_row: torch.Tensor
    want_index: torch.Tensor
    block_tables: List[torch.Tensor]
    max_q_len: int = 1                 # longest row of the step
    max_seq_len: int = 1               # longest request after the step
    all_single: bool = False           # every row brings exactly one token
    single_prefix: int = 0             # how many leading rows bring exactly one token (decoding rows come first)
    wants_all_rows: bool = False       # the logits of every token are wanted, in token order
    host: Dict[str, object] = field(default_factory=dict)    # the same tables as NumPy arrays on the host
    extra: Dict[str, object] = field(default_factory=dict)   # room for parts defined elsewhere


class BatchError(ValueError):
    pass


def validate_entries(entries: Sequence[StepEntry], vocab_size: int, max_context: int | None) -> None:
    seen = set()
    if not entries:
        raise BatchError("a step needs at least one entry")
    for e in entries:
        rid = e.cache.request_id
        if id(e.cache) in seen:
            raise BatchError(f"request {rid!r} appears twice in one step")
        seen.add(id(e.cache))
        if not e.cache.open:
            raise BatchError(f"request {rid!r} is closed")
        n = len(e.tokens)
        if n < 1:
            raise BatchError(f"request {rid!r}: an entry needs at least one token")
        if n == 1:
            bad = not 0 <= int(e.tokens[0]) < vocab_size
        else:
            a = np.asarray(e.tokens, dtype=np.int64)
            bad = int(a.min()) < 0 or int(a.max()) >= vocab_size
        if bad:
            t = next(t for t in e.tokens if not 0 <= int(t) < vocab_size)
            raise BatchError(f"request {rid!r}: token {t} is outside the vocabulary (0..{vocab_size - 1})")
        for w in e.want:
            if not 0 <= int(w) < n:
                raise BatchError(f"request {rid!r}: wanted place {w} is outside its {n} token(s)")
        if max_context is not None and e.cache.n_tokens + n > max_context:
            raise BatchError(f"request {rid!r}: {e.cache.n_tokens} + {n} tokens exceed the context of {max_context}")


def layout_entries(entries: Sequence[StepEntry], cache: CacheManager, table_width: int | None = None):
    """Host arrays for a step (after the entries' pages were reserved).  `table_width` fixes the
    width of the block tables (a captured step needs the same shapes every time)."""
    R = len(entries)
    lens = [len(e.tokens) for e in entries]
    T = int(sum(lens))
    tokens = np.empty(T, np.int32)
    positions = np.empty(T, np.int32)
    row_of_token = np.empty(T, np.int32)
    cu_q = np.zeros(R + 1, np.int32)
    slot = np.empty(R, np.int32)
    want: List[int] = []
    o = 0
    for r, e in enumerate(entries):
        n = lens[r]
        tokens[o:o + n] = np.asarray(e.tokens, dtype=np.int64)
        positions[o:o + n] = np.arange(e.cache.n_tokens, e.cache.n_tokens + n)
        row_of_token[o:o + n] = r
        cu_q[r + 1] = o + n
        slot[r] = e.cache.slot
        want.extend(o + int(w) for w in e.want)
        o += n
    rcs = [e.cache for e in entries]
    tables = [cache.block_table(g, rcs, table_width) for g in range(len(cache.groups))]
    return dict(tokens=tokens, positions=positions, row_of_token=row_of_token, cu_q=cu_q, slot_of_row=slot,
                want_index=np.asarray(want, np.int32), block_tables=tables,
                max_q_len=max(lens), max_seq_len=max(e.cache.n_tokens + n for e, n in zip(entries, lens)),
                all_single=all(n == 1 for n in lens), wants_all_rows=want == list(range(T)),
                single_prefix=next((i for i, n in enumerate(lens) if n != 1), R))


def to_device(host: dict, device: torch.device, act_dtype: torch.dtype, static=None) -> StepContext:
    """Packs the host arrays into one int32 buffer, copies it once, and cuts views.  `static`
    = (pinned host buffer, device buffer) reuses fixed buffers, so that the views keep their
    addresses from step to step (a captured step reads them)."""
    parts = [host["tokens"], host["positions"], host["row_of_token"], host["cu_q"], host["slot_of_row"],
             host["want_index"]] + [t.reshape(-1) for t in host["block_tables"]]
    sizes = [p.size for p in parts]
    offs, total = [], 0
    for s in sizes:
        offs.append(total)
        total += (s + 3) // 4 * 4            # 16-byte aligned pieces
    if static is None:
        flat = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=torch.cuda.is_available())
    else:
        flat = static[0]
        assert flat.numel() >= total
        if len(static) > 2 and static[2] is not None:
            static[2].synchronize()          # the previous copy out of this buffer has been made
    flat_np = flat.numpy()
    for p, o in zip(parts, offs):
        flat_np[o:o + p.size] = p
    if static is None:
        dev = flat.to(device, non_blocking=True)
    else:
        dev = static[1]
        dev[:total].copy_(flat[:total], non_blocking=True)
        if len(static) > 2 and static[2] is not None:
            static[2].record()
    cut = [dev[o:o + s] for o, s in zip(offs, sizes)]
    R = host["cu_q"].size - 1
    tables = [c.view(R, -1) for c, t in zip(cut[6:], host["block_tables"])]
    return StepContext(device=device, act_dtype=act_dtype, n_tokens=host["tokens"].size, n_rows=R,
                       n_wanted=host["want_index"].size, tokens=cut[0], positions=cut[1], row_of_token=cut[2],
                       cu_q=cut[3], slot_of_row=cut[4], want_index=cut[5], block_tables=tables,
                       max_q_len=host["max_q_len"], max_seq_len=host["max_seq_len"],
                       all_single=host["all_single"], wants_all_rows=host["wants_all_rows"],
                       single_prefix=host.get("single_prefix", 0), host=host)
