"""Builders of replay traces for the tests: the same requests cut into steps in
different ways.  Each builder returns (steps, wanted) where `steps` are the JSON
records for bin/trace_run and `wanted[step]` lists (request id, position) for
every logits row that step writes."""
import numpy as np


def _finish(steps):
    wanted = {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            rows += [(e["id"], e["_pos0"] + w) for w in e["want"]]
        if rows:
            wanted[s["step"]] = rows
    clean = [dict(step=s["step"], entries=[{k: v for k, v in e.items() if k != "_pos0"} for e in s["entries"]],
                  end=s["end"]) for s in steps]
    return clean, wanted


def whole(requests):
    """Each request alone, whole, in one step; all logits wanted."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append(dict(step=i, entries=[dict(id=rid, tokens=list(toks), want=list(range(len(toks))), _pos0=0)],
                          end=[rid]))
    return _finish(steps)


def tail_decoded(requests, tail=32):
    """Most of a request in one step, its last `tail` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = len(toks) - tail
        assert head >= 1
        steps.append(dict(step=n, entries=[dict(id=rid, tokens=list(toks[:head]), want=[head - 1], _pos0=0)], end=[]))
        n += 1
        for p in range(head, len(toks)):
            steps.append(dict(step=n, entries=[dict(id=rid, tokens=[toks[p]], want=[0], _pos0=p)],
                              end=[rid] if p == len(toks) - 1 else []))
            n += 1
    return _finish(steps)


def portions(requests, sizes=(5, 2, 7, 3, 2, 16, 2, 9, 1, 4, 2, 33)):
    """Each request alone in portions of changing size, down to two tokens (and one)."""
    steps, n = [], 0
    for rid, toks in requests.items():
        p, k = 0, 0
        while p < len(toks):
            m = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append(dict(step=n, entries=[dict(id=rid, tokens=list(toks[p:p + m]), want=list(range(m)), _pos0=p)],
                              end=[rid] if p + m == len(toks) else []))
            p += m
            n += 1
    return _finish(steps)


def mixed(requests, seed=0, max_live=4, decode_tail=12):
    """Up to `max_live` requests at a time: every step takes, for each live request, either a
    portion of its prompt (2..11 tokens) or, within its last `decode_tail` tokens, one token;
    a request is sometimes left out of a step.  New requests join as others end."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live, steps, n = {}, [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            rid, toks = waiting.pop(0)
            live[rid] = [list(toks), 0]
        entries, ends = [], []
        for rid, (toks, p) in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # sits this step out
            left = len(toks) - p
            m = 1 if left <= decode_tail else int(min(left - decode_tail, rng.integers(2, 12)))
            want = list(range(m)) if rng.random() < 0.7 or m == 1 else [m - 1]
            entries.append(dict(id=rid, tokens=toks[p:p + m], want=want, _pos0=p))
            live[rid][1] = p + m
            if p + m == len(toks):
                ends.append(rid)
                del live[rid]
        if entries:
            steps.append(dict(step=n, entries=entries, end=ends))
            n += 1
    return _finish(steps)


def tokens_needed(steps, round_to=64):
    """The --max-tokens a trace needs: the most tokens live requests hold at any time, each
    request's count rounded up to a multiple of `round_to`."""
    held, most = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum((v + round_to - 1) // round_to * round_to for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most
