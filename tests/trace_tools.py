"""Traces for the replay tests and the comparison with the plain implementation.

A trace is a list of step records in the format of ``bin/trace_run``.  Every
builder below wants the logits at every position of every request exactly once
over the whole trace, so that one replay can be compared with whole-sequence
logits of the plain implementation.
"""

from __future__ import annotations

import numpy as np

import plain_gpt2


def whole(requests: dict[str, list[int]]):
    """Each request alone and whole, one step each."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail_decoded(requests, tail=32):
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return _number(steps)


def portions(requests, sizes=(7, 2, 24, 3, 2, 5, 16, 2, 1, 9)):
    """Portions of changing size, down to two tokens (and one)."""
    steps, k = [], 0
    for rid, toks in requests.items():
        p = 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}], "end": []})
            p += n
        steps[-1]["end"] = [rid]
    return _number(steps)


def mixed(requests, seed=0, max_live=4, decode_after=0.6, sizes=(2, 3, 5, 8, 13, 24), live0=None):
    """Up to ``max_live`` live requests; each step takes portions of some beside
    single tokens of others; a request is sometimes left out of a step.  After
    ``decode_after`` of its tokens a request goes on one token at a time.
    ``live0``: requests that are live already, with the tokens they hold."""
    rs = np.random.RandomState(seed)
    live: dict[str, int] = dict(live0 or {})
    waiting = [(rid, toks) for rid, toks in requests.items() if rid not in live]
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rs.rand() < 0.7):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            toks = requests[rid]
            if len(live) > 1 and rs.rand() < 0.25:
                continue                                  # left out of this step
            p = live[rid]
            n = 1 if p >= decode_after * len(toks) else int(sizes[rs.randint(len(sizes))])
            n = min(n, len(toks) - p)
            entries.append({"id": rid, "tokens": toks[p:p + n], "want": list(range(n))})
            live[rid] = p + n
            if live[rid] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": ended})
    return _number(steps)


def reopened(requests, seed=0):
    """A request that is dropped mid-way and starts over, as a preempted request does: the first
    request runs 45 % of its tokens in two steps and is ended; the others start and take the pages
    it gave back; then its id is opened again from token 0 and everything runs to the end, mixed.
    Logits are wanted at every position of every life."""
    (first, toks), (second, toks2) = list(requests.items())[:2]
    n1, n2 = max(1, len(toks) // 4), max(2, int(len(toks) * 0.45))
    m1 = max(1, len(toks2) // 3)
    steps = [{"entries": [{"id": first, "tokens": toks[:n1], "want": list(range(n1))}], "end": []},
             {"entries": [{"id": first, "tokens": toks[n1:n2], "want": list(range(n2 - n1))},
                          {"id": second, "tokens": toks2[:m1], "want": list(range(m1))}], "end": [first]}]
    others = {rid: t for rid, t in requests.items() if rid != first}
    rest = list(others.items())
    # the others go on alone for a few steps: the pages that came back are handed out again
    p = m1
    for _ in range(2):
        n = min(5, len(toks2) - p)
        if n > 0:
            entries = [{"id": second, "tokens": toks2[p:p + n], "want": list(range(n))}]
            if len(rest) > 1 and _ == 0:
                rid3, toks3 = rest[1]
                k = max(1, len(toks3) // 2)
                entries.append({"id": rid3, "tokens": toks3[:k], "want": list(range(k))})
            steps.append({"entries": entries, "end": []})
            p += n
    live0 = {second: p}
    if len(rest) > 1:
        live0[rest[1][0]] = max(1, len(rest[1][1]) // 2)
    done = [rid for rid, at in live0.items() if at >= len(requests[rid])]
    for rid in done:                     # a request that is complete already ends with the step before
        steps[-1]["end"].append(rid)
        del live0[rid]
    again = {first: toks, **{rid: t for rid, t in others.items() if rid not in done}}
    steps += mixed(again, seed=seed, live0=live0)
    return _number(steps)


def _number(steps):
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def tokens_needed(trace, round_to=64):
    """The largest number of tokens that live requests hold at any time, each
    request's count rounded up to ``round_to``: what --max-tokens must be."""
    held: dict[str, int] = {}
    worst = 0
    for step in trace:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return worst


def collect(trace, outputs, lives=False):
    """outputs[i]: array [wanted, V] of step i (or None).  Returns
    {request: {position: logits row}}; a request that ends and is opened again starts at
    position 0 again (its later rows replace the earlier ones, or, with ``lives``, every
    life is kept under "<request>#<life>")."""
    got: dict[str, dict[int, np.ndarray]] = {}
    pos: dict[str, int] = {}
    life: dict[str, int] = {}
    for step, out in zip(trace, outputs):
        row = 0
        for e in step["entries"]:
            p0 = pos.get(e["id"], 0)
            key = f"{e['id']}#{life.get(e['id'], 0)}" if lives else e["id"]
            for w in e.get("want", []):
                got.setdefault(key, {})[p0 + w] = out[row]
                row += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        assert out is None or row == len(out)
        for rid in step["end"]:
            pos.pop(rid, None)
            life[rid] = life.get(rid, 0) + 1
    return got


def oracle(cfg, weights, requests):
    """Whole-sequence logits of the plain implementation: {request: [T, V]}."""
    return {rid: plain_gpt2.forward(cfg, weights, toks) for rid, toks in requests.items()}


def first_difference(got, want, tolerance, partial=()):
    """(request, position, |diff|) of the first position beyond the tolerance,
    in position order, or None.  Requests named in ``partial`` are compared only at the
    positions they have."""
    for rid in want:
        for p in range(want[rid].shape[0]):
            if rid in partial and p not in got.get(rid, {}):
                continue
            if p not in got.get(rid, {}):
                return rid, p, float("nan")
            d = float(np.abs(got[rid][p] - want[rid][p]).max())
            if not d <= tolerance:
                return rid, p, d
    return None
