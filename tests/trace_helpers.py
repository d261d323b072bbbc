"""Building traces (lists of step records) for the replay tests, and reading their results."""
from itertools import cycle
from typing import Dict, List, Sequence


def whole(rid, toks, step0=0, end=True):
    """One step with the whole request; every position wanted."""
    return [{"step": step0, "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
             "end": [rid] if end else []}]


def tail_decode(rid, toks, tail=32, step0=0):
    """Most of it in one step, the last ``tail`` tokens one by one (all one by one if short)."""
    head = max(0, len(toks) - tail)
    steps, s = [], step0
    if head:
        steps.append({"step": s, "entries": [{"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}], "end": []})
        s += 1
    for i in range(head, len(toks)):
        steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
        s += 1
    steps[-1]["end"] = [rid]
    return steps


def portions(rid, toks, sizes=(7, 2, 5, 3, 2, 11, 2, 4), step0=0):
    """Portions of changing size, down to two tokens."""
    steps, s, i = [], step0, 0
    for n in cycle(sizes):
        if i >= len(toks):
            break
        n = min(n, len(toks) - i)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": list(toks[i:i + n]), "want": list(range(n))}], "end": []})
        i += n
        s += 1
    steps[-1]["end"] = [rid]
    return steps


def mixed(requests: Dict[str, Sequence[int]], plan: List[Dict[str, int]]):
    """``plan[s]`` maps request -> how many of its next tokens run in step s.  A request ends
    after the step in which its last token ran."""
    done = {r: 0 for r in requests}
    steps = []
    for s, row in enumerate(plan):
        entries, end = [], []
        for r, n in row.items():
            toks = requests[r]
            n = min(n, len(toks) - done[r])
            if n <= 0:
                continue
            entries.append({"id": r, "tokens": list(toks[done[r]:done[r] + n]), "want": list(range(n))})
            done[r] += n
            if done[r] == len(toks):
                end.append(r)
        steps.append({"step": s, "entries": entries, "end": end})
    assert all(done[r] == len(requests[r]) for r in requests), "the plan does not consume every request"
    return steps


def by_position(steps, results):
    """{(request, absolute position): logits row} from a replay's results."""
    pos = {}
    out = {}
    for rec in steps:
        rows = results.get(rec["step"])
        i = 0
        for e in rec["entries"]:
            p0 = pos.get(e["id"], 0)
            for w in e.get("want", ()):
                out[(e["id"], p0 + w)] = rows[i]
                i += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        for r in rec.get("end", ()):
            pos.pop(r, None)
        assert rows is None or i == len(rows)
    return out


def peak_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each request rounded up to ``round_to``."""
    held, peak = {}, 0
    for rec in steps:
        for e in rec["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for r in rec.get("end", ()):
            held.pop(r, None)
    return peak
