"""Companions of the replay program: traces of the four families from given token lists, and a comparer.

A trace is a list of step records as ``bin/trace_run`` reads them (one JSON object a line):

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 1, 2]}], "end": []}

The families cut the same requests in different ways; what a replay writes for them must agree position by position:

* ``whole``        each request alone and whole, one step;
* ``tail_decode``  most of it in one step, the last tokens one by one;
* ``portions``     portions of changing size, down to two tokens;
* ``mixed``        several live requests, portions of some beside single tokens of others, by a plan.

``by_position`` turns a replay's results into ``{(request, absolute position): logits row}``, ``compare`` holds two
such maps against each other.  ``bin/trace_make`` and ``bin/trace_compare`` are the same functions from the command
line.  (The reference has no such instrument; its nearest is ``perplexity()``, scripts/jiuge.py:588-639.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from itertools import cycle
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np


# ---- the four families ---------------------------------------------------------------------------------------------
def whole(rid, toks: Sequence[int], step0: int = 0, end: bool = True) -> List[dict]:
    """One step with the whole request; every position wanted."""
    return [{"step": step0, "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
             "end": [rid] if end else []}]


def tail_decode(rid, toks: Sequence[int], tail: int = 32, step0: int = 0) -> List[dict]:
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


def portions(rid, toks: Sequence[int], sizes: Sequence[int] = (7, 2, 5, 3, 2, 11, 2, 4), step0: int = 0) -> List[dict]:
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


def mixed(requests: Dict[str, Sequence[int]], plan: List[Dict[str, int]]) -> List[dict]:
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


def staggered_plan(requests: Dict[str, Sequence[int]], live: int = 4, portion: int = 5, tail: int = 8) -> List[Dict[str, int]]:
    """A plan for ``mixed``: at most ``live`` requests at a time, admitted in order; a request runs in portions of
    ``portion`` tokens (its first a token longer, so that requests fall out of step) and its last ``tail`` tokens one by
    one, beside whatever the others run.  Requests that end make room for the next ones, whose pages are then the
    ones given back."""
    order = list(requests)
    left = {r: len(requests[r]) for r in order}
    waiting, running, plan = list(order), [], []
    while waiting or running:
        while waiting and len(running) < live:
            running.append(waiting.pop(0))
        row = {}
        for i, r in enumerate(running):
            n = 1 if left[r] <= tail else min(portion + (1 if left[r] == len(requests[r]) and i % 2 else 0), left[r] - tail)
            row[r] = n
            left[r] -= n
        plan.append(row)
        running = [r for r in running if left[r] > 0]
    return plan


# ---- reading what a replay wrote -------------------------------------------------------------------------------------
def by_position(steps: Iterable[dict], results: Dict[int, np.ndarray]) -> Dict[Tuple[object, int], np.ndarray]:
    """{(request, absolute position): logits row} from a replay's results (``{step: [wanted, vocab]}``)."""
    pos: Dict[object, int] = {}
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


def peak_tokens(steps: Iterable[dict], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request rounded up to ``round_to``: what
    ``bin/trace_run --max-tokens`` wants."""
    held: Dict[object, int] = {}
    peak = 0
    for rec in steps:
        for e in rec["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for r in rec.get("end", ()):
            held.pop(r, None)
    return peak


def read_results(out_dir: str, steps: Iterable[dict]) -> Dict[int, np.ndarray]:
    """The ``<step>.f32`` files of a replay as ``{step: float32 [wanted, vocab]}``."""
    results = {}
    for rec in steps:
        wanted = sum(len(e.get("want", ())) for e in rec["entries"])
        if not wanted:
            continue
        data = np.fromfile(os.path.join(out_dir, f"{rec['step']}.f32"), dtype="<f4")
        if data.size % wanted:
            raise ValueError(f"step {rec['step']}: {data.size} values are no whole number of rows for {wanted} wanted places")
        results[rec["step"]] = data.reshape(wanted, -1)
    return results


# ---- the comparer ---------------------------------------------------------------------------------------------------
def compare(a: Dict[Tuple[object, int], np.ndarray], b: Dict[Tuple[object, int], np.ndarray],
            rtol: float = 0.0, atol: float = 0.0, worst: int = 5) -> dict:
    """Hold two maps of logits by (request, position) against each other.  A row differs if
    ``max |a - b| > atol + rtol * max |b|`` (one bound a row, scaled by the row's largest logit: rounding shows in all
    logits alike).  Returns ``{"positions", "only_a", "only_b", "failed", "max_abs", "worst": [...]}``; ``worst`` lists the
    rows with the largest difference with their request, position, difference, the row's scale and both argmaxes."""
    keys = sorted(set(a) & set(b), key=lambda k: (str(k[0]), k[1]))
    rows = []
    for k in keys:
        x, y = np.asarray(a[k], dtype=np.float64), np.asarray(b[k], dtype=np.float64)
        if x.shape != y.shape:
            raise ValueError(f"{k}: rows of {x.shape} and {y.shape}")
        diff = float(np.max(np.abs(x - y))) if x.size else 0.0
        if not np.isfinite(diff):
            diff = float("inf")
        scale = float(np.max(np.abs(y))) if y.size else 0.0
        rows.append((diff, k, scale, int(np.argmax(x)) if x.size else -1, int(np.argmax(y)) if y.size else -1))
    failed = [r for r in rows if not r[0] <= atol + rtol * r[2]]
    rows.sort(key=lambda r: -r[0])
    return {
        "positions": len(keys),
        "only_a": sorted((str(k[0]), k[1]) for k in set(a) - set(b)),
        "only_b": sorted((str(k[0]), k[1]) for k in set(b) - set(a)),
        "failed": len(failed),
        "first_failed": min(((str(r[1][0]), r[1][1]) for r in failed), default=None),
        "max_abs": rows[0][0] if rows else 0.0,
        "worst": [{"request": str(r[1][0]), "position": r[1][1], "max_abs": r[0], "scale": r[2], "argmax_a": r[3], "argmax_b": r[4]}
                  for r in rows[:worst]],
    }


# ---- command lines ---------------------------------------------------------------------------------------------------
def _load_trace(path: str) -> List[dict]:
    with (sys.stdin if path == "-" else open(path)) as f:
        return [json.loads(line) for line in f if line.strip()]


def make_main(argv=None) -> int:
    """bin/trace_make: a trace of one family for the requests of a JSON file ``{"id": [token, ...], ...}``."""
    ap = argparse.ArgumentParser(prog="trace_make", description=make_main.__doc__)
    ap.add_argument("--requests", required=True, help="JSON file {id: [token ids]}, or - for standard input")
    ap.add_argument("--family", required=True, choices=["whole", "tail", "portions", "mixed"])
    ap.add_argument("--tail", type=int, default=32, help="tail: how many last tokens run one by one")
    ap.add_argument("--sizes", default="7,2,5,3,2,11,2,4", help="portions: the cycle of portion sizes")
    ap.add_argument("--live", type=int, default=4, help="mixed: most requests live at a time")
    ap.add_argument("--portion", type=int, default=5, help="mixed: tokens of a prompt portion")
    ap.add_argument("--plan", default=None, help="mixed: JSON file [{id: tokens in this step}, ...] instead of the built-in plan")
    args = ap.parse_args(argv)
    with (sys.stdin if args.requests == "-" else open(args.requests)) as f:
        requests = json.load(f)
    if args.family == "mixed":
        if args.plan:
            with open(args.plan) as f:
                plan = json.load(f)
        else:
            plan = staggered_plan(requests, live=args.live, portion=args.portion, tail=min(args.tail, 8))
        steps = mixed(requests, plan)
    else:
        steps, s = [], 0
        for rid, toks in requests.items():
            if args.family == "whole":
                part = whole(rid, toks, step0=s)
            elif args.family == "tail":
                part = tail_decode(rid, toks, tail=args.tail, step0=s)
            else:
                part = portions(rid, toks, sizes=tuple(int(x) for x in args.sizes.split(",")), step0=s)
            steps.extend(part)
            s += len(part)
    for rec in steps:
        print(json.dumps(rec))
    print(f"[trace_make] {len(steps)} steps; --max-tokens {peak_tokens(steps)}", file=sys.stderr)
    return 0


def compare_main(argv=None) -> int:
    """bin/trace_compare: two replays (their traces and output folders) against each other, position by position."""
    ap = argparse.ArgumentParser(prog="trace_compare", description=compare_main.__doc__)
    ap.add_argument("--trace-a", required=True)
    ap.add_argument("--out-a", required=True)
    ap.add_argument("--trace-b", required=True)
    ap.add_argument("--out-b", required=True)
    ap.add_argument("--rtol", type=float, default=0.0, help="allowed difference as a fraction of a row's largest logit")
    ap.add_argument("--atol", type=float, default=0.0)
    args = ap.parse_args(argv)
    ta, tb = _load_trace(args.trace_a), _load_trace(args.trace_b)
    report = compare(by_position(ta, read_results(args.out_a, ta)), by_position(tb, read_results(args.out_b, tb)),
                     rtol=args.rtol, atol=args.atol)
    print(json.dumps(report, indent=1))
    return 0 if not report["failed"] and not report["only_a"] and not report["only_b"] else 1
