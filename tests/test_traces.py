"""The companions of the replay program: the generators of the four families of traces and the comparer.
Without a GPU: what the generators promise (every token once, in order; the cuts; the ends) and what the comparer
reports.  With one: ``bin/trace_make | bin/trace_run`` for all four families, held against each other by
``bin/trace_compare``."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, random_tokens
from infinicore_infer_b200 import traces

REQUESTS = {"a": list(range(100, 171)), "b": list(range(200, 233)), "c": list(range(300, 390)),
            "d": list(range(400, 402)), "e": [7], "f": list(range(500, 561))}


def consumed(steps):
    """{request: its tokens in the order the trace runs them}; also checks ids of steps, wants and ends."""
    seen, ended = {}, set()
    for i, rec in enumerate(steps):
        assert rec["step"] == i
        for e in rec["entries"]:
            assert e["id"] not in ended and e["tokens"]
            assert all(0 <= w < len(e["tokens"]) for w in e["want"])
            seen.setdefault(e["id"], []).extend(e["tokens"])
        assert len({e["id"] for e in rec["entries"]}) == len(rec["entries"])
        ended |= set(rec["end"])
    assert ended == set(seen)
    return seen


@pytest.mark.parametrize("rid", list(REQUESTS))
def test_each_family_runs_every_token_once_and_in_order(rid):
    toks = REQUESTS[rid]
    for steps in (traces.whole(rid, toks), traces.tail_decode(rid, toks, tail=32), traces.tail_decode(rid, toks, tail=5),
                  traces.portions(rid, toks), traces.portions(rid, toks, sizes=(2, 3))):
        assert consumed(steps) == {rid: toks}
        assert steps[-1]["end"] == [rid] and all(not s["end"] for s in steps[:-1])
        wanted = sum(len(e["want"]) for s in steps for e in s["entries"])
        assert wanted == len(toks)


def test_the_cuts_of_the_families():
    toks = REQUESTS["a"]
    assert [len(s["entries"][0]["tokens"]) for s in traces.tail_decode("a", toks, tail=32)] == [len(toks) - 32] + [1] * 32
    assert [len(s["entries"][0]["tokens"]) for s in traces.tail_decode("d", REQUESTS["d"], tail=32)] == [1, 1]
    sizes = [len(s["entries"][0]["tokens"]) for s in traces.portions("a", toks)]
    assert sizes[:8] == [7, 2, 5, 3, 2, 11, 2, 4] and sum(sizes) == len(toks) and min(sizes[:-1]) == 2
    assert traces.whole("a", toks, step0=3, end=False) == [
        {"step": 3, "entries": [{"id": "a", "tokens": toks, "want": list(range(len(toks)))}], "end": []}]


@pytest.mark.parametrize("live,portion,tail", [(4, 5, 8), (2, 16, 3), (1, 7, 1), (3, 2, 32)])
def test_the_staggered_plan_keeps_its_bounds(live, portion, tail):
    plan = traces.staggered_plan(REQUESTS, live=live, portion=portion, tail=tail)
    steps = traces.mixed(REQUESTS, plan)
    assert consumed(steps) == REQUESTS
    held = set()
    for rec in steps:
        held |= {e["id"] for e in rec["entries"]}
        assert len(held) <= live
        held -= set(rec["end"])
    if live > 1:
        # portions of some beside single tokens of others, in one step
        assert any(len({len(e["tokens"]) == 1 for e in rec["entries"]}) == 2 for rec in steps)
    # the last tokens of a request of some length run one by one
    lens = [len(e["tokens"]) for rec in steps for e in rec["entries"] if e["id"] == "c"]
    assert lens[-min(tail, len(REQUESTS["c"])):] == [1] * min(tail, len(REQUESTS["c"]))


def test_a_plan_that_leaves_tokens_over_is_refused():
    with pytest.raises(AssertionError, match="does not consume"):
        traces.mixed({"a": [1, 2, 3]}, [{"a": 2}])


def test_peak_tokens_counts_what_live_requests_hold_rounded_by_request():
    steps = traces.mixed({"a": list(range(70)), "b": list(range(10))}, [{"a": 65}, {"a": 5, "b": 9}, {"b": 1}])
    assert traces.peak_tokens(steps, round_to=64) == 128 + 64       # a holds 70 -> 128, b 9 -> 64, in step 1
    assert traces.peak_tokens(steps, round_to=16) == 80 + 16
    assert traces.peak_tokens(traces.whole("a", [1] * 64) + traces.whole("b", [1] * 65, step0=1)) == 128


def fake_logits(rid, pos, vocab=11):
    rng = np.random.default_rng(sum(map(ord, rid)) * 1000 + pos)
    return rng.standard_normal(vocab).astype(np.float32)


def fake_results(steps, noise=0.0, seed=0):
    """What a replay would return if the logits of (request, position) were ``fake_logits`` (plus noise)."""
    rng = np.random.default_rng(seed)
    pos, out = {}, {}
    for rec in steps:
        rows = []
        for e in rec["entries"]:
            p0 = pos.get(e["id"], 0)
            rows += [fake_logits(e["id"], p0 + w) + noise * rng.standard_normal(11).astype(np.float32) for w in e["want"]]
            pos[e["id"]] = p0 + len(e["tokens"])
        if rows:
            out[rec["step"]] = np.stack(rows)
    return out


def test_by_position_and_the_comparer_over_all_families(tmp_path):
    plan = traces.staggered_plan(REQUESTS, live=3, portion=6, tail=4)
    families = {"mixed": traces.mixed(REQUESTS, plan)}
    for name, make in (("whole", traces.whole), ("tail", traces.tail_decode), ("portions", traces.portions)):
        steps = []
        for rid, toks in REQUESTS.items():
            steps += make(rid, toks, step0=len(steps))
        families[name] = steps
    maps = {name: traces.by_position(steps, fake_results(steps)) for name, steps in families.items()}
    keys = {(r, p) for r, toks in REQUESTS.items() for p in range(len(toks))}
    for name, m in maps.items():
        assert set(m) == keys, name
        report = traces.compare(m, maps["whole"])
        assert report["positions"] == len(keys) and report["failed"] == 0 and report["max_abs"] == 0.0
        assert report["only_a"] == [] and report["only_b"] == [] and report["first_failed"] is None

    # one row off, a position missing, another one extra: the report names them
    off = dict(maps["mixed"])
    off[("c", 41)] = off[("c", 41)] + np.float32(0.5) * (np.arange(11) == 3)
    off[("a", 71)] = off.pop(("a", 69))
    report = traces.compare(off, maps["whole"], rtol=1e-3)
    assert report["failed"] == 1 and report["first_failed"] == ("c", 41)
    assert report["worst"][0]["request"] == "c" and report["worst"][0]["position"] == 41
    assert abs(report["worst"][0]["max_abs"] - 0.5) < 1e-6
    assert report["only_a"] == [("a", 71)] and report["only_b"] == [("a", 69)]
    # a not-a-number never passes
    off = dict(maps["tail"])
    off[("b", 0)] = off[("b", 0)] * np.float32("nan")
    assert traces.compare(off, maps["whole"], rtol=1.0, atol=1.0)["failed"] == 1
    # noise below the bound passes, above it fails; the bound is a fraction of the row's largest logit
    noisy = traces.by_position(families["portions"], fake_results(families["portions"], noise=1e-4))
    assert traces.compare(noisy, maps["whole"], rtol=1e-2)["failed"] == 0
    assert traces.compare(noisy, maps["whole"], rtol=1e-7)["failed"] > 0


def test_results_come_back_from_the_files_of_a_replay(tmp_path):
    steps = traces.portions("a", REQUESTS["a"]) + [{"step": 99, "entries": [{"id": "z", "tokens": [1, 2], "want": []}], "end": ["z"]}]
    steps[-1]["step"] = len(steps) - 1
    results = fake_results(steps)
    for s, rows in results.items():
        rows.astype("<f4").tofile(tmp_path / f"{s}.f32")
    back = traces.read_results(str(tmp_path), steps)
    assert sorted(back) == sorted(results) and all(np.array_equal(back[s], results[s]) for s in back)
    (tmp_path / "0.f32").write_bytes(b"\0" * 4 * 10)               # 10 values for 7 wanted places
    with pytest.raises(ValueError, match="no whole number of rows"):
        traces.read_results(str(tmp_path), steps)


def test_trace_make_writes_what_the_functions_give(tmp_path):
    path = tmp_path / "requests.json"
    path.write_text(json.dumps(REQUESTS))
    make = [sys.executable, os.path.join(ROOT, "bin", "trace_make"), "--requests", str(path)]
    for family, args, want in (
            ("whole", [], lambda: [s for r, t in REQUESTS.items() for s in traces.whole(r, t)]),
            ("tail", ["--tail", "9"], lambda: [s for r, t in REQUESTS.items() for s in traces.tail_decode(r, t, tail=9)]),
            ("portions", ["--sizes", "4,2,9"], lambda: [s for r, t in REQUESTS.items() for s in traces.portions(r, t, sizes=(4, 2, 9))]),
            ("mixed", ["--live", "3", "--portion", "11"],
             lambda: traces.mixed(REQUESTS, traces.staggered_plan(REQUESTS, live=3, portion=11, tail=8)))):
        proc = subprocess.run(make + ["--family", family] + args, capture_output=True, text=True, timeout=120)
        assert proc.returncode == 0, proc.stderr[-2000:]
        got = [json.loads(line) for line in proc.stdout.splitlines()]
        expect = want()
        for i, s in enumerate(expect):
            s["step"] = i
        assert got == expect, family
        assert f"--max-tokens {traces.peak_tokens(got)}" in proc.stderr
    plan = tmp_path / "plan.json"
    plan.write_text(json.dumps([{"a": 71, "b": 2}, {"b": 31, "c": 90}, {"d": 2, "e": 1, "f": 61}]))
    proc = subprocess.run(make + ["--family", "mixed", "--plan", str(plan)], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0 and len(proc.stdout.splitlines()) == 3


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,rtol", [("float32", 6e-5), ("bfloat16", 5e-2)])
def test_the_three_programs_together(tiny_models, tmp_path, dtype, rtol):
    """Token lists -> bin/trace_make (each family) -> bin/trace_run -> bin/trace_compare against the whole requests.
    The bound is twice the one a replay keeps against the plain implementation: two replays differ from each other."""
    folder, cfg, _ = tiny_models["A"]
    requests = {r: random_tokens(900 + i, n, cfg["vocab_size"]) for i, (r, n) in
                enumerate({"a": 70, "b": 33, "c": 90, "d": 48, "e": 61, "f": 20}.items())}
    (tmp_path / "requests.json").write_text(json.dumps(requests))
    bin_ = lambda name: [sys.executable, os.path.join(ROOT, "bin", name)]
    for family in ("whole", "tail", "portions", "mixed"):
        proc = subprocess.run(bin_("trace_make") + ["--requests", str(tmp_path / "requests.json"), "--family", family, "--live", "4"],
                              capture_output=True, text=True, timeout=120)
        assert proc.returncode == 0, proc.stderr[-2000:]
        (tmp_path / f"{family}.jsonl").write_text(proc.stdout)
        peak = int(proc.stderr.split("--max-tokens")[1].split()[0])
        run = subprocess.run(bin_("trace_run") + ["--model", folder, "--dtype", dtype, "--out", str(tmp_path / family),
                                                  "--max-tokens", str(peak)],
                             input=proc.stdout, capture_output=True, text=True, timeout=600)
        assert run.returncode == 0, run.stderr[-2000:]
        assert run.stdout.count("done") == len(proc.stdout.splitlines())
    for family in ("tail", "portions", "mixed"):
        cmp_ = subprocess.run(bin_("trace_compare") + ["--trace-a", str(tmp_path / f"{family}.jsonl"), "--out-a", str(tmp_path / family),
                                                       "--trace-b", str(tmp_path / "whole.jsonl"), "--out-b", str(tmp_path / "whole"),
                                                       "--rtol", str(rtol)], capture_output=True, text=True, timeout=120)
        report = json.loads(cmp_.stdout)
        assert cmp_.returncode == 0 and report["failed"] == 0, (family, report)
        assert report["positions"] == sum(len(t) for t in requests.values())
    # a stricter bound than rounding allows makes it fail with status 1 (bfloat16 only: float32 replays may agree to the bit)
    if dtype == "bfloat16":
        cmp_ = subprocess.run(bin_("trace_compare") + ["--trace-a", str(tmp_path / "mixed.jsonl"), "--out-a", str(tmp_path / "mixed"),
                                                       "--trace-b", str(tmp_path / "whole.jsonl"), "--out-b", str(tmp_path / "whole"),
                                                       "--rtol", "1e-9"], capture_output=True, text=True, timeout=120)
        assert cmp_.returncode == 1 and json.loads(cmp_.stdout)["failed"] > 0
