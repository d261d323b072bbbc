"""Replay of the same requests cut in different ways, in float32 and bfloat16, against the plain
implementation: whole; most in one step and the last 32 one by one; portions of changing size;
mixed with other requests in a pool so small that pages are used again."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, random_tokens
from plain_minicpm import plain_forward
from trace_helpers import by_position, mixed, peak_tokens, portions, tail_decode, whole

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# float32: only the order of additions differs from the float64 plain implementation.
# bfloat16: activations are rounded to 8 significant bits about five times a layer; with 2-3 layers
# the logits carry an error of about sqrt(5 L) * 2^-9 = 0.8 % of their scale; three times that is allowed.
TOL = {"float32": 3e-5, "bfloat16": 2.5e-2}
LENGTHS = {"A": [5, 47, 130], "B": [1, 40, 97], "C": [33, 64, 100], "D": [9, 140, 300], "E": [3, 70, 200]}


def make_engine(folder, dtype, cache_tokens, page_size=16, **kw):
    from infinicore_infer_b200.engine import Engine
    return Engine.from_folder(folder, dtype=DTYPES[dtype], cache_tokens=cache_tokens, page_size=page_size,
                              max_requests=8, max_step_tokens=1024, **kw)


def run(engine, steps):
    from infinicore_infer_b200.trace import replay
    return by_position(steps, replay(engine, steps))


_expected = {}


def expected(models, name, seed, n):
    key = (name, seed, n)
    if key not in _expected:
        _, cfg, w = models[name]
        toks = random_tokens(seed, n, cfg["vocab_size"])
        _expected[key] = (toks, plain_forward(cfg, w, toks).numpy())
    return _expected[key]


def check(got, rid, want, tol, what):
    scale = np.abs(want).max()
    for p in range(len(want)):
        err = np.abs(got[(rid, p)].astype(np.float64) - want[p]).max()
        assert err <= tol * scale, f"{what}: request {rid} position {p}: error {err:.3e} > {tol * scale:.3e}"


@pytest.fixture(scope="module")
def engines(tiny_models):
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = make_engine(tiny_models[name][0], dtype, 1024)
        return cache[(name, dtype)]
    return get


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_tail_and_portions_agree_with_the_plain_implementation(tiny_models, engines, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate(LENGTHS[name]):
        toks, want = expected(tiny_models, name, 100 + i, n)
        results = {}
        for what, steps in (("whole", whole("r", toks)), ("tail", tail_decode("r", toks)),
                            ("portions", portions("r", toks))):
            got = run(eng, steps)
            check(got, "r", want, TOL[dtype], f"{name} {dtype} {what} n={n}")
            results[what] = np.stack([got[("r", p)] for p in range(n)])
        # The ways of cutting agree with one another.  float32: every kernel adds in the same order
        # whatever the batch, so they agree to the last bits.  bfloat16: a portion runs on the
        # tensor-core tile kernel and a decoded token on the split-key kernel, two evaluations that
        # round independently, so they agree as well as each agrees with the plain implementation.
        cut_tol = 1e-5 if dtype == "float32" else TOL[dtype]
        for what in ("tail", "portions"):
            assert np.abs(results[what] - results["whole"]).max() <= cut_tol * np.abs(want).max(), (name, dtype, what, n)
        assert not eng.cache.lengths and all(g.pool.in_use == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_product_kernel_gives_the_same_model(tiny_models, name):
    """The bfloat16 products have four homes: the tiled tcgen05 kernel (many rows; here forced on for any
    step of more than 16 rows), the few-rows tcgen05 kernel with the weights on the MMA's M side (17 to 128
    rows once it has a block per SM; here forced on for any size), the weight-streaming kernel (up to 16
    rows) and the library.  The model's logits must not care."""
    toks, want = expected(tiny_models, name, 150, 120)
    steps = portions("r", toks, sizes=(70, 3, 33, 14))       # 70 and 33 rows: tcgen05; 3 and 14: weight streaming
    for mode in ("tcgen05", "few rows", "library"):
        eng = make_engine(tiny_models[name][0], "bfloat16", 256)
        if mode == "tcgen05":
            eng.runtime.tcgen05_min_tiles = 1
            eng.runtime.tcgen05_min_rows = 17
            eng.runtime.tcgen05_min_fill_pct = 0
        elif mode == "few rows":
            eng.runtime.skinny_min_blocks = 1
        else:
            eng.runtime.library_products_only = True
        got = run(eng, steps)
        check(got, "r", want, TOL["bfloat16"], f"{name} products by {mode}")


@pytest.fixture(params=[1, 2], ids=["single blocks", "pairs of blocks"])
def product_pairs(request):
    from infinicore_infer_b200 import kernels
    before = kernels.gemm_tcgen05_pairs(request.param)
    yield request.param
    kernels.gemm_tcgen05_pairs(1 if before < 0 else before)


def test_the_tcgen05_kernels_carry_a_whole_model(tiny_models, product_pairs):
    """Heads of 64: portions of more than 8 rows run the tcgen05 attention kernel; with the row limit of
    the tcgen05 product lowered, the q/k/v product rotates and writes the cache in its epilogue, gate/up
    applies SwiGLU in its epilogue and o/down add into the residual stream by TMA.  Whole, in portions
    (several 128-row tiles, ragged ends) and mixed with decoded tokens, against the plain implementation;
    once with every product on single blocks (tiny products never reach pairs by themselves), once with
    every product of more than 128 rows on pairs of blocks."""
    eng = make_engine(tiny_models["D"][0], "bfloat16", 1024)
    eng.runtime.tcgen05_min_tiles = 1
    eng.runtime.tcgen05_min_rows = 17
    eng.runtime.tcgen05_min_fill_pct = 0
    toks, want = expected(tiny_models, "D", 400, 300)
    toks2, want2 = expected(tiny_models, "D", 401, 150)
    for what, steps in (("whole", whole("r", toks)), ("portions", portions("r", toks, sizes=(140, 2, 129, 20, 9))),
                        ("tail", tail_decode("r", toks))):
        got = run(eng, steps)
        check(got, "r", want, TOL["bfloat16"], f"D tcgen05 {what}")
    # two requests at once: a portion of one beside decoded tokens of the other
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:200], "want": list(range(200))}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[200:201], "want": [0]},
                                     {"id": "b", "tokens": toks2[:149], "want": list(range(149))}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[201:300], "want": list(range(99))},
                                     {"id": "b", "tokens": toks2[149:150], "want": [0]}], "end": ["a", "b"]}]
    got = run(eng, steps)
    check(got, "a", want, TOL["bfloat16"], "D tcgen05 mixed a")
    check(got, "b", want2, TOL["bfloat16"], "D tcgen05 mixed b")
    eng.check()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_mixed_requests_in_a_pool_so_small_that_pages_are_used_again(tiny_models, name, dtype):
    lens = {"a": 70, "b": 33, "c": 90, "d": 48, "e": 61, "f": 20}
    reqs, wants = {}, {}
    for i, (r, n) in enumerate(lens.items()):
        reqs[r], wants[r] = expected(tiny_models, name, 200 + i, n)
    plan = [
        {"a": 40},                              # a portion alone
        {"a": 2, "b": 30},                      # two tokens of a beside a portion of b
        {"a": 1, "b": 1, "c": 50},              # decoded tokens beside a portion
        {"a": 1, "b": 1, "c": 38, "d": 9},      # four live, portions beside single tokens
        {"a": 26, "b": 1, "c": 1, "d": 2},      # a ends, b ends
        {"c": 1, "d": 37, "e": 13},             # c ends; e takes pages that a and b gave back
        {"e": 2, "f": 3},
        {"e": 1, "f": 1},
        {"e": 45, "f": 16},
    ]
    steps = mixed(reqs, plan)
    assert max(len(s["entries"]) for s in steps) == 4
    peak = peak_tokens(steps, round_to=16)      # exactly the pages the live requests need at the worst moment
    eng = make_engine(tiny_models[name][0], dtype, peak)
    assert sum(lens.values()) > 1.3 * peak      # the pool cannot hold them all: pages must come back
    got = run(eng, steps)
    for r in reqs:
        check(got, r, wants[r], TOL[dtype], f"{name} {dtype} mixed")
    g = eng.cache.groups[0]
    assert g.pool.high_water == g.pool.capacity == peak // 16 and g.pool.in_use == 0


# Pages of other sizes than 16: tiny-B at its own 8; tiny-D (heads of 64: the tcgen05 attention builds another TMA box per
# page size, and 128 keys are one page, two, or sixteen) at 8, 64 and 128; tiny-C (head size 48, the mma.sync kernels) at 4.
PAGE_CASES = [("B", 8), ("D", 8), ("D", 64), ("D", 128), ("C", 4), ("A", 32)]


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name,page", PAGE_CASES)
def test_every_way_of_cutting_at_other_page_sizes(tiny_models, name, page, dtype):
    eng = make_engine(tiny_models[name][0], dtype, 1024, page_size=page)
    for i, n in enumerate(LENGTHS[name][1:]):
        toks, want = expected(tiny_models, name, 101 + i, n)
        for what, steps in (("whole", whole("r", toks)), ("tail", tail_decode("r", toks)), ("portions", portions("r", toks))):
            check(run(eng, steps), "r", want, TOL[dtype], f"{name} page {page} {dtype} {what} n={n}")
    # mixed, in a pool of exactly the pages the live requests need at the worst moment
    lens = {"a": 70, "b": 33, "c": 90, "d": 48, "e": 61, "f": 20}
    reqs, wants = {}, {}
    for i, (r, n) in enumerate(lens.items()):
        reqs[r], wants[r] = expected(tiny_models, name, 200 + i, n)
    plan = [{"a": 40}, {"a": 2, "b": 30}, {"a": 1, "b": 1, "c": 50}, {"a": 1, "b": 1, "c": 38, "d": 9},
            {"a": 26, "b": 1, "c": 1, "d": 2}, {"c": 1, "d": 37, "e": 13}, {"e": 2, "f": 3}, {"e": 1, "f": 1}, {"e": 45, "f": 16}]
    steps = mixed(reqs, plan)
    peak = peak_tokens(steps, round_to=page)
    eng = make_engine(tiny_models[name][0], dtype, peak, page_size=page)
    got = run(eng, steps)
    for r in reqs:
        check(got, r, wants[r], TOL[dtype], f"{name} page {page} {dtype} mixed")
    g = eng.cache.groups[0]
    assert g.pool.high_water == g.pool.capacity == peak // page and g.pool.in_use == 0
    eng.check()


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_an_entry_may_want_nothing_in_a_decode_step(tiny_models, engines, dtype):
    """A decode step (single tokens only, so it runs as a captured graph) in which one request asks for no logits
    and another for its one row: the rows that come back are the wanted ones, in order."""
    name = "A"
    ta, wa = expected(tiny_models, name, 410, 20)
    tb, wb = expected(tiny_models, name, 411, 16)
    tc, wc = expected(tiny_models, name, 412, 12)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ta[:10], "want": []}, {"id": "b", "tokens": tb[:10], "want": [9]},
                                     {"id": "c", "tokens": tc[:10], "want": []}], "end": []}]
    for s in range(1, 3):
        steps.append({"step": s, "entries": [{"id": "a", "tokens": [ta[9 + s]], "want": [0] if s == 2 else []},
                                             {"id": "b", "tokens": [tb[9 + s]], "want": []},
                                             {"id": "c", "tokens": [tc[9 + s]], "want": [0]}], "end": []})
    steps.append({"step": 3, "entries": [{"id": "a", "tokens": [ta[12]], "want": []}, {"id": "b", "tokens": [tb[12]], "want": []}],
                  "end": ["a", "b", "c"]})
    from infinicore_infer_b200.trace import replay
    results = replay(engines(name, dtype), steps)
    assert sorted(results) == [0, 1, 2]                     # step 3 wants nothing: no rows, no file
    got = by_position(steps, results)
    assert sorted(got) == [("a", 11), ("b", 9), ("c", 10), ("c", 11)]
    tol = TOL[dtype]
    for (r, p), row in got.items():
        want = {"a": wa, "b": wb, "c": wc}[r]
        assert np.abs(row - want[p]).max() <= tol * np.abs(want).max(), (r, p)


def test_logits_of_a_captured_step_are_the_caller_s_own(tiny_models):
    """``Engine.step`` hands back rows that the next captured decode step must not change."""
    from infinicore_infer_b200.engine import StepEntry
    folder, cfg, _ = tiny_models["A"]
    eng = make_engine(folder, "bfloat16", 256)
    toks = random_tokens(3, 12, cfg["vocab_size"])
    eng.step([StepEntry("a", toks[:8], [7])])
    first = eng.step([StepEntry("a", [toks[8]], [0])])
    keep = first.clone()
    eng.step([StepEntry("a", [toks[9]], [0])])
    eng.step([StepEntry("a", [toks[10]], [0])])
    assert torch.equal(first, keep)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_decoding_and_the_first_tokens(tiny_models, engines, dtype):
    name = "B"
    toks, want = expected(tiny_models, name, 300, 260)
    eng = engines(name, dtype)
    # the first tokens of a sequence, one by one from position 0, then a long run of single tokens
    steps = tail_decode("r", toks, tail=len(toks))
    assert all(len(s["entries"][0]["tokens"]) == 1 for s in steps)
    got = run(eng, steps)
    check(got, "r", want, TOL[dtype], f"{name} {dtype} long decode")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_batched_decode_steps_of_changing_size(tiny_models, engines, dtype):
    """Decode steps run as captured graphs per batch-size bucket; requests join and leave."""
    name = "A"
    lens = {"a": 30, "b": 12, "c": 25, "d": 9, "e": 17}
    reqs, wants = {}, {}
    for i, (r, n) in enumerate(lens.items()):
        reqs[r], wants[r] = expected(tiny_models, name, 400 + i, n)
    plan = [{"a": 5, "b": 3}] + [{"a": 1, "b": 1}] * 4 + [{"a": 1, "b": 1, "c": 1}] * 5 + \
           [{"a": 1, "c": 1, "d": 1, "e": 1}] * 9 + [{"a": 1, "c": 11, "e": 1}] + [{"a": 1, "e": 1, "c": 1}] * 10
    steps = mixed(reqs, plan)
    got = run(engines(name, dtype), steps)
    for r in reqs:
        check(got, r, wants[r], TOL[dtype], f"{name} {dtype} batched decode")


def test_a_step_that_does_not_fit_changes_nothing(tiny_models):
    from infinicore_infer_b200.cache import OutOfPages
    from infinicore_infer_b200.engine import StepEntry, StepError
    folder, cfg, _ = tiny_models["A"]
    eng = make_engine(folder, "float32", 64)
    toks = random_tokens(1, 80, cfg["vocab_size"])
    eng.step([StepEntry("a", toks[:40], [39])])
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", toks[40:60], [0]), StepEntry("b", toks[:30], [0])])
    assert eng.position("a") == 40 and not eng.cache.is_live("b")
    eng.cache.check_invariants()
    with pytest.raises(StepError, match="vocabulary"):
        eng.step([StepEntry("a", [cfg["vocab_size"]], [0])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(StepError, match="twice"):
        eng.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    out = eng.step([StepEntry("a", toks[40:64], [23])])
    assert out.shape == (1, cfg["vocab_size"]) and eng.position("a") == 64
    eng.cache.check_invariants()


def test_the_command_line_program(tiny_models, tmp_path):
    """bin/trace_run as a user runs it: steps on standard input, files and ``done`` lines out."""
    folder, cfg, w = tiny_models["B"]
    toks = random_tokens(9, 21, cfg["vocab_size"])
    other = random_tokens(10, 6, cfg["vocab_size"])
    steps = [
        {"step": 0, "entries": [{"id": "x", "tokens": toks[:9], "want": [0, 8]}], "end": []},
        {"step": 1, "entries": [{"id": "x", "tokens": toks[9:11], "want": []},
                                {"id": "y", "tokens": other, "want": [5]}], "end": ["y"]},
        {"step": 2, "entries": [{"id": "x", "tokens": toks[11:], "want": [9]}], "end": ["x"]},
    ]
    want = plain_forward(cfg, w, toks).numpy()
    want_y = plain_forward(cfg, w, other).numpy()
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        proc = subprocess.run(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
             "--out", str(out), "--max-tokens", "128"],
            input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert proc.stdout.split() == ["done", "0", "done", "1", "done", "2"]
        V = cfg["vocab_size"]
        r0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
        r1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
        r2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
        assert r0.shape[0] == 2 and r1.shape[0] == 1 and r2.shape[0] == 1
        tol = TOL[dtype] * np.abs(want).max()
        assert np.abs(r0[0] - want[0]).max() <= tol and np.abs(r0[1] - want[8]).max() <= tol
        assert np.abs(r1[0] - want_y[5]).max() <= TOL[dtype] * np.abs(want_y).max()
        assert np.abs(r2[0] - want[20]).max() <= tol
