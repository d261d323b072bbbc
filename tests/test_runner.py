"""The native step (csrc/runner.cu) replays a model's launch records.  A whole run of records in one call may let
neighbouring records share work (steps of few rows run without norm kernels); every record as a call of its own is the
unfused way of running the same program.  The two must give the same logits, and models with parts that emit no
records must run too, with those parts as host steps."""
import numpy as np
import pytest
import torch

from test_replay import TOL, check, expected, make_engine, run
from trace_helpers import mixed, portions, tail_decode, whole

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_native_runner_and_parts_give_the_same_logits(tiny_models, name):
    folder = tiny_models[name][0]
    native = make_engine(folder, "bfloat16", 1024)
    native.runtime.fused_norms = False       # the same kernels both ways: what neighbouring records share is tested below
    parts = make_engine(folder, "bfloat16", 1024, native_runner=False)
    assert not native.runner.one_by_one and parts.runner.one_by_one and native.program.native_only
    toks, want = expected(tiny_models, name, 500, 200)
    toks2, want2 = expected(tiny_models, name, 501, 90)
    reqs = {"a": toks, "b": toks2}
    plan = [{"a": 150}, {"a": 1, "b": 60}, {"a": 2, "b": 1}, {"a": 1, "b": 1}, {"a": 46, "b": 28}]
    for what, steps in (("whole", whole("a", toks)), ("tail", tail_decode("a", toks)),
                        ("portions", portions("a", toks, sizes=(40, 3, 130, 9, 2))), ("mixed", mixed(reqs, plan))):
        got_n, got_p = run(native, steps), run(parts, steps)
        assert got_n.keys() == got_p.keys()
        scale = np.abs(want).max()
        for key in got_n:
            # the same kernels in the same order: equal to the last bit, except where a product of 17 to
            # 1023 rows went to the library through two doors (torch.mm there, cublasGemmEx here), whose
            # choice of kernel may differ
            assert np.abs(got_n[key] - got_p[key]).max() <= 2e-3 * scale, (name, what, key)
        check(got_n, "a", want, TOL["bfloat16"], f"{name} native {what}")
    # decoded tokens only: the same product kernels; a product that waits for the next norm is added by the norm's
    # kernel in one way of running and by a kernel of its own in the other, the same float32 sum from two kernels
    steps = tail_decode("a", toks[:40], tail=40)
    got_n, got_p = run(native, steps), run(parts, steps)
    for key in got_n:
        assert np.abs(got_n[key] - got_p[key]).max() <= 2e-3 * np.abs(want).max(), (name, "decode", key)
    native.check()


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_steps_of_few_rows_run_without_norm_kernels(tiny_models, name):
    """The runner's own way for steps of at most 16 rows: the products around a norm share its work (the one before
    adds itself into the residual stream and leaves activations and sums of squares, the one after scales its rows),
    so the activations are rounded to bfloat16 before the 1 / rms instead of after.  Against the plain implementation,
    however the request is cut; the same bits every time; fewer launches than with the norm kernels."""
    folder = tiny_models[name][0]
    fused = make_engine(folder, "bfloat16", 1024)
    kept = make_engine(folder, "bfloat16", 1024)
    kept.runtime.fused_norms = False         # before its first step: decode steps are captured once
    assert fused.runtime.fused_norms and fused.program.native_only
    toks, want = expected(tiny_models, name, 500, 200)
    toks2, want2 = expected(tiny_models, name, 501, 90)
    plan = [{"a": 150}, {"a": 1, "b": 60}, {"a": 2, "b": 1}, {"a": 1, "b": 1}, {"a": 46, "b": 28}]
    for what, steps in (("tail", tail_decode("a", toks)), ("portions", portions("a", toks, sizes=(40, 3, 130, 9, 2, 16))),
                        ("mixed", mixed({"a": toks, "b": toks2}, plan)), ("one by one", tail_decode("a", toks[:60], tail=60))):
        got = run(fused, steps)
        check(got, "a", want[:60] if what == "one by one" else want, TOL["bfloat16"], f"{name} without norm kernels, {what}")
        if what == "mixed":
            check(got, "b", want2, TOL["bfloat16"], f"{name} without norm kernels, {what} (b)")
        again = run(fused, steps)
        for key in got:
            assert np.array_equal(got[key], again[key]), (name, what, key)
    steps = tail_decode("a", toks[:40], tail=40)
    counts = []
    for eng in (fused, kept):
        before = eng.kernel_launches
        run(eng, steps)
        counts.append((eng.kernel_launches - before) // len(steps))
    layers = tiny_models[name][1]["num_hidden_layers"]
    # two norm kernels a layer fewer, but the first layer's first; one clearing of the sums more
    assert counts[1] - counts[0] == 2 * layers - 1 - 1, counts
    fused.check()


@pytest.mark.parametrize("name", ["B", "D"])
def test_runner_and_parts_route_few_rows_alike(tiny_models, name):
    """With the few-rows tcgen05 kernel forced on for every size (a tiny model never has a block per SM), steps of
    17 to 128 rows take it on both ways of running a step: o and down add into the residual stream from several
    blocks that split K, gate/up applies SwiGLU, the logits are stored."""
    folder = tiny_models[name][0]
    native = make_engine(folder, "bfloat16", 1024)
    parts = make_engine(folder, "bfloat16", 1024, native_runner=False)
    native.runtime.skinny_min_blocks = parts.runtime.skinny_min_blocks = 1
    native.runtime.fused_norms = False       # this test is about the products
    toks, want = expected(tiny_models, name, 510, 180)
    for what, steps in (("portions", portions("a", toks, sizes=(100, 17, 30, 5, 28))), ("tail", tail_decode("a", toks))):
        got_n, got_p = run(native, steps), run(parts, steps)
        scale = np.abs(want).max()
        for key in got_n:
            # partial sums of the blocks that split K are added in the order the blocks finish: rounding only
            assert np.abs(got_n[key] - got_p[key]).max() <= 2e-3 * scale, (name, what, key)
        check(got_n, "a", want, TOL["bfloat16"], f"{name} few rows {what}")
        check(got_p, "a", want, TOL["bfloat16"], f"{name} few rows {what} (parts)")
    native.check()
    assert native.runner.env.routing.skinny_min_blocks == 1


def test_every_model_has_a_program_of_records(tiny_models):
    """Sizes outside the fast kernels (hidden 80, heads of 48) and float32 run from records too: the native step picks
    other kernels for them, it does not hand the model back."""
    eng = make_engine(tiny_models["C"][0], "bfloat16", 256)
    assert eng.program.native_only
    layers = tiny_models["C"][1]["num_hidden_layers"]
    assert eng.program.launch_list() == ["embed"] + ["norm", "qkv", "attention", "residual", "norm", "gate_up", "residual"] * layers + ["norm", "linear"]
    eng = make_engine(tiny_models["A"][0], "float32", 256)
    assert eng.program.native_only and len(eng.program.launch_list()) == 7 * 2 + 3
