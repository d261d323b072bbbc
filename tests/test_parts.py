"""Each part alone against its plain function, and models put together in other ways than
MiniCPM's: windows on some layers, a layer that runs twice, a layer that reads another's cache."""
import math
from dataclasses import replace

import numpy as np
import pytest
import torch

from conftest import TINY_A, TINY_B, TINY_C, random_tokens
from plain_minicpm import (plain_attention_layer, plain_forward, plain_rmsnorm, plain_swiglu_ffn)
from trace_helpers import by_position, portions, tail_decode, whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def _ctx(cache, reqs):
    """A StepContext for ``reqs`` = [(request id, start position, number of rows)], built by hand."""
    from infinicore_infer_b200.parts import StepContext
    rows = sum(n for _, _, n in reqs)
    pos = torch.cat([torch.arange(s, s + n) for _, s, n in reqs]).to(torch.int32)
    row_req = torch.cat([torch.full((n,), i) for i, (_, _, n) in enumerate(reqs)]).to(torch.int32)
    starts = np.cumsum([0] + [n for _, _, n in reqs])
    tables = []
    for gi in range(len(cache.groups)):
        arr = np.zeros((len(reqs), cache.max_blocks), dtype=np.int32)
        cache.block_table_rows(gi, [r for r, _, _ in reqs], arr)
        tables.append(torch.from_numpy(arr).to(DEV))
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=DEV)
    return StepContext(ntok=rows, nreq=len(reqs), tokens=i32([0] * rows), positions=pos.to(DEV),
                       row_req=row_req.to(DEV), req_start=i32(starts), req_pos=i32([s for _, s, _ in reqs]),
                       slot_ids=i32(cache.slot_ids([r for r, _, _ in reqs])), block_tables=tables,
                       want_rows=i32(list(range(rows))), n_want=rows,
                       host_req_start=list(starts), host_req_pos=[s for _, s, _ in reqs])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part_does_the_pending_addition(dtype):
    from infinicore_infer_b200.config import RMSNormSpec
    from infinicore_infer_b200.parts import ResidualStream, Runtime, part_class
    from infinicore_infer_b200.weights import DictWeights
    g = torch.Generator().manual_seed(0)
    w = 1 + 0.1 * torch.randn(96, generator=g)
    spec = RMSNormSpec(size=96, eps=1e-6)
    rt = Runtime(dtype, DEV)
    norm = part_class("norm", spec)(spec, DictWeights({"n.weight": w}, dtype, DEV), "n.", rt)
    x, delta = torch.randn(5, 96, generator=g), torch.randn(5, 96, generator=g)
    res = ResidualStream(x.to(DEV).clone())
    res.add(delta.to(DEV), 0.5)
    h = norm.forward(res, None)
    assert h.dtype == dtype and res.delta is None
    want = plain_rmsnorm(x.double() + 0.5 * delta.double(), w.double(), 1e-6)
    assert (h.double().cpu() - want).abs().max() <= _tol(dtype) * want.abs().max()
    assert torch.allclose(res.x.cpu(), x + 0.5 * delta, atol=1e-6)


def test_rotary_tables_are_float32_roundings_of_float64_angles():
    from infinicore_infer_b200.config import RopeSpec
    from infinicore_infer_b200.parts import Runtime, part_class
    spec = RopeSpec(head_dim=48, theta=50000.0, max_positions=300)
    rope = part_class("position", spec)(spec, None, "", Runtime(torch.float32, DEV))
    j = torch.arange(24, dtype=torch.float64)
    ang = torch.arange(300, dtype=torch.float64)[:, None] / 50000.0 ** (j / 24)
    assert torch.equal(rope.cos.cpu(), ang.cos().float()) and torch.equal(rope.sin.cpu(), ang.sin().float())
    assert rope.cos.shape == (300, 24)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [TINY_B, TINY_C])
def test_attention_part_alone_in_portions(cfg, dtype):
    """The mixer over its own cache: a sequence fed in two portions beside another request."""
    from infinicore_infer_b200.cache import CacheManager
    from infinicore_infer_b200.config import MiniCPMConfig
    from infinicore_infer_b200.parts import Runtime, part_class
    from infinicore_infer_b200.weights import DictWeights, random_tensors
    spec = MiniCPMConfig.from_dict(cfg).model_spec().layers[0].mixer
    cls = part_class("mixer", spec)
    w = random_tensors(cls.tensor_decls(spec), seed=3, std=0.1)
    rt = Runtime(dtype, DEV)
    attn = cls(spec, DictWeights({"a." + k: v for k, v in w.items()}, dtype, DEV), "a.", rt)
    cache = CacheManager([cls.cache_need(spec)], 16, 8, 4, 128, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(1)
    T = 27
    h = torch.randn(T, spec.hidden_size, generator=g).to(dtype)
    other = torch.randn(6, spec.hidden_size, generator=g).to(dtype)
    wf = {"a." + k: v.double() for k, v in w.items()}
    want, _ = plain_attention_layer(h.double(), wf, "a.", torch.arange(T), spec.num_heads, spec.num_kv_heads,
                                    spec.head_dim, spec.position.theta)
    cache.admit("x"); cache.admit("y")
    got = []
    for lo, hi, with_other in ((0, 11, False), (11, 27, True)):
        reqs = [("x", lo, hi - lo)] + ([("y", 0, 6)] if with_other else [])
        cache.reserve("x", hi)
        if with_other:
            cache.reserve("y", 6)
        ctx = _ctx(cache, reqs)
        rows = torch.cat([h[lo:hi]] + ([other] if with_other else [])).to(DEV)
        out = attn.forward(rows, ctx, cache.views[0], True)
        got.append(out[:hi - lo].double().cpu())
        cache.commit("x", hi)
    got = torch.cat(got)
    assert (got - want).abs().max() <= _tol(dtype) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part_alone(dtype):
    from infinicore_infer_b200.config import SwiGLUSpec
    from infinicore_infer_b200.parts import Runtime, part_class
    from infinicore_infer_b200.weights import DictWeights, random_tensors
    spec = SwiGLUSpec(hidden_size=80, intermediate_size=136)
    cls = part_class("feed_forward", spec)
    w = random_tensors(cls.tensor_decls(spec), seed=4, std=0.1)
    ffn = cls(spec, DictWeights({"m." + k: v for k, v in w.items()}, dtype, DEV), "m.", Runtime(dtype, DEV))
    h = torch.randn(9, 80, generator=torch.Generator().manual_seed(2)).to(dtype)
    out = ffn.forward(h.to(DEV), None)
    want = plain_swiglu_ffn(h.double(), w["gate_proj.weight"].double(), w["up_proj.weight"].double(),
                            w["down_proj.weight"].double())
    assert (out.double().cpu() - want).abs().max() <= _tol(dtype) * want.abs().max()


def _engine_for(cfg, spec, weights, dtype, cache_tokens=512, **kw):
    from infinicore_infer_b200.engine import Engine
    from infinicore_infer_b200.weights import DictWeights
    return Engine(spec, DictWeights(weights, dtype, DEV), dtype=dtype, device=DEV, cache_tokens=cache_tokens,
                  page_size=8, max_requests=4, max_step_tokens=512, **kw)


def _replay_all(eng, toks, want, tol, what):
    from infinicore_infer_b200.trace import replay
    scale = np.abs(want).max()
    for name, steps in (("whole", whole("r", toks)), ("tail", tail_decode("r", toks, tail=20)),
                        ("portions", portions("r", toks, sizes=(5, 2, 9, 3)))):
        got = by_position(steps, replay(eng, steps))
        for p in range(len(toks)):
            err = np.abs(got[("r", p)] - want[p]).max()
            assert err <= tol * scale, f"{what} {name} position {p}: {err:.3e} > {tol * scale:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_windows_on_some_layers_get_a_cache_group_of_their_own(tiny_models, dtype):
    """Layer 0 keeps all keys, layers 1 and 2 a window of 12: two groups; the window group's pages
    come back while the sequence grows, and logits still match the plain implementation."""
    from infinicore_infer_b200.config import MiniCPMConfig, ModelSpec
    _, cfg, w = tiny_models["B"]
    spec = MiniCPMConfig.from_dict(cfg).model_spec()
    windows = [None, 12, 12]
    layers = tuple(replace(l, mixer=replace(l.mixer, window=win)) for l, win in zip(spec.layers, windows))
    spec = replace(spec, layers=layers)
    eng = _engine_for(cfg, spec, w, dtype)
    assert len(eng.cache.groups) == 2 and eng.cache.groups[1].cache_ids == [1, 2]
    toks = random_tokens(21, 90, cfg["vocab_size"])
    want = plain_forward(cfg, w, toks, windows=windows).numpy()
    full = plain_forward(cfg, w, toks).numpy()
    assert np.abs(want - full).max() > 0.05 * np.abs(full).max()         # the window matters
    _replay_all(eng, toks, want, 3e-5 if dtype == torch.float32 else 2.5e-2, "windows")
    # decoding one by one, the window group never held more than window/page + 2 pages
    assert eng.cache.groups[1].pool.high_water >= 2
    from infinicore_infer_b200.trace import replay
    steps = tail_decode("r", toks, tail=len(toks))
    eng2 = _engine_for(cfg, spec, w, dtype)
    replay(eng2, steps)
    assert eng2.cache.groups[1].pool.high_water <= 12 // 8 + 2 < eng2.cache.groups[0].pool.high_water


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_run_order_a_layer_twice_and_a_layer_that_reads_anothers_cache(tiny_models, dtype):
    from infinicore_infer_b200.config import MiniCPMConfig, RunEntry
    _, cfg, w = tiny_models["A"]
    spec = MiniCPMConfig.from_dict(cfg).model_spec()
    order = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(1, 0, writes_cache=False))
    spec = replace(spec, order=order)
    eng = _engine_for(cfg, spec, w, dtype)
    assert len(eng.cache.views) == 3
    toks = random_tokens(22, 50, cfg["vocab_size"])
    want = plain_forward(cfg, w, toks, order=[(e.layer, e.cache, e.writes_cache) for e in order]).numpy()
    _replay_all(eng, toks, want, 3e-5 if dtype == torch.float32 else 2.5e-2, "order")
