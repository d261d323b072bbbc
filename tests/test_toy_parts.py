"""Parts defined in a test can be registered, built and stepped without a change to the framework:
a mixer with per-request state of its own, a feed-forward with routing, another position encoding."""
from dataclasses import dataclass, replace
from typing import Optional

import numpy as np
import pytest
import torch

from conftest import random_tokens
from plain_minicpm import plain_attention, plain_forward, plain_rmsnorm, plain_swiglu_ffn
from trace_helpers import by_position, mixed, portions, tail_decode, whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---- a toy mixer with state: the running mean of everything the request has fed so far ------------
@dataclass(frozen=True)
class RunningMeanSpec:
    hidden_size: int
    kind: str = "toy_running_mean"


def _register_toys():
    from infinicore_infer_b200.cache import StateSlot
    from infinicore_infer_b200.parts import register
    from infinicore_infer_b200.weights import MATRIX, TensorDecl

    @register("mixer", "toy_running_mean")
    class RunningMean:
        """out[t] = W @ mean(h[0..t]); the state is the running sum, one vector per request slot."""

        @staticmethod
        def tensor_decls(spec):
            return {"mix.weight": TensorDecl((spec.hidden_size, spec.hidden_size))}

        @staticmethod
        def cache_need(spec):
            return StateSlot((spec.hidden_size,), "float32")

        def __init__(self, spec, weights, prefix, runtime):
            self.w = weights.get(prefix + "mix.weight", MATRIX).float()

        def forward(self, h, ctx, view, writes_cache=True):
            # device-side only, so that a decode step can be replayed from a CUDA graph
            hf = h.float()
            row_req = ctx.row_req.long()
            slots = ctx.slot_ids.long()
            cs = torch.cumsum(hf, 0)
            seg0 = (cs - hf)[ctx.req_start.long()[:-1]]              # sum of the rows before each request
            running = cs - seg0[row_req] + view.state[slots][row_req]
            last = ctx.req_start.long()[1:] - 1
            view.state[slots] = running[last]
            mean = running / (ctx.positions.float() + 1)[:, None]
            return mean @ self.w.T


@dataclass(frozen=True)
class Top1RoutedSpec:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    kind: str = "toy_top1_experts"


def _register_routed():
    from infinicore_infer_b200.parts import register
    from infinicore_infer_b200.weights import MATRIX, TensorDecl

    @register("feed_forward", "toy_top1_experts")
    class Top1Experts:
        """A router picks one SwiGLU expert per token (router logits in float32)."""

        @staticmethod
        def tensor_decls(spec):
            d, di, e = spec.hidden_size, spec.intermediate_size, spec.num_experts
            out = {"router.weight": TensorDecl((e, d))}
            for i in range(e):
                out.update({f"experts.{i}.gate.weight": TensorDecl((di, d)), f"experts.{i}.up.weight": TensorDecl((di, d)),
                            f"experts.{i}.down.weight": TensorDecl((d, di))})
            return out

        def __init__(self, spec, weights, prefix, runtime):
            self.spec = spec
            g = lambda n: weights.get(prefix + n, MATRIX).float()
            self.router = g("router.weight")
            self.experts = [(g(f"experts.{i}.gate.weight"), g(f"experts.{i}.up.weight"), g(f"experts.{i}.down.weight"))
                            for i in range(spec.num_experts)]

        def forward(self, h, ctx):
            hf = h.float()
            choice = (hf @ self.router.T).argmax(-1)
            out = torch.zeros_like(hf)
            for i, (g, u, d) in enumerate(self.experts):
                a = hf @ g.T
                y = (a * torch.sigmoid(a) * (hf @ u.T)) @ d.T
                out = torch.where((choice == i)[:, None], y, out)
            return out


@dataclass(frozen=True)
class AlibiLikeSpec:
    """A position encoding that is not rotary: a learned-free additive ramp on the queries."""
    head_dim: int
    max_positions: int
    slope: float = 0.01
    interleaved: bool = False
    kind: str = "toy_scaled_rope"
    theta: float = 10000.0


def _register_position():
    from infinicore_infer_b200.parts import register

    @register("position", "toy_scaled_rope")
    class ScaledRotary:
        """Rotary tables whose angles are stretched by a constant: another encoding, same interface."""

        @staticmethod
        def tensor_decls(spec):
            return {}

        def __init__(self, spec, weights, prefix, runtime):
            half = spec.head_dim // 2
            j = torch.arange(half, dtype=torch.float64)
            ang = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * spec.slope / spec.theta ** (j / half)
            self.cos = ang.cos().float().to(runtime.device)
            self.sin = ang.sin().float().to(runtime.device)
            self.interleaved = False


def _toy_model(cfg, typed):
    """Layer 0: running-mean mixer + routed experts.  Layer 1: attention with the stretched rotary + SwiGLU."""
    spec = typed.model_spec()
    l0, l1 = spec.layers[0], spec.layers[1]
    toy0 = replace(l0, mixer=RunningMeanSpec(spec.hidden_size),
                   feed_forward=Top1RoutedSpec(spec.hidden_size, 24, 3))
    pos = AlibiLikeSpec(head_dim=l1.mixer.head_dim, max_positions=spec.max_positions, slope=0.37,
                        theta=l1.mixer.position.theta)
    toy1 = replace(l1, mixer=replace(l1.mixer, position=pos))
    return replace(spec, layers=(toy0, toy1))


def _plain_toy(cfg, w, toks):
    """The toy model, whole sequence, plain torch in float64."""
    from plain_minicpm import plain_embedding, plain_scales
    W = {k: v.double() for k, v in w.items()}
    d, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    dh = d // nh
    se, sr, sl = plain_scales(cfg)
    T = len(toks)
    x = plain_embedding(torch.tensor(toks), W["model.embed_tokens.weight"], se)
    p = "model.layers.0."
    h = plain_rmsnorm(x, W[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    x = x + sr * (mean @ W[p + "self_attn.mix.weight"].T)
    h = plain_rmsnorm(x, W[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    choice = (h @ W[p + "mlp.router.weight"].T).argmax(-1)
    y = torch.stack([plain_swiglu_ffn(h[t:t + 1], W[p + f"mlp.experts.{int(c)}.gate.weight"],
                                      W[p + f"mlp.experts.{int(c)}.up.weight"],
                                      W[p + f"mlp.experts.{int(c)}.down.weight"])[0] for t, c in enumerate(choice)])
    x = x + sr * y
    p = "model.layers.1."
    h = plain_rmsnorm(x, W[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    half = dh // 2
    j = torch.arange(half, dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * 0.37 / cfg["rope_theta"] ** (j / half)
    def rot(t):
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        return torch.cat([t[..., :half] * c - t[..., half:] * s, t[..., :half] * s + t[..., half:] * c], -1)
    q = rot((h @ W[p + "self_attn.q_proj.weight"].T).view(T, nh, dh))
    k = rot((h @ W[p + "self_attn.k_proj.weight"].T).view(T, nh, dh))
    v = (h @ W[p + "self_attn.v_proj.weight"].T).view(T, nh, dh)
    o = plain_attention(q, k, v, dh ** -0.5).reshape(T, d) @ W[p + "self_attn.o_proj.weight"].T
    x = x + sr * o
    h = plain_rmsnorm(x, W[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + sr * plain_swiglu_ffn(h, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])
    h = plain_rmsnorm(x, W["model.norm.weight"], cfg["rms_norm_eps"]) * sl
    return (h @ W["model.embed_tokens.weight"].T).numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_parts_are_registered_built_and_stepped(dtype):
    from conftest import TINY_A
    from infinicore_infer_b200.cache import StateSlot
    from infinicore_infer_b200.config import MiniCPMConfig
    from infinicore_infer_b200.engine import Engine
    from infinicore_infer_b200.parts import cache_needs, model_manifest
    from infinicore_infer_b200.trace import replay
    from infinicore_infer_b200.weights import DictWeights, random_tensors
    _register_toys(); _register_routed(); _register_position()
    cfg = dict(TINY_A)
    spec = _toy_model(cfg, MiniCPMConfig.from_dict(cfg))
    needs = cache_needs(spec)
    assert isinstance(needs[0], StateSlot) and needs[1].num_kv_heads == 4
    manifest = model_manifest(spec)
    assert "model.layers.0.self_attn.mix.weight" in manifest and "model.layers.0.mlp.experts.2.down.weight" in manifest
    w = {k: v.float() for k, v in random_tensors(manifest, seed=5, std=0.125).items()}
    eng = Engine(spec, DictWeights(w, dtype, DEV), dtype=dtype, device=DEV, cache_tokens=256, page_size=8,
                 max_requests=4, max_step_tokens=256)
    assert eng.cache.views[0].state.shape == (5, 64)
    # the toy parts run by their own forward between the records; the standard parts around them (the norms, layer 1's
    # attention with the toy position encoding's tables, its SwiGLU) are launch records of the native step
    assert eng.program.launch_list() == [
        "embed", "norm", "host:RunningMean.forward", "norm", "host:Top1Experts.forward",
        "norm", "qkv", "attention", "residual", "norm", "gate_up", "residual", "norm", "linear"]
    tol = 3e-5 if dtype == torch.float32 else 2.5e-2
    reqs = {r: random_tokens(30 + i, n, cfg["vocab_size"]) for i, (r, n) in enumerate({"a": 40, "b": 23, "c": 31}.items())}
    wants = {r: _plain_toy(cfg, w, t) for r, t in reqs.items()}

    def check(steps, what):
        got = by_position(steps, replay(eng, steps))
        for (r, p), row in got.items():
            want = wants[r]
            err = np.abs(row - want[p]).max()
            assert err <= tol * np.abs(want).max(), f"{what}: {r} position {p}: {err:.3e}"

    if dtype == torch.float32:
        check(whole("a", reqs["a"]), "whole")
        check(tail_decode("a", reqs["a"], tail=20), "tail")       # state carried across single tokens (graph replays)
        check(portions("a", reqs["a"], sizes=(5, 2, 9)), "portions")
        plan = [{"a": 17}, {"a": 3, "b": 20}, {"a": 1, "b": 1, "c": 9}, {"a": 1, "b": 1, "c": 2}, {"a": 18, "b": 1, "c": 20}]
        check(mixed(reqs, plan), "mixed")                          # slots are given back and taken again
    else:
        # bfloat16: the experts' router may tip on near-ties, so only the cuts' agreement with each
        # other is asked for here (same kernels, same roundings)
        a = by_position(whole("a", reqs["a"]), replay(eng, whole("a", reqs["a"])))
        b = by_position(portions("a", reqs["a"], sizes=(5, 2, 9)), replay(eng, portions("a", reqs["a"], sizes=(5, 2, 9))))
        diff = max(np.abs(a[k] - b[k]).max() for k in a)
        assert diff <= 2.5e-2 * np.abs(wants["a"]).max()
    assert not eng.cache.lengths and eng.cache.slots.available == 4
