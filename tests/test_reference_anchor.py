"""This package held against the reference's OWN Python code, run here on the CPU.

The reference's model code is C++ over the external InfiniCore libraries and cannot be built on this machine; its
Python side can be imported given a stub library (see ``reference_scripts.py``).  What is pinned here, and by what:

* ``MiniCPMConfig``             against ``JiugeMetaFromLlama``  (scripts/jiuge.py:86-135): the eight sizes, eps, theta
                                and the four scales, for the tiny configurations and the 1B / 2B / 8B shapes;
* ``Attention.pack``, ``SwiGLU.pack`` and the model's scales
                                against ``JiugeWeightsImpl``    (scripts/jiuge.py:139-352): its q/k rows de-permuted
                                are our fused [q | k | v]; gate rows then up rows; its o and down are ours times the
                                residual scale; its final norm is ours times the logit scale; its embedding is ours
                                times the embedding scale; the output matrix falls back to the embedding and back;
* the plain implementation      against a forward pass over the reference's packed buffers in the reference's own
                                conventions (adjacent-pair rotation of permuted rows, scales inside the weights);
* ``tasks.InferTask / KVCache / KVCachePool``
                                against scripts/infer_task.py and scripts/kvcache_pool.py under one random sequence
                                of operations: equal positions, pending tokens, finish reasons, matches, records.

Everything skips cleanly where the reference's scripts are absent.  ``tests/golden/`` keeps the reference's packed
buffers of one very small model, so that the packing stays pinned on machines without the reference.
"""
import math
import os
import random

import pytest
import torch

from conftest import TINY, TINY_A, TINY_B, TINY_D
from plain_minicpm import plain_forward
import reference_scripts

from infinicore_infer_b200.config import MiniCPMConfig
from infinicore_infer_b200.parts import model_manifest, part_class
from infinicore_infer_b200.weights import DictWeights, random_tensors

SHAPES = {
    "1b": dict(model_type="minicpm", num_hidden_layers=52, hidden_size=1536, num_attention_heads=24, num_key_value_heads=8,
               intermediate_size=3840, vocab_size=73440, max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0,
               scale_emb=12, scale_depth=1.4, dim_model_base=256),
    "2b": dict(model_type="minicpm", num_hidden_layers=40, hidden_size=2304, num_attention_heads=36, num_key_value_heads=36,
               intermediate_size=5760, vocab_size=122753, max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0,
               scale_emb=12, scale_depth=1.4, dim_model_base=256),
    "8b": dict(model_type="fm9g", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=2,
               intermediate_size=16384, vocab_size=73448, max_position_embeddings=32768, rms_norm_eps=1e-5,
               scale_emb=12, scale_depth=1.4, dim_model_base=256),
    # the same graph with the scales at 1, heads without a key/value count, no theta: the reference's defaults
    "llama": dict(model_type="llama", num_hidden_layers=4, hidden_size=256, num_attention_heads=8, intermediate_size=688,
                  vocab_size=1000, max_position_embeddings=512, rms_norm_eps=1e-6, scale_emb=12, scale_depth=1.4,
                  dim_model_base=32),
    # a MiniCPM type without all three scale keys: no scale applies
    "half-scaled": dict(TINY_A, dim_model_base=None),
}
SHAPES["half-scaled"].pop("dim_model_base")


@pytest.fixture(scope="module")
def ref(tmp_path_factory):
    if reference_scripts.scripts_dir() is None:
        pytest.skip("the reference's scripts are not on this machine")
    try:
        root = reference_scripts.stub_library(str(tmp_path_factory.mktemp("infini_root")))
        jiuge, infer_task, kvcache_pool = reference_scripts.import_reference(root, ("jiuge", "infer_task", "kvcache_pool"))
    except Exception as e:       # noqa: BLE001 - a missing compiler or an import the machine lacks: nothing to anchor on
        pytest.skip(f"the reference's scripts do not import here: {e}")
    return jiuge, infer_task, kvcache_pool


def all_configs():
    out = {f"tiny-{n}": TINY[n][0] for n in ("A", "B", "D")}        # tiny-C sets head_dim, a key the reference never reads
    out.update(SHAPES)
    return out


@pytest.mark.parametrize("name", sorted(all_configs()))
def test_the_configuration_reads_what_the_reference_reads(ref, name):
    jiuge = ref[0]
    cfg = all_configs()[name]
    for max_tokens in (None, 77):
        meta = jiuge.JiugeMetaFromLlama(cfg, dtype=torch.float32, max_tokens=max_tokens)
        ours = MiniCPMConfig.from_dict(cfg, max_tokens=max_tokens)
        assert (meta.nlayer, meta.d, meta.nh, meta.nkvh, meta.dh, meta.di, meta.dctx, meta.dvoc) == (
            ours.num_hidden_layers, ours.hidden_size, ours.num_attention_heads, ours.num_key_value_heads, ours.head_dim,
            ours.intermediate_size, ours.max_position_embeddings, ours.vocab_size)
        assert meta.epsilon == pytest.approx(ours.rms_norm_eps, rel=1e-6)        # a C float on their side
        assert meta.theta == pytest.approx(ours.rope_theta, rel=1e-6)
        assert float(meta.scale_input) == ours.scale_emb
        assert float(meta.scale_output) == ours.logit_scale
        assert float(meta.scale_o) == ours.residual_scale and float(meta.scale_down) == ours.residual_scale
        spec = ours.model_spec()
        assert (spec.embed_scale, spec.logit_scale, spec.layers[0].residual_scale) == (
            float(meta.scale_input), float(meta.scale_output), float(meta.scale_o))


def reference_buffers(jiuge, cfg, state):
    meta = jiuge.JiugeMetaFromLlama(cfg, dtype=torch.float32)
    return meta, jiuge.JiugeWeightsImpl(meta, jiuge.LlamaWeightsNaming(), state, torch_dt_mat=torch.float32,
                                        torch_dt_norm=torch.float32)


def depermute(rows: torch.Tensor, heads: int, dh: int) -> torch.Tensor:
    """Undo scripts/jiuge.py:217-227: row 2j + s of a head came from row s * dh/2 + j."""
    return rows.reshape(heads, dh // 2, 2, -1).transpose(1, 2).reshape(heads * dh, -1)


def our_packing(cfg, state):
    typed = MiniCPMConfig.from_dict(cfg)
    spec = typed.model_spec()
    src = DictWeights(state, torch.float32, "cpu")
    layers = []
    for i, b in enumerate(spec.layers):
        p = spec.layer_prefix.format(i)
        one = dict(part_class("mixer", b.mixer).pack(b.mixer, src, p + b.mixer_prefix))
        one.update(part_class("feed_forward", b.feed_forward).pack(b.feed_forward, src, p + b.ffn_prefix))
        layers.append(one)
    return typed, spec, layers


def check_packing(cfg, state, w, nlayer):
    """``w``: the reference's tensors by the attribute names of JiugeWeightsImpl (lists per layer)."""
    typed, spec, layers = our_packing(cfg, state)
    nh, nkvh, dh, d = typed.num_attention_heads, typed.num_key_value_heads, typed.head_dim, typed.hidden_size
    s = typed.residual_scale
    for i in range(nlayer):
        theirs = w["qkv_tensor"][i].reshape((nh + 2 * nkvh) * dh, d)
        q, k, v = theirs[:nh * dh], theirs[nh * dh:(nh + nkvh) * dh], theirs[(nh + nkvh) * dh:]
        restored = torch.cat([depermute(q, nh, dh), depermute(k, nkvh, dh), v])
        assert torch.equal(restored, layers[i]["w_qkv"]), f"layer {i}: q | k | v"
        assert torch.equal(w["gate_up_tensors"][i], layers[i]["w_gate_up"]), f"layer {i}: gate | up"
        assert torch.allclose(w["attn_o_tensor"][i].reshape(d, nh * dh), layers[i]["w_o"] * s, rtol=1e-6, atol=0)
        assert torch.allclose(w["ffn_down_tensor"][i].reshape(d, -1), layers[i]["w_down"] * s, rtol=1e-6, atol=0)
    embed = state[spec.embed_name].float()
    assert torch.allclose(w["input_embd_tensor"], embed * typed.scale_emb, rtol=1e-6, atol=0)
    assert torch.allclose(w["output_norm_tensor"], state[spec.final_norm_prefix + "weight"].float() * typed.logit_scale,
                          rtol=1e-6, atol=0)
    head = state[spec.lm_head_name].float() if spec.lm_head_name in state else embed
    assert torch.equal(w["output_embd_tensor"], head)


def tensors_of(weights_impl) -> dict:
    return {k: getattr(weights_impl, k) for k in ("qkv_tensor", "gate_up_tensors", "attn_o_tensor", "ffn_down_tensor",
                                                  "input_embd_tensor", "output_norm_tensor", "output_embd_tensor",
                                                  "attn_norm_tensors", "ffn_norm_tensors")}


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_the_packed_weights_are_the_reference_s_up_to_its_permutation_and_folded_scales(ref, name):
    cfg, seed, std, norm_std = TINY[name]
    typed = MiniCPMConfig.from_dict(cfg)
    state = random_tensors(model_manifest(typed.model_spec()), seed, std, norm_std, matrix_dtype=torch.float32,
                           include_optional=not typed.tie_word_embeddings)
    meta, theirs = reference_buffers(ref[0], cfg, state)
    check_packing(cfg, state, tensors_of(theirs), typed.num_hidden_layers)


def test_the_output_matrix_falls_back_both_ways(ref):
    """scripts/jiuge.py:182-191: without ``lm_head.weight`` the embedding serves as output matrix, and a checkpoint that
    only has ``lm_head.weight`` feeds the embedding from it.  Ours does the first (one device copy); the second
    layout does not occur in this architecture's checkpoints and is refused by the manifest check."""
    cfg, seed, std, norm_std = TINY["A"]
    typed = MiniCPMConfig.from_dict(cfg)
    state = random_tensors(model_manifest(typed.model_spec()), seed, std, norm_std, matrix_dtype=torch.float32)
    assert "lm_head.weight" not in state
    _, theirs = reference_buffers(ref[0], cfg, state)
    assert torch.equal(theirs.output_embd_tensor, state["model.embed_tokens.weight"])
    only_head = dict(state)
    only_head["lm_head.weight"] = only_head.pop("model.embed_tokens.weight")
    _, theirs = reference_buffers(ref[0], cfg, only_head)
    assert torch.allclose(theirs.input_embd_tensor, only_head["lm_head.weight"] * typed.scale_emb)
    from infinicore_infer_b200.weights import WeightError, check_manifest
    with pytest.raises(WeightError, match="embed_tokens"):
        check_manifest(model_manifest(typed.model_spec()), {n: tuple(t.shape) for n, t in only_head.items()})


def forward_over_reference_buffers(meta, w, tokens, dtype=torch.float64):
    """One whole sequence through the reference's packed buffers, in the reference's conventions
    (src/models/jiuge/jiuge.cpp:164-264): embedding rows already scaled, query and key heads rotated in ADJACENT
    pairs (2j, 2j+1) because the loader permuted their rows, o and down already scaled, the logit scale inside the
    final norm's weight.  ``w``: tensors by the attribute names of JiugeWeightsImpl."""
    nh, nkvh, dh, d, di = meta["nh"], meta["nkvh"], meta["dh"], meta["d"], meta["di"]
    eps, theta = meta["epsilon"], meta["theta"]
    T = len(tokens)
    pos = torch.arange(T, dtype=torch.float64)

    def norm(x, weight):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(dtype)

    def rope_adjacent(x):
        j = torch.arange(dh // 2, dtype=torch.float64)
        ang = pos[:, None] / theta ** (j / (dh // 2))
        c, s = ang.cos()[:, None, :].to(dtype), ang.sin()[:, None, :].to(dtype)
        out = torch.empty_like(x)
        out[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s
        out[..., 1::2] = x[..., 0::2] * s + x[..., 1::2] * c
        return out

    x = w["input_embd_tensor"].to(dtype)[torch.as_tensor(list(tokens))]
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    for i in range(meta["nlayer"]):
        h = norm(x, w["attn_norm_tensors"][i])
        qkv = h @ w["qkv_tensor"][i].to(dtype).reshape((nh + 2 * nkvh) * dh, d).T
        q = rope_adjacent(qkv[:, :nh * dh].reshape(T, nh, dh))
        k = rope_adjacent(qkv[:, nh * dh:(nh + nkvh) * dh].reshape(T, nkvh, dh))
        v = qkv[:, (nh + nkvh) * dh:].reshape(T, nkvh, dh)
        o = torch.empty(T, nh, dh, dtype=dtype)
        for hq in range(nh):
            s = (q[:, hq] @ k[:, hq // (nh // nkvh)].T) / math.sqrt(dh)
            o[:, hq] = torch.softmax(s.masked_fill(~causal, float("-inf")), -1) @ v[:, hq // (nh // nkvh)]
        x = x + o.reshape(T, nh * dh) @ w["attn_o_tensor"][i].to(dtype).reshape(d, nh * dh).T
        h = norm(x, w["ffn_norm_tensors"][i])
        gu = h @ w["gate_up_tensors"][i].to(dtype).T
        g, u = gu[:, :di], gu[:, di:]
        x = x + ((g * torch.sigmoid(g)) * u) @ w["ffn_down_tensor"][i].to(dtype).reshape(d, di).T
    return norm(x, w["output_norm_tensor"]) @ w["output_embd_tensor"].to(dtype).T


def meta_dict(meta) -> dict:
    return {k: getattr(meta, k) for k in ("nlayer", "d", "nh", "nkvh", "dh", "di", "dctx", "dvoc", "epsilon", "theta")}


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_the_plain_implementation_agrees_with_a_pass_over_the_reference_s_buffers(ref, name):
    cfg, seed, std, norm_std = TINY[name]
    typed = MiniCPMConfig.from_dict(cfg)
    state = random_tensors(model_manifest(typed.model_spec()), seed, std, norm_std, matrix_dtype=torch.float32,
                           include_optional=not typed.tie_word_embeddings)
    meta, theirs = reference_buffers(ref[0], cfg, state)
    tokens = [random.Random(5).randrange(typed.vocab_size) for _ in range(40)]
    got = forward_over_reference_buffers(meta_dict(meta), tensors_of(theirs), tokens)
    want = plain_forward(typed.to_dict(), state, tokens)
    # the reference multiplies its scales into float32 weights: 2^-24 relative per weight, nothing more
    assert float((got - want).abs().max()) <= 2e-6 * float(want.abs().max())


# ---- the golden copy: the reference's buffers of one very small model ------------------------------------------
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_the_golden_copy_of_the_reference_s_buffers_still_matches_our_packing():
    """Runs without the reference: ``tests/golden/reference_packing.safetensors`` holds what JiugeWeightsImpl made of the
    small model that ``tests/golden/make_reference_packing.py`` defines, ``reference_packing.json`` what
    JiugeMetaFromLlama made of its configuration."""
    import json
    from infinicore_infer_b200.weights import index_directory, read_tensor
    import importlib.util
    spec_ = importlib.util.spec_from_file_location("make_reference_packing", os.path.join(GOLDEN, "make_reference_packing.py"))
    maker = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(maker)
    with open(os.path.join(GOLDEN, "reference_packing.json")) as f:
        gold = json.load(f)
    stored = {n: read_tensor(i) for n, i in index_directory(GOLDEN).items()}
    cfg = maker.CONFIG
    typed = MiniCPMConfig.from_dict(cfg)
    assert gold["meta"] == {"nlayer": typed.num_hidden_layers, "d": typed.hidden_size, "nh": typed.num_attention_heads,
                            "nkvh": typed.num_key_value_heads, "dh": typed.head_dim, "di": typed.intermediate_size,
                            "dctx": typed.max_position_embeddings, "dvoc": typed.vocab_size}
    assert gold["scales"] == {"scale_input": typed.scale_emb, "scale_output": typed.logit_scale,
                              "scale_o": typed.residual_scale, "scale_down": typed.residual_scale}
    state = maker.state_dict()
    L = typed.num_hidden_layers
    w = {k: [stored[f"{k}.{i}"] for i in range(L)] for k in ("qkv_tensor", "gate_up_tensors", "attn_o_tensor",
                                                              "ffn_down_tensor", "attn_norm_tensors", "ffn_norm_tensors")}
    w.update({k: stored[k] for k in ("input_embd_tensor", "output_norm_tensor", "output_embd_tensor")})
    check_packing(cfg, state, w, L)
    meta = dict(gold["meta"], epsilon=gold["epsilon"], theta=gold["theta"])
    got = forward_over_reference_buffers(meta, w, gold["tokens"])
    want = plain_forward(typed.to_dict(), state, gold["tokens"])
    assert float((got - want).abs().max()) <= 2e-6 * float(want.abs().max())
    assert torch.allclose(got.float(), stored["logits"], rtol=1e-5, atol=1e-5)


def test_the_golden_copy_is_what_the_reference_makes_today(ref, tmp_path):
    import importlib.util
    import json
    from infinicore_infer_b200.weights import index_directory, read_tensor
    spec_ = importlib.util.spec_from_file_location("make_reference_packing", os.path.join(GOLDEN, "make_reference_packing.py"))
    maker = importlib.util.module_from_spec(spec_)
    spec_.loader.exec_module(maker)
    maker.write(ref[0], str(tmp_path))
    old = {n: read_tensor(i) for n, i in index_directory(GOLDEN).items()}
    new = {n: read_tensor(i) for n, i in index_directory(str(tmp_path)).items()}
    assert sorted(old) == sorted(new)
    for n in old:
        if n != "logits":       # the logits come from a float64 pass: equal up to the platform's libm
            assert torch.equal(old[n], new[n]), n
    assert json.load(open(os.path.join(GOLDEN, "reference_packing.json"))) == json.load(open(tmp_path / "reference_packing.json"))


# ---- the request objects --------------------------------------------------------------------------------------
class FakeModel:
    """What KVCache and KVCachePool ask of a model (scripts/infer_task.py:39-47)."""

    def __init__(self, context):
        self.context, self.made, self.dropped = context, 0, []

    def max_context_len(self):
        return self.context

    def create_kv_cache(self):
        self.made += 1
        return self.made

    def drop_kv_cache(self, handle):
        self.dropped.append(handle)


@pytest.mark.parametrize("seed", range(6))
def test_request_objects_move_like_the_reference_s_under_random_operations(ref, seed, capsys):
    from infinicore_infer_b200 import tasks as ours
    _, their_task, their_pool = ref
    rng = random.Random(seed)
    context, max_caches, end_tokens = 24, 3, [7]
    stems = [[rng.randrange(10, 20) for _ in range(rng.randint(2, 9))] for _ in range(3)]

    sides = []
    for task_mod, pool_mod in ((ours, ours), (their_task, their_pool)):
        model = FakeModel(context)
        sides.append({"model": model, "pool": pool_mod.KVCachePool(model, max_caches), "Task": task_mod.InferTask,
                      "waiting": [], "running": [], "done": []})

    def snapshot(side):
        pool = side["pool"]
        return {
            "tasks": [(t.id, t.pos, list(t.tokens), t.finish_reason) for t in side["running"] + side["waiting"] + side["done"]],
            "pool": (pool.num_caches, [list(c.tokens) for c in pool._available], [c.data() for c in pool._available]),
            "model": (side["model"].made, list(side["model"].dropped)),
        }

    next_id = 0
    for _ in range(300):
        op = rng.random()
        if op < 0.25:                       # a new request, often sharing a stem with earlier ones
            stem = rng.choice(stems)
            prompt = stem[:rng.randint(1, len(stem))] + [rng.randrange(10, 20) for _ in range(rng.randint(0, 4))]
            limit = rng.choice([context, len(prompt) + rng.randint(0, 5)])
            for side in sides:
                side["waiting"].append(side["Task"](next_id, list(prompt), limit, 1.0, 1, 1.0, end_tokens))
            next_id += 1
        elif op < 0.5:                      # admit the oldest waiting request if the pool would not block
            for side in sides:
                pool = side["pool"]
                if side["waiting"] and (pool._available or pool.num_caches < pool.max_caches):
                    t = side["waiting"].pop(0)
                    pool.acquire_sync(t)
                    side["running"].append(t)
        elif sides[0]["running"]:           # one round: every running request gets a token
            outs = [rng.choice([7, None] + [rng.randrange(10, 20)] * 10) for _ in sides[0]["running"]]
            for side in sides:
                for t, tok in zip(list(side["running"]), outs):
                    t.next(tok)
                    if t.finish_reason is not None:
                        side["running"].remove(t)
                        side["pool"].release_sync(t)
                        side["done"].append(t)
        assert snapshot(sides[0]) == snapshot(sides[1])
    for side in sides:
        while side["running"]:
            t = side["running"].pop()
            side["pool"].release_sync(t)
        side["pool"].finalize()
    assert snapshot(sides[0]) == snapshot(sides[1])
    assert sorted(sides[0]["model"].dropped) == list(range(1, sides[0]["model"].made + 1))
    capsys.readouterr()
