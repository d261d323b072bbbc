"""Long contexts: prompts of thousands of tokens in portions, then batched decoding under CUDA graphs, against the
plain implementation.  At these lengths the decode attention cuts each row's keys into several blocks: for heads of
64 up to eight cuts merge inside a thread-block cluster through distributed shared memory, more cuts (and every cut
of heads of 128) through partial results in scratch memory and a merge kernel.  The tiny configurations elsewhere
never reach two cuts, so this file is where those paths run inside a whole model."""
import numpy as np
import pytest
import torch

from conftest import random_tokens
from plain_minicpm import plain_forward
from trace_helpers import by_position

pytestmark = pytest.mark.gpu

# two layers, heads of 64 (grouped 2:1) and heads of 128 (grouped 4:1); matrices N(0, 1/sqrt(hidden)) so that the
# softmax is sharp and a lost key, page or cut moves the logits far beyond the tolerance
LONG = {
    "h64": (dict(model_type="minicpm", num_hidden_layers=2, hidden_size=128, num_attention_heads=2, num_key_value_heads=1,
                 intermediate_size=192, vocab_size=333, max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=20000.0,
                 scale_emb=5.0, scale_depth=1.7, dim_model_base=32, tie_word_embeddings=True), 0.09),
    "h64-8k": (dict(model_type="minicpm", num_hidden_layers=2, hidden_size=128, num_attention_heads=2, num_key_value_heads=2,
                    intermediate_size=160, vocab_size=301, max_position_embeddings=8192, rms_norm_eps=1e-6, rope_theta=1e6,
                    scale_emb=4.0, scale_depth=1.2, dim_model_base=64, tie_word_embeddings=True), 0.09),
    "h128": (dict(model_type="fm9g", num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=1,
                  head_dim=128, intermediate_size=320, vocab_size=290, max_position_embeddings=4096, rms_norm_eps=1e-5,
                  rope_theta=10000.0, scale_emb=3.0, scale_depth=1.4, dim_model_base=128, tie_word_embeddings=False), 0.0625),
}
TOL = {"float32": 3e-5, "bfloat16": 2.5e-2}


@pytest.fixture(scope="module")
def long_models(tmp_path_factory):
    from infinicore_infer_b200.config import MiniCPMConfig
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    out = {}
    for name, (cfg, std) in LONG.items():
        d = str(tmp_path_factory.mktemp(f"long_{name}"))
        write_model_folder(MiniCPMConfig.from_dict(cfg), d, seed=len(name), std=std, norm_std=0.02)
        out[name] = (d, cfg, {n: read_tensor(i).float() for n, i in index_directory(d).items()})
    return out


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", list(LONG))
def test_three_long_requests_in_portions_then_decoded_together(long_models, name, dtype):
    from infinicore_infer_b200 import kernels
    from infinicore_infer_b200.kernels import host
    from infinicore_infer_b200.engine import Engine
    from infinicore_infer_b200.trace import replay
    folder, cfg, w = long_models[name]
    # the longest request decides the context that a decode step is planned for: beyond 4,096 tokens the model with a
    # context of 8,192 cuts its rows' keys more than eight ways
    prompt_len, decoded = {"a": 5000 if name == "h64-8k" else 3000, "b": 2200, "c": 2913}, 64
    toks = {r: random_tokens(40 + i, n + decoded, cfg["vocab_size"]) for i, (r, n) in enumerate(prompt_len.items())}
    eng = Engine.from_folder(folder, dtype=getattr(torch, dtype), cache_tokens=sum(prompt_len.values()) + 3 * (decoded + 16) + 64, page_size=16, max_requests=4,
                             max_step_tokens=1024)
    if dtype == "bfloat16":
        a = eng.spec.layers[0].mixer
        context = host.context_bucket(prompt_len["a"] + 64, eng.spec.max_positions)
        splits = host.decode_splits(4, a.num_kv_heads, a.num_heads // a.num_kv_heads, context, 0, kernels._sm_count(eng.device), a.head_dim)
        assert splits >= 2 and (splits > 8) == (name == "h64-8k")
        assert eng.use_graphs and eng.program.native_only
    # prompts in 512-token portions, two requests' portions side by side where both still have some; the last rows of a
    # portion and a few inside it are wanted
    steps, done, s = [], {r: 0 for r in toks}, 0
    while any(done[r] < prompt_len[r] for r in toks):
        entries = []
        for r in toks:
            n = min(512, prompt_len[r] - done[r])
            if n > 0 and len(entries) < 2:
                entries.append({"id": r, "tokens": toks[r][done[r]:done[r] + n], "want": sorted({0, n // 3, n - 1})})
                done[r] += n
        steps.append({"step": s, "entries": entries, "end": []})
        s += 1
    for t in range(decoded):
        steps.append({"step": s, "entries": [{"id": r, "tokens": [toks[r][prompt_len[r] + t]], "want": [0]} for r in toks],
                      "end": list(toks) if t == decoded - 1 else []})
        s += 1
    got = by_position(steps, replay(eng, steps))
    eng.check()
    if dtype == "bfloat16":
        assert any(bucket == 4 for bucket, _ in eng._graphs)     # the decode steps ran as the captured graph of the bucket of 4
    for r in toks:
        want = plain_forward(cfg, w, toks[r]).numpy()
        scale = np.abs(want).max()
        mine = sorted(p for (rid, p) in got if rid == r)
        assert len(mine) >= 3 * (prompt_len[r] // 512) + decoded
        for p in mine:
            err = np.abs(got[(r, p)].astype(np.float64) - want[p]).max()
            assert err <= TOL[dtype] * scale, f"{name} {dtype} request {r} position {p}: {err:.3e} > {TOL[dtype] * scale:.3e}"
