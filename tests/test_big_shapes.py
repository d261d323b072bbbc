"""The engine at the benchmark's layer sizes (the 2B, 1B and 8B-class shapes with one or two layers) against the plain
float64 implementation on the same weights: the bfloat16 path, which at these sizes runs the tcgen05 product kernel,
the tensor-core prefill attention and the weight-streaming decode kernels, and the float32 path."""
import numpy as np
import pytest
import torch

from conftest import random_tokens
from plain_minicpm import plain_forward
from trace_helpers import by_position, mixed

pytestmark = pytest.mark.gpu

SHAPES = {
    "2b": dict(model_type="minicpm", num_hidden_layers=2, hidden_size=2304, num_attention_heads=36,
               num_key_value_heads=36, intermediate_size=5760, vocab_size=122753, max_position_embeddings=1024,
               rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
               tie_word_embeddings=True),
    "1b-gqa": dict(model_type="minicpm", num_hidden_layers=2, hidden_size=1536, num_attention_heads=24,
                   num_key_value_heads=8, intermediate_size=3840, vocab_size=73440, max_position_embeddings=1024,
                   rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                   tie_word_embeddings=True),
    "8b-class": dict(model_type="fm9g", num_hidden_layers=1, hidden_size=4096, num_attention_heads=32,
                     num_key_value_heads=2, intermediate_size=16384, vocab_size=73448, max_position_embeddings=1024,
                     rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                     tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", list(SHAPES))
def test_both_precisions_agree_with_the_plain_implementation_at_the_benchmark_sizes(name):
    from infinicore_infer_b200.config import MiniCPMConfig
    from infinicore_infer_b200.engine import Engine
    from infinicore_infer_b200.parts import model_manifest
    from infinicore_infer_b200.trace import replay
    from infinicore_infer_b200.weights import DeviceRandomWeights
    cfg = MiniCPMConfig.from_dict(SHAPES[name])
    spec = cfg.model_spec()
    V = cfg.vocab_size
    reqs = {"a": random_tokens(1, 300, V), "b": random_tokens(2, 70, V), "c": random_tokens(3, 9, V)}
    # a long portion (many rows: tcgen05), short ones and single tokens (few rows: weight streaming), mixed
    plan = [{"a": 280}, {"a": 1, "b": 64}, {"a": 1, "b": 1, "c": 9}] + [{"a": 1, "b": 1}] * 5 + [{"a": 13}]
    steps = mixed(reqs, plan)
    for s in steps:                                    # logits of each entry's last token only
        for e in s["entries"]:
            e["want"] = [len(e["tokens"]) - 1]
    out = {}
    for dtype in (torch.float32, torch.bfloat16):
        weights = DeviceRandomWeights(model_manifest(spec), seed=7, compute_dtype=dtype, device="cuda:0",
                                      std=0.03, norm_std=0.02, untied=not cfg.tie_word_embeddings)
        eng = Engine(spec, weights, dtype=dtype, cache_tokens=1024, page_size=16, max_requests=4, max_step_tokens=512)
        out[dtype] = by_position(steps, replay(eng, steps))
        del eng, weights
        torch.cuda.empty_cache()
    # the same weights on the host, in float64 (what the generator made, rounded to bfloat16 as a checkpoint holds it)
    from infinicore_infer_b200.weights import MATRIX, VECTOR
    source = DeviceRandomWeights(model_manifest(spec), seed=7, compute_dtype=torch.float32, device="cuda:0",
                                 std=0.03, norm_std=0.02, untied=not cfg.tie_word_embeddings)
    w = {n: source.get(n, VECTOR if len(d.shape) == 1 else MATRIX).double().cpu()
         for n, d in model_manifest(spec).items() if source.has(n)}
    del source
    torch.cuda.empty_cache()
    keys = sorted(out[torch.float32])
    assert set(keys) == set(out[torch.bfloat16]) and len(keys) >= 12
    want = {}
    for r in reqs:
        rows = [p for (rid, p) in keys if rid == r]
        logits = plain_forward(cfg.to_dict(), w, reqs[r], rows=rows).numpy()
        want.update({(r, p): logits[i] for i, p in enumerate(rows)})
    scale = max(np.abs(v).max() for v in want.values())
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 2.5e-2)):
        for key in keys:
            err = np.abs(out[dtype][key].astype(np.float64) - want[key]).max()
            assert err <= tol * scale, f"{name} {dtype} {key}: {err:.3e} > {tol * scale:.3e}"
