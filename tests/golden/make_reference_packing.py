#!/usr/bin/env python3
"""Writes ``reference_packing.safetensors`` and ``reference_packing.json`` beside this file: what the REFERENCE's own
Python classes make of one very small random model, so that tests can hold this package's configuration reader and
weight packing against the reference on machines that do not have it.

    python tests/golden/make_reference_packing.py          (needs the reference's scripts and a C compiler)

``JiugeMetaFromLlama`` (scripts/jiuge.py:86-135) gives the sizes and the four scales, ``JiugeWeightsImpl``
(scripts/jiuge.py:139-352) the packed buffers: q and k rows permuted inside each head, q | k | v and gate | up fused,
o and down multiplied by scale_depth / sqrt(layers), the final norm by hidden // dim_model_base, the embedding by
scale_emb.  ``logits`` are a float64 pass over those buffers in the reference's conventions (the function
``forward_over_reference_buffers`` of tests/test_reference_anchor.py); the reference's C++ model itself cannot be
built here (it calls the external InfiniCore libraries), so no output of ITS forward pass exists to store.
The model's weights are not stored: ``state_dict()`` below makes them again from the seed.
"""
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CONFIG = dict(model_type="minicpm", num_hidden_layers=2, hidden_size=48, num_attention_heads=3, num_key_value_heads=1,
              intermediate_size=40, vocab_size=50, max_position_embeddings=32, rms_norm_eps=2e-6, rope_theta=5000.0,
              scale_emb=3.5, scale_depth=1.3, dim_model_base=16, tie_word_embeddings=False, eos_token_id=[2])
SEED, STD, NORM_STD = 11, 0.15, 0.05
TOKENS = [3, 41, 7, 7, 19, 0, 49, 23, 8, 30, 12, 5]


def state_dict():
    from infinicore_infer_b200.config import MiniCPMConfig
    from infinicore_infer_b200.parts import model_manifest
    from infinicore_infer_b200.weights import random_tensors
    typed = MiniCPMConfig.from_dict(CONFIG)
    return random_tensors(model_manifest(typed.model_spec()), SEED, STD, NORM_STD, matrix_dtype=torch.float32,
                          include_optional=True)


def write(jiuge, out_dir: str) -> None:
    """``jiuge``: the reference's scripts/jiuge.py, imported."""
    from infinicore_infer_b200.weights import write_file
    from test_reference_anchor import forward_over_reference_buffers, meta_dict, tensors_of
    meta = jiuge.JiugeMetaFromLlama(CONFIG, dtype=torch.float32)
    packed = jiuge.JiugeWeightsImpl(meta, jiuge.LlamaWeightsNaming(), state_dict(), torch_dt_mat=torch.float32,
                                    torch_dt_norm=torch.float32)
    w = tensors_of(packed)
    out = {}
    for k, v in w.items():
        if isinstance(v, list):
            out.update({f"{k}.{i}": t.contiguous() for i, t in enumerate(v)})
        else:
            out[k] = v.contiguous()
    out["logits"] = forward_over_reference_buffers(meta_dict(meta), w, TOKENS).float()
    write_file(os.path.join(out_dir, "reference_packing.safetensors"), out)
    record = {
        "meta": {k: int(getattr(meta, k)) for k in ("nlayer", "d", "nh", "nkvh", "dh", "di", "dctx", "dvoc")},
        "epsilon": float(meta.epsilon), "theta": float(meta.theta),
        "scales": {k: float(getattr(meta, k)) for k in ("scale_input", "scale_output", "scale_o", "scale_down")},
        "tokens": TOKENS,
    }
    with open(os.path.join(out_dir, "reference_packing.json"), "w") as f:
        json.dump(record, f, indent=1)


if __name__ == "__main__":
    import reference_scripts
    root = reference_scripts.stub_library(tempfile.mkdtemp())
    (jiuge,) = reference_scripts.import_reference(root)
    write(jiuge, HERE)
    print("written to", HERE)
