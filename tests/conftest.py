"""Shared test set-up: the ``gpu`` marker, tiny configurations, model folders in temp dirs."""
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations of the architecture that differ in every size and option, and a
# third with sizes that are no power of two at all (odd vocabulary, head size 48 != hidden/heads).
TINY_A = dict(
    model_type="minicpm", architectures=["MiniCPMForCausalLM"], num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=4, intermediate_size=160, vocab_size=256,
    max_position_embeddings=320, rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4,
    dim_model_base=16, tie_word_embeddings=True, eos_token_id=2)
TINY_B = dict(
    model_type="fm9g", num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1,
    intermediate_size=224, vocab_size=384, max_position_embeddings=416, rms_norm_eps=1e-6,
    rope_theta=1000000.0, scale_emb=2.5, scale_depth=1.0, dim_model_base=48, tie_word_embeddings=False,
    eos_token_id=[1, 5])
TINY_C = dict(
    model_type="minicpm", num_hidden_layers=2, hidden_size=80, num_attention_heads=6, num_key_value_heads=2,
    head_dim=48, intermediate_size=136, vocab_size=301, max_position_embeddings=288, rms_norm_eps=3e-6,
    rope_theta=50000.0, scale_emb=7.0, scale_depth=2.1, dim_model_base=20, tie_word_embeddings=True)
# A fourth with heads of 64, the size for which the tcgen05 attention kernel and the fused q/k/v epilogue
# of the tcgen05 product are built (grouped heads 2:1).
TINY_D = dict(
    model_type="minicpm", num_hidden_layers=2, hidden_size=128, num_attention_heads=2, num_key_value_heads=1,
    intermediate_size=192, vocab_size=333, max_position_embeddings=448, rms_norm_eps=1e-5,
    rope_theta=20000.0, scale_emb=5.0, scale_depth=1.7, dim_model_base=32, tie_word_embeddings=True)
# A fifth with biases on the query, key and value projections (the reference's optional ``attn_qkv_b``, scripts/jiuge.py:252-282)
# and heads of 64 grouped 2:1.
TINY_E = dict(
    model_type="fm9g", num_hidden_layers=2, hidden_size=128, num_attention_heads=2, num_key_value_heads=1,
    intermediate_size=160, vocab_size=270, max_position_embeddings=384, rms_norm_eps=2e-5, rope_theta=30000.0,
    scale_emb=6.0, scale_depth=1.5, dim_model_base=64, tie_word_embeddings=False, attention_bias=True)
# Matrices are N(0, std) with std near 1/sqrt(hidden): every product keeps its input's variance, so
# attention scores spread over several units (a sharp softmax) and a wrong key, page or position
# moves the logits far beyond any tolerance.  (With N(0, 0.02) scores are all near zero, every
# softmax is flat, and dropping one key among hundreds would hide inside the rounding.)
TINY = {"A": (TINY_A, 0, 0.125, 0.01), "B": (TINY_B, 1, 0.1, 0.02), "C": (TINY_C, 2, 0.11, 0.03),
        "D": (TINY_D, 3, 0.09, 0.02), "E": (TINY_E, 4, 0.09, 0.02)}


def make_folder(tmp_path_factory, name):
    """Write config.json + model.safetensors of a tiny configuration; return (dir, cfg dict, weights)."""
    from infinicore_infer_b200.config import config_class_for
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    cfg, seed, std, norm_std = TINY[name]
    d = str(tmp_path_factory.mktemp(f"tiny_{name}"))
    typed = config_class_for(cfg).from_dict(cfg)
    write_model_folder(typed, d, seed=seed, std=std, norm_std=norm_std)
    with open(os.path.join(d, "config.json")) as f:
        cfg_disk = json.load(f)
    weights = {n: read_tensor(i).float() for n, i in index_directory(d).items()}
    return d, cfg_disk, weights


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    return {name: make_folder(tmp_path_factory, name) for name in TINY}


def random_tokens(seed, n, vocab):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
