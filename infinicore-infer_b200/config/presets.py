"""Named configurations for the random-weights mode: config.json contents as data, not sizes in code.

``tiny-A`` and ``tiny-B`` are two small configurations of the architecture that differ in every size and option
(multi-head against grouped heads 3:1, tied against untied embeddings, every scale, eps and theta); ``1b``, ``2b``
and ``8b`` have the layer sizes of MiniCPM-1B, MiniCPM-2B and an FM9G/MiniCPM4-8B-class model.  Each entry gives
the keys of a config.json of this architecture (the ones ``MiniCPMConfig.from_dict`` reads) and the spread of its
random weights: matrices N(0, std), norm weights 1 + N(0, norm_std).  The reference has no random mode.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict


@dataclass(frozen=True)
class Preset:
    config: dict
    std: float
    norm_std: float
    page_size: int          # the cache page this configuration is meant to run with


PRESETS: Dict[str, Preset] = {
    "tiny-A": Preset(dict(model_type="minicpm", num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                          num_key_value_heads=4, intermediate_size=160, vocab_size=256, max_position_embeddings=64,
                          rms_norm_eps=1e-5, rope_theta=1e4, scale_emb=12, scale_depth=1.4, dim_model_base=16,
                          tie_word_embeddings=True, eos_token_id=2), 0.02, 0.01, 16),
    "tiny-B": Preset(dict(model_type="fm9g", num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
                          num_key_value_heads=1, intermediate_size=224, vocab_size=384, max_position_embeddings=96,
                          rms_norm_eps=1e-6, rope_theta=1e6, scale_emb=2.5, scale_depth=1.0, dim_model_base=48,
                          tie_word_embeddings=False, eos_token_id=2), 0.03, 0.02, 8),
    "1b": Preset(dict(model_type="minicpm", num_hidden_layers=52, hidden_size=1536, num_attention_heads=24,
                      num_key_value_heads=8, intermediate_size=3840, vocab_size=73440, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                      tie_word_embeddings=True, eos_token_id=2), 0.02, 0.01, 16),
    "2b": Preset(dict(model_type="minicpm", num_hidden_layers=40, hidden_size=2304, num_attention_heads=36,
                      num_key_value_heads=36, intermediate_size=5760, vocab_size=122753, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                      tie_word_embeddings=True, eos_token_id=2), 0.02, 0.01, 16),
    "8b": Preset(dict(model_type="fm9g", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                      num_key_value_heads=2, intermediate_size=16384, vocab_size=73448, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                      tie_word_embeddings=False, eos_token_id=2), 0.02, 0.01, 16),
}
