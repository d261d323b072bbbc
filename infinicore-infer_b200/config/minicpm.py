"""The MiniCPM / FM9G configuration, read from the keys of its config.json.

The reference reads these keys in ``JiugeMetaFromLlama``
(scripts/jiuge.py:86-136).  ``llama`` is the same decoder with the three
MiniCPM scales at 1 (scripts/jiuge.py:97-114: the scales apply only when
``model_type`` is ``fm9g`` or ``minicpm`` and all three keys are present).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Optional, Tuple

from .specs import (AttentionSpec, BlockSpec, ConfigError, ModelSpec, RMSNormSpec,
                    RopeSpec, SwiGLUSpec, default_order)

# rope_theta when config.json has none (scripts/jiuge.py:133).
_REFERENCE_DEFAULT_THETA = 100000.0

_REQUIRED = ("num_hidden_layers", "hidden_size", "num_attention_heads",
             "intermediate_size", "max_position_embeddings", "vocab_size", "rms_norm_eps")


@dataclass(frozen=True)
class MiniCPMConfig:
    model_type: str
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    scale_emb: float
    scale_depth: Optional[float]
    dim_model_base: Optional[int]
    tie_word_embeddings: bool
    attention_bias: bool
    eos_token_id: Tuple[int, ...]
    logit_scale_override: Optional[float] = None

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, max_tokens: Optional[int] = None) -> "MiniCPMConfig":
        missing = [k for k in _REQUIRED if k not in cfg]
        if missing:
            raise ConfigError("config.json lacks the keys: " + ", ".join(missing))
        model_type = cfg.get("model_type", "minicpm")
        d = _pos_int(cfg, "hidden_size")
        nh = _pos_int(cfg, "num_attention_heads")
        nkvh = _pos_int(cfg, "num_key_value_heads") if cfg.get("num_key_value_heads") else nh
        if nh % nkvh:
            raise ConfigError(f"num_attention_heads {nh} is no multiple of num_key_value_heads {nkvh}")
        if cfg.get("head_dim"):
            dh = _pos_int(cfg, "head_dim")
        else:
            if d % nh:
                raise ConfigError(f"hidden_size {d} is no multiple of num_attention_heads {nh}")
            dh = d // nh  # scripts/jiuge.py:126
        if dh % 2:
            raise ConfigError(f"head size {dh} is odd; rotary pairs need an even size")
        scaled = (model_type in ("fm9g", "minicpm") and "scale_emb" in cfg
                  and "scale_depth" in cfg and "dim_model_base" in cfg)
        eos = cfg.get("eos_token_id", ())
        if eos is None:
            eos = ()
        if isinstance(eos, int):
            eos = (eos,)
        ctx = _pos_int(cfg, "max_position_embeddings") if max_tokens is None else int(max_tokens)
        if cfg.get("rope_scaling"):
            raise ConfigError("rope_scaling is not supported: the reference builds plain tables only")
        return cls(
            model_type=model_type,
            num_hidden_layers=_pos_int(cfg, "num_hidden_layers"),
            hidden_size=d,
            num_attention_heads=nh,
            num_key_value_heads=nkvh,
            head_dim=dh,
            intermediate_size=_pos_int(cfg, "intermediate_size"),
            max_position_embeddings=ctx,
            vocab_size=_pos_int(cfg, "vocab_size"),
            rms_norm_eps=float(cfg["rms_norm_eps"]),
            rope_theta=float(cfg.get("rope_theta", _REFERENCE_DEFAULT_THETA)),
            scale_emb=float(cfg["scale_emb"]) if scaled else 1.0,
            scale_depth=float(cfg["scale_depth"]) if scaled else None,
            dim_model_base=int(cfg["dim_model_base"]) if scaled else None,
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            attention_bias=bool(cfg.get("attention_bias", False)),
            eos_token_id=tuple(int(e) for e in eos),
            logit_scale_override=(float(cfg["logit_scale"]) if "logit_scale" in cfg else None),
        )

    def to_dict(self) -> dict:
        """config.json keys that read back to this configuration."""
        out = asdict(self)
        out.pop("logit_scale_override")
        if self.logit_scale_override is not None:
            out["logit_scale"] = self.logit_scale_override
        if self.scale_depth is None:
            for k in ("scale_emb", "scale_depth", "dim_model_base"):
                out.pop(k)
        out["eos_token_id"] = list(self.eos_token_id)
        out["architectures"] = ["MiniCPMForCausalLM" if self.model_type != "llama" else "LlamaForCausalLM"]
        return out

    # ---- the three scales (scripts/jiuge.py:101-114) ---------------------------------
    @property
    def residual_scale(self) -> float:
        if self.scale_depth is None:
            return 1.0
        return self.scale_depth / math.sqrt(self.num_hidden_layers)

    @property
    def logit_scale(self) -> float:
        """The reference multiplies the final norm's weight by hidden // dim_model_base."""
        if self.logit_scale_override is not None:
            return self.logit_scale_override
        if self.dim_model_base is None:
            return 1.0
        return float(self.hidden_size // self.dim_model_base)

    # ---- the model as parts ------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        rope = RopeSpec(head_dim=self.head_dim, theta=self.rope_theta,
                        max_positions=self.max_position_embeddings)
        attn = AttentionSpec(hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                             num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                             softmax_scale=1.0 / math.sqrt(self.head_dim),  # jiuge.cpp:223
                             position=rope, window=None, bias=self.attention_bias)
        ffn = SwiGLUSpec(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)
        norm = RMSNormSpec(size=self.hidden_size, eps=self.rms_norm_eps)
        block = BlockSpec(mixer=attn, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm,
                          residual_scale=self.residual_scale)
        return ModelSpec(
            architecture=self.model_type,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            layers=tuple(block for _ in range(self.num_hidden_layers)),
            order=default_order(self.num_hidden_layers),
            final_norm=norm,
            embed_scale=self.scale_emb,
            logit_scale=self.logit_scale,
            tie_embeddings=self.tie_word_embeddings,
            eos_token_ids=self.eos_token_id,
        )


def _pos_int(cfg: dict, key: str) -> int:
    v = cfg[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or v <= 0:
        raise ConfigError(f"config.json key {key} must be a positive integer, found {v!r}")
    return int(v)
