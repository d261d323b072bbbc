"""One registry from an architecture's name to its configuration class.

The reference dispatches on ``config["model_type"]`` with an if/elif chain
(scripts/jiuge.py:422-502).  Here the chain is a dictionary; a configuration
class is anything with ``from_dict(dict, max_tokens=None)`` and
``model_spec() -> ModelSpec``.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

from .specs import ConfigError

_ARCHITECTURES: Dict[str, type] = {}


def register_architecture(name: str, config_cls: type) -> None:
    _ARCHITECTURES[name.lower()] = config_cls


def architecture_names():
    return sorted(_ARCHITECTURES)


def config_class_for(cfg: dict) -> type:
    """Look the architecture up by ``model_type``, then by ``architectures``."""
    keys = []
    if cfg.get("model_type"):
        keys.append(str(cfg["model_type"]))
    keys.extend(str(a) for a in cfg.get("architectures") or ())
    for k in keys:
        cls = _ARCHITECTURES.get(k.lower())
        if cls is not None:
            return cls
    raise ConfigError(
        f"Unsupported model architecture {keys or '(config.json names none)'}; "
        f"registered: {', '.join(architecture_names())}")


def read_config(model_dir: str, max_tokens: Optional[int] = None):
    """Parse ``model_dir/config.json`` into the typed configuration of its architecture."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path) as f:
        cfg = json.load(f)
    return config_class_for(cfg).from_dict(cfg, max_tokens=max_tokens)
