"""Parts of a model: norm, position encoding, mixer, feed-forward, block; and the model built of them."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, ResidualStream, Runtime, StepContext, part_class,
                   register)
from .program import HostIO, Program, ProgramRunner
from .norm import RMSNorm
from .rope import RotaryTables
from .attention import Attention
from .feed_forward import SwiGLU
from .block import PreNormBlock
from .model import Model, cache_needs, model_manifest

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "ResidualStream", "Runtime", "StepContext", "Program",
           "ProgramRunner", "HostIO", "part_class", "register", "RMSNorm", "RotaryTables", "Attention", "SwiGLU",
           "PreNormBlock", "Model", "cache_needs", "model_manifest"]
