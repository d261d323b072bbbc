"""A small, whole, single-GPU inference engine for the MiniCPM/FM9G decoder on B200.

Sub-packages: ``config`` (typed configuration, architecture registry), ``weights``
(safetensors by tensor name, random-weights mode), ``parts`` (norm, position encoding,
mixer, feed-forward, block, model), ``cache`` (paged keys/values, state slots),
``engine`` (step function, scheduler), ``sampling``, ``kernels`` (bindings of the
sm_100a CUDA sources in ``csrc``).
"""
__version__ = "0.1.0"
