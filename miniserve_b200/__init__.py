"""miniserve_b200: a small, whole inference engine for the Qwen3 dense decoder on one B200.

Everything between a request's tokens and its next token: typed configuration and an
architecture registry, safetensors loading and random weights, layers composed from parts,
a paged cache manager, one step function, a continuous-batching scheduler, sampling, and
hand-written CUDA kernels for sm_100a underneath.
"""

from . import models  # noqa: F401  (registers the architectures)

__version__ = "0.1.0"
