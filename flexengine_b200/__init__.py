"""flexengine_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors, or seeded random weights) to generated
tokens: typed config and architecture registry, by-name weight loader, a model put together
from parts, a paged cache manager, one step function over mixed batches, a token-budget
scheduler, sampling, and hand-written CUDA kernels under ``csrc/``.
"""
__version__ = "0.1.0"
