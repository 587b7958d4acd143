"""An inference engine for OPT-family language models on one NVIDIA B200.

``swifttransformer_b200`` follows what LLMServe/SwiftTransformer does - a model
step over a paged key/value cache, driven by a batching loop - rebuilt for
sm_100a: typed configuration read from config.json, weights from safetensors,
layers put together from parts, a paged cache manager, one step function for
mixed batches, a continuous-batching scheduler, sampling, and hand-written
CUDA kernels.
"""
from .config import OptConfig, load_config
from .models import load_model, random_model, write_random_model

__version__ = "0.1.0"
__all__ = ["OptConfig", "load_config", "load_model", "random_model", "write_random_model"]
