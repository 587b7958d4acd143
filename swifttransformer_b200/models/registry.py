"""One registry from an architecture's name to its model builder.

``build_model_def(config)`` looks the builder up by ``config.ARCHITECTURE`` (the
string in config.json's ``architectures``).  The reference registers its three
model classes by hand (src/csrc/pybinding.cc:53-80).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from ..config.base import ConfigError, ModelConfig, load_config
from ..weights.loader import load_named_tensors
from ..weights.random_init import random_named_tensors, write_random_checkpoint
from .base import CausalLM, ModelDef

_BUILDERS: Dict[str, Callable[[ModelConfig], ModelDef]] = {}


def register_model(architecture: str, builder: Optional[Callable[[ModelConfig], ModelDef]] = None):
    """Register ``builder(config) -> ModelDef`` for an architecture name (usable as a decorator)."""
    def deco(fn):
        _BUILDERS[architecture] = fn
        return fn
    return deco(builder) if builder is not None else deco


def known_models() -> list:
    return sorted(_BUILDERS)


def build_model_def(config: ModelConfig) -> ModelDef:
    arch = config.ARCHITECTURE
    if arch not in _BUILDERS:
        raise ConfigError(f"no model is registered for architecture '{arch}'; known: {', '.join(known_models())}")
    return _BUILDERS[arch](config)


def _torch_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.float32, torch.bfloat16):
            return dtype
        raise ValueError(f"unsupported compute dtype {dtype}")
    names = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if str(dtype).lower() not in names:
        raise ValueError(f"unknown dtype '{dtype}' (bfloat16 or float32)")
    return names[str(dtype).lower()]


def load_model(model_dir: str, dtype="bfloat16", device="cuda") -> CausalLM:
    """config.json + safetensors of ``model_dir`` -> a model on ``device``."""
    dtype, device = _torch_dtype(dtype), torch.device(device)
    cfg = load_config(model_dir)
    mdef = build_model_def(cfg)
    tensors = load_named_tensors(model_dir, mdef.param_specs(), dtype, device, mdef.canonical_name)
    return CausalLM(mdef, tensors, dtype, device)


def random_model(config: ModelConfig, seed: int = 0, dtype="bfloat16", device="cuda", std: float = 0.02) -> CausalLM:
    """A model with random weights generated on ``device`` (nothing touches the disk)."""
    dtype, device = _torch_dtype(dtype), torch.device(device)
    mdef = build_model_def(config)
    tensors = random_named_tensors(mdef.param_specs(), seed, dtype, device, std)
    return CausalLM(mdef, tensors, dtype, device)


def write_random_model(model_dir: str, config: ModelConfig, seed: int = 0, std: float = 0.02) -> str:
    """Write config.json and model.safetensors with random weights; returns ``model_dir``."""
    from ..config.base import save_config
    mdef = build_model_def(config)
    save_config(config, model_dir)
    write_random_checkpoint(model_dir, mdef.param_specs(), seed, std)
    return model_dir
