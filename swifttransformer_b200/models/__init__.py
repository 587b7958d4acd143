from .base import CausalLM, LayerStep, ModelDef
from .registry import (build_model_def, known_models, load_model, random_model, register_model,
                       write_random_model)
from . import opt as _opt  # registers OPTForCausalLM

__all__ = ["CausalLM", "LayerStep", "ModelDef", "build_model_def", "known_models", "load_model",
           "random_model", "register_model", "write_random_model"]
