"""Configuration of the OPT architecture (``OPTForCausalLM``).

Field names are the keys of an OPT ``config.json``.  The reference fills the
same quantities by hand: src/csrc/model/gpt/gpt_hyper_param.h:51-77
(GetOptHyperParam: pre-LN, no rotary, ReLU, LayerNorm, biased qkv/out,
kv heads = heads), src/examples/lib/common_gpt_hyper_params.h:10-68 (size
tables).  The reference rejects post-LN (src/csrc/model/gpt/gpt.cc:238-240)
and has no word_embed_proj_dim / enable_bias / affine switches; here they are
ordinary options.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import ClassVar, Dict

from .base import ConfigError, ModelConfig, register_config

SUPPORTED_ACTIVATIONS = ("relu", "gelu")


@register_config
@dataclasses.dataclass(frozen=True)
class OptConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "OPTForCausalLM"
    KEY_ALIASES: ClassVar[Dict[str, str]] = {"_remove_final_layer_norm": "remove_final_layer_norm"}

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    ffn_dim: int
    num_attention_heads: int
    max_position_embeddings: int
    # width of the token embedding; differs from hidden_size only in models
    # with project_in / project_out.  0 means "same as hidden_size".
    word_embed_proj_dim: int = 0
    do_layer_norm_before: bool = True
    enable_bias: bool = True
    layer_norm_elementwise_affine: bool = True
    activation_function: str = "relu"
    tie_word_embeddings: bool = True
    remove_final_layer_norm: bool = False
    # OPT's config.json carries no eps; the architecture's value is 1e-5
    # (src/csrc/model/gpt/gpt_weight.h:63).  The key is honoured when present.
    layer_norm_eps: float = 1e-5
    # learned positions are stored with two leading rows that are never used
    # by position 0 (scripts/lib/converter_lib.py:271 strips them offline).
    position_offset: int = 2
    bos_token_id: int = 2
    eos_token_id: int = 2
    pad_token_id: int = 1
    torch_dtype: str = "bfloat16"
    model_type: str = "opt"

    def __post_init__(self) -> None:
        if self.word_embed_proj_dim == 0:
            object.__setattr__(self, "word_embed_proj_dim", self.hidden_size)

    # derived sizes -----------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def has_projections(self) -> bool:
        return self.word_embed_proj_dim != self.hidden_size

    @property
    def has_final_layer_norm(self) -> bool:
        return self.do_layer_norm_before and not self.remove_final_layer_norm

    def validate(self) -> None:
        a = self.ARCHITECTURE
        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "ffn_dim",
                    "num_attention_heads", "max_position_embeddings", "word_embed_proj_dim"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{a}: '{key}' must be positive, got {getattr(self, key)}")
        if self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"{a}: 'hidden_size' ({self.hidden_size}) is not a multiple of "
                f"'num_attention_heads' ({self.num_attention_heads})")
        if self.activation_function not in SUPPORTED_ACTIVATIONS:
            raise ConfigError(
                f"{a}: 'activation_function' = '{self.activation_function}' is not supported "
                f"(supported: {', '.join(SUPPORTED_ACTIVATIONS)})")
        if self.layer_norm_eps <= 0:
            raise ConfigError(f"{a}: 'layer_norm_eps' must be positive, got {self.layer_norm_eps}")
        if self.position_offset < 0:
            raise ConfigError(f"{a}: 'position_offset' must not be negative")


_PRESET_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def preset_names() -> list:
    return sorted(f[:-5] for f in os.listdir(_PRESET_DIR) if f.endswith(".json"))


def opt_preset(name: str) -> OptConfig:
    """A named OPT size (``opt_1.3b`` ...) for random-weight runs.

    The sizes are data files under ``config/presets`` (the numbers of
    src/examples/lib/common_gpt_hyper_params.h:10-68), read like any config.json.
    """
    key = name.lower().replace("-", "_")
    path = os.path.join(_PRESET_DIR, key + ".json")
    if not os.path.isfile(path):
        raise ConfigError(f"unknown model name '{name}'; known: {', '.join(preset_names())}")
    with open(path, "r", encoding="utf-8") as f:
        cfg = OptConfig.from_dict(json.load(f))
    return cfg
