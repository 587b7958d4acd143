"""OPT (``OPTForCausalLM``) put together from the parts.

Tensor names are those of an OPT checkpoint (``model.decoder...``; a leading
``model.`` may be absent).  What the reference reads, for comparison
(src/csrc/model/gpt/gpt_weight.cc:274-321): the same tensors after an offline
conversion that fuses q/k/v into one pre-transposed matrix, transposes
out_proj and cuts the two unused position rows
(scripts/lib/converter_lib.py:259-281).  Here the checkpoint is read as it is:
all matrices stay [out, in], q/k/v are fused at load time, and the position
table keeps its offset rows.
"""
from __future__ import annotations

from typing import Optional

from ..config.opt import OptConfig
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS
from ..parts.embedding import Embedding, OutputHead
from .base import LayerStep, ModelDef
from .registry import register_model

ROOT = "model.decoder."


def _canonical(name: str) -> Optional[str]:
    if name.endswith("decoder.version"):
        return None
    if name.startswith("decoder."):
        return "model." + name
    return name


@register_model(OptConfig.ARCHITECTURE)
def build_opt(cfg: OptConfig) -> ModelDef:
    H, E = cfg.hidden_size, cfg.word_embed_proj_dim
    proj = cfg.has_projections
    embedding = Embedding(cfg.vocab_size, E, H, ROOT + "embed_tokens.weight",
                          ROOT + "project_in.weight" if proj else None)
    position = POSITION_ENCODINGS.build("learned", max_positions=cfg.max_position_embeddings, width=H,
                                        offset=cfg.position_offset, name=ROOT + "embed_positions.weight")

    def norm(prefix: str):
        return NORMS.build("layernorm", width=H, eps=cfg.layer_norm_eps,
                           affine=cfg.layer_norm_elementwise_affine, prefix=prefix)

    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"{ROOT}layers.{i}."
        mixer = MIXERS.build("attention", hidden=H, num_heads=cfg.num_attention_heads, head_dim=cfg.head_dim,
                             num_kv_heads=cfg.num_attention_heads, bias=cfg.enable_bias,
                             names={k: f"{p}self_attn.{k if k != 'o' else 'out'}_proj" for k in "qkvo"})
        ffn = FEED_FORWARDS.build("dense", hidden=H, inner=cfg.ffn_dim, activation=cfg.activation_function,
                                  fc1_name=p + "fc1", fc2_name=p + "fc2", bias=cfg.enable_bias)
        blocks.append(BLOCKS.build("pre_norm" if cfg.do_layer_norm_before else "post_norm",
                                   mixer=mixer, feed_forward=ffn, norm1=norm(p + "self_attn_layer_norm"),
                                   norm2=norm(p + "final_layer_norm")))
    final_norm = norm(ROOT + "final_layer_norm") if cfg.has_final_layer_norm else None
    head = OutputHead(cfg.vocab_size, E, H, "lm_head.weight",
                      tied_to=ROOT + "embed_tokens.weight" if cfg.tie_word_embeddings else None,
                      project_out_name=ROOT + "project_out.weight" if proj else None)
    order = [LayerStep(block=i, cache=i) for i in range(cfg.num_hidden_layers)]
    return ModelDef(cfg, embedding, position, blocks, order, final_norm, head, _canonical,
                    max_seq_len=cfg.max_position_embeddings)
