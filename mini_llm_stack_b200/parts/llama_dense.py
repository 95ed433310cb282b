"""The dense Llama-style decoder of the reference, as a list of parts.

Reference: ``Transformer`` (train/model.py:220-244) made of ``Block``s
(train/model.py:200-217) with ``RMSNorm`` (:23-33), ``Attention`` + ``Rotary``
(:36-52, :73-124) and ``SwiGLU`` (:127-135); tensor names are the reference's
``state_dict`` names (``embed.weight``, ``blocks.{i}.attn.wq.weight``, ...,
``final_norm.weight``, ``lm_head.weight``).
"""

from __future__ import annotations

from ..config.model_config import DenseLlamaConfig
from ..config.registry import register_architecture
from .attention import GroupedQueryAttention
from .block import PreNormBlock
from .feedforward import SwiGLUFeedForward
from .model import ComposedModel, LayerCall, OutputHead, TokenEmbedding
from .norm import RMSNorm
from .position import RotaryPosition


def build_llama_dense(cfg: DenseLlamaConfig) -> ComposedModel:
    embedding = TokenEmbedding(cfg.vocab_size, cfg.d_model)
    blocks = []
    for i in range(cfg.n_layers):
        position = RotaryPosition(cfg.head_dim, cfg.rope_theta, cfg.max_seq_len)
        mixer = GroupedQueryAttention(cfg.d_model, cfg.n_heads, cfg.n_kv_heads,
                                      cfg.head_dim, cfg.attention_scale, position,
                                      window=cfg.layer_windows[i])
        ffn = SwiGLUFeedForward(cfg.d_model, cfg.intermediate_size)
        blocks.append(PreNormBlock(RMSNorm(cfg.d_model, cfg.norm_eps), mixer,
                                   RMSNorm(cfg.d_model, cfg.norm_eps), ffn))
    calls, slot_of_call = [], {}
    for c, layer in enumerate(cfg.layer_order):
        src = cfg.cache_source[c]
        if src is None:
            slot_of_call[c] = len(slot_of_call)
            calls.append(LayerCall(layer, slot_of_call[c], writes=True))
        else:
            calls.append(LayerCall(layer, slot_of_call[src], writes=False))
    head = OutputHead(cfg.vocab_size, cfg.d_model,
                      tied_to=embedding if cfg.tie_embeddings else None)
    return ComposedModel(cfg, embedding, blocks, calls,
                         RMSNorm(cfg.d_model, cfg.norm_eps), head)


register_architecture("llama_dense", DenseLlamaConfig, build_llama_dense)
