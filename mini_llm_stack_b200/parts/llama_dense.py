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


# The spellings Llama model folders commonly use for the reference's state_dict names
# (same tensors, same layouts: [out, in] matrices, rotate-half pairing of q and k).
_FOLDER_NAMES = {
    "embed.weight": "model.embed_tokens.weight",
    "final_norm.weight": "model.norm.weight",
    "attn_norm.weight": "input_layernorm.weight",
    "mlp_norm.weight": "post_attention_layernorm.weight",
    "attn.wq.weight": "self_attn.q_proj.weight",
    "attn.wk.weight": "self_attn.k_proj.weight",
    "attn.wv.weight": "self_attn.v_proj.weight",
    "attn.wo.weight": "self_attn.o_proj.weight",
    "mlp.w_gate.weight": "mlp.gate_proj.weight",
    "mlp.w_up.weight": "mlp.up_proj.weight",
    "mlp.w_down.weight": "mlp.down_proj.weight",
}


def folder_names(name: str) -> list:
    """Other names a weight file may give the tensor the reference calls ``name``."""
    if name in _FOLDER_NAMES:
        return [_FOLDER_NAMES[name]]
    parts = name.split(".", 2)
    if (len(parts) == 3 and parts[0] == "blocks" and parts[1].isdigit()
            and parts[2] in _FOLDER_NAMES):
        return [f"model.layers.{parts[1]}.{_FOLDER_NAMES[parts[2]]}"]
    return []


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
                         RMSNorm(cfg.d_model, cfg.norm_eps), head, aliases=folder_names)


register_architecture("llama_dense", DenseLlamaConfig, build_llama_dense,
                      aliases=("LlamaForCausalLM",))
