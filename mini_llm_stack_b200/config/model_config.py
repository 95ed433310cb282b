"""Typed configuration of the dense Llama-style decoder, read from config.json.

The canonical keys are the names the reference's ``ModelConfig`` dataclass uses
(train/config.py:6-40): ``vocab_size, d_model, n_layers, n_heads, max_seq_len,
ffn_mult, rope_theta, norm_eps, tie_embeddings``.  The reference derives
``head_dim = d_model // n_heads`` (train/config.py:27-30) and the feed-forward
width ``ffn_hidden = round_up_32(int(2 * ffn_mult * d_model / 3))``
(train/config.py:32-35); here both may also be given explicitly
(``head_dim``, ``intermediate_size``) and ``n_kv_heads`` adds grouped-query
attention, which the reference (all-MHA, train/model.py:79-82) does not have.

Every size and constant the model uses comes from this object; nothing in the
parts or kernels hard-codes one.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can build."""


# Spellings found in common Llama model folders -> canonical reference names.
_ALIASES = {
    "hidden_size": "d_model",
    "num_hidden_layers": "n_layers",
    "num_attention_heads": "n_heads",
    "num_key_value_heads": "n_kv_heads",
    "rms_norm_eps": "norm_eps",
    "max_position_embeddings": "max_seq_len",
    "tie_word_embeddings": "tie_embeddings",
    "torch_dtype": "dtype",
}

# Keys usual in Llama model folders that say nothing about the math of this decoder:
# read and dropped.  Any other unknown key is an error.
_IGNORED_KEYS = frozenset({
    "model_type", "transformers_version", "bos_token_id", "eos_token_id", "pad_token_id",
    "use_cache", "initializer_range", "pretraining_tp", "_name_or_path",
})
# Keys that would change the math: accepted only with the value that leaves it as it is.
_NEUTRAL_VALUES = {
    "rope_scaling": (None,),
    "attention_bias": (False, None),
    "mlp_bias": (False, None),
    "hidden_act": ("silu", "swish", None),
    "sliding_window": (None,),
    "attention_dropout": (0, 0.0, None),
}

# Names model folders give this architecture (registered as aliases of ``llama_dense``).
_FOLDER_ARCHITECTURES = ("LlamaForCausalLM",)

_DTYPE_NAMES = {
    "bfloat16": "bfloat16", "bf16": "bfloat16",
    "float32": "float32", "fp32": "float32", "float": "float32",
}


def canonical_dtype_name(name: str) -> str:
    try:
        return _DTYPE_NAMES[str(name).lower()]
    except KeyError:
        raise ConfigError(
            f"dtype {name!r} is not supported (bfloat16 or float32)") from None


@dataclass(frozen=True)
class DenseLlamaConfig:
    """Hyper-parameters of the dense Llama-style decoder (train/config.py:6-40).

    ``layer_order``, ``cache_source`` and ``layer_windows`` describe the
    arrangement as data: the order in which layers run (a layer may be named
    twice), which earlier call's cache a call reads instead of writing its own,
    and a per-layer attention window.  All three default to the reference's
    arrangement: every layer once, in order, own cache, full causal attention.
    """

    architecture: str = "llama_dense"
    vocab_size: int = 256
    d_model: int = 256
    n_layers: int = 4
    n_heads: int = 4
    n_kv_heads: int = 4
    head_dim: int = 64
    intermediate_size: int = 704
    max_seq_len: int = 512
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    tie_embeddings: bool = True
    dtype: str = "bfloat16"
    layer_order: tuple = ()
    cache_source: tuple = ()
    layer_windows: tuple = ()

    # ------------------------------------------------------------------ derived
    @property
    def group_size(self) -> int:
        return self.n_heads // self.n_kv_heads

    @property
    def attention_scale(self) -> float:
        """``head_dim ** -0.5`` (train/model.py:62)."""
        return float(self.head_dim) ** -0.5

    # --------------------------------------------------------------- validation
    def __post_init__(self):
        def need(cond, msg):
            if not cond:
                raise ConfigError(msg)

        for name in ("vocab_size", "d_model", "n_layers", "n_heads", "n_kv_heads",
                     "head_dim", "intermediate_size", "max_seq_len"):
            v = getattr(self, name)
            need(isinstance(v, int) and not isinstance(v, bool) and v > 0,
                 f"{name} must be a positive integer, got {v!r}")
        need(self.n_heads % self.n_kv_heads == 0,
             f"n_heads ({self.n_heads}) must be a multiple of n_kv_heads "
             f"({self.n_kv_heads})")
        need(self.head_dim % 2 == 0,
             f"head_dim ({self.head_dim}) must be even for rotate-half RoPE")
        need(self.rope_theta > 0, "rope_theta must be positive")
        need(self.norm_eps > 0, "norm_eps must be positive")
        canonical_dtype_name(self.dtype)
        # an arrangement left empty means the reference's: each layer once, in
        # order, with its own cache and full causal attention
        if len(self.layer_order) == 0:
            object.__setattr__(self, "layer_order", tuple(range(self.n_layers)))
        if len(self.cache_source) == 0:
            object.__setattr__(self, "cache_source",
                               tuple([None] * len(self.layer_order)))
        if len(self.layer_windows) == 0:
            object.__setattr__(self, "layer_windows",
                               tuple([None] * self.n_layers))
        order = self.layer_order
        need(len(order) > 0, "layer_order must name at least one layer")
        for i in order:
            need(isinstance(i, int) and 0 <= i < self.n_layers,
                 f"layer_order entry {i!r} is not a layer index < {self.n_layers}")
        need(len(self.layer_windows) == self.n_layers,
             "layer_windows needs one entry per layer")
        for w in self.layer_windows:
            need(w is None or (isinstance(w, int) and w > 0),
                 f"layer_windows entry {w!r} must be null or a positive integer")
        need(len(self.cache_source) == len(order),
             "cache_source needs one entry per layer_order entry")
        for c, src in enumerate(self.cache_source):
            if src is None:
                continue
            need(isinstance(src, int) and 0 <= src < c,
                 f"cache_source[{c}]={src!r} must name an earlier call")
            need(self.cache_source[src] is None,
                 f"cache_source[{c}] points at call {src}, which has no cache "
                 f"of its own")
            ws, wr = self.layer_windows[order[src]], self.layer_windows[order[c]]
            need(ws is None or (wr is not None and wr <= ws),
                 f"call {c} reads the cache of call {src}, whose window ({ws}) "
                 f"keeps fewer keys than call {c} needs ({wr})")

    # -------------------------------------------------------------- (de)serialise
    @classmethod
    def from_dict(cls, raw: dict) -> "DenseLlamaConfig":
        d: dict[str, Any] = {}
        for k, v in raw.items():
            if k in _NEUTRAL_VALUES:
                if v not in _NEUTRAL_VALUES[k]:
                    raise ConfigError(
                        f"config.json asks for {k} = {v!r}, which changes the model's math "
                        f"and is not supported (only {list(_NEUTRAL_VALUES[k])!r} is)")
                continue
            if k in _IGNORED_KEYS:
                continue
            d[_ALIASES.get(k, k)] = v
        if "architecture" not in d and isinstance(d.get("architectures"), list):
            d["architecture"] = d["architectures"][0]
        d.pop("architectures", None)
        if d.get("architecture") in _FOLDER_ARCHITECTURES:
            d["architecture"] = "llama_dense"

        if int(d.get("n_experts", 0) or 0) > 0:
            raise ConfigError(
                "n_experts > 0: routed experts (train/model.py:138-197) are not "
                "supported by this engine; only the dense SwiGLU feed-forward is")
        # keys of the reference dataclass that carry no information here
        for k in ("n_experts", "top_k", "moe_every", "attn_impl", "routing_impl"):
            d.pop(k, None)

        for req in ("vocab_size", "d_model", "n_layers", "n_heads"):
            if req not in d:
                raise ConfigError(f"config.json lacks the required key {req!r}")
        defaults = {f.name: f.default for f in fields(cls)}
        d.setdefault("n_kv_heads", d["n_heads"])
        if "head_dim" not in d:
            if d["d_model"] % d["n_heads"] != 0:
                raise ConfigError(
                    f"d_model ({d['d_model']}) is not a multiple of n_heads "
                    f"({d['n_heads']}) and head_dim is not given")
            d["head_dim"] = d["d_model"] // d["n_heads"]
        ffn_mult = d.pop("ffn_mult", None)
        if "intermediate_size" not in d:
            mult = 4.0 if ffn_mult is None else float(ffn_mult)
            h = int(2 * mult * d["d_model"] / 3)          # train/config.py:33
            d["intermediate_size"] = ((h + 31) // 32) * 32  # train/config.py:34
        d["dtype"] = canonical_dtype_name(d.get("dtype", defaults["dtype"]))
        order = d.get("layer_order")
        d["layer_order"] = () if order is None else tuple(order)
        src = d.get("cache_source")
        d["cache_source"] = () if src is None else tuple(src)
        win = d.get("layer_windows")
        d["layer_windows"] = () if win is None else tuple(win)
        for k in ("rope_theta", "norm_eps"):
            if k in d:
                d[k] = float(d[k])
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(d) - known)
        if unknown:
            raise ConfigError(f"config.json has keys this architecture does not "
                              f"know: {unknown}")
        return cls(**d)

    def to_dict(self) -> dict:
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            out[f.name] = list(v) if isinstance(v, tuple) else v
        return out


def read_config_json(folder: str | Path) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in model folder {str(folder)!r}")
    with open(path, "r", encoding="utf-8") as fh:
        raw = json.load(fh)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return raw


def write_config_json(folder: str | Path, config) -> None:
    Path(folder).mkdir(parents=True, exist_ok=True)
    with open(Path(folder) / "config.json", "w", encoding="utf-8") as fh:
        json.dump(config.to_dict(), fh, indent=1)
        fh.write("\n")
