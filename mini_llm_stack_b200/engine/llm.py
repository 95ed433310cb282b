"""The Python entry point: load or draw a model, generate from token prompts.

The reference's entry is ``Engine(model, ...)`` + ``submit`` + ``run_until_done``
with the result in ``req.generated`` (serve/engine.py:163-185,258-267;
serve/api.py:92-97).  ``LLM`` wraps the same three calls.
"""

from __future__ import annotations

from ..config.registry import config_from_dict
from .engine import Engine
from .runner import load_model, random_model


class LLM:
    def __init__(self, model, options=None, **engine_options):
        """``options``: an ``EngineOptions`` record, or the engine's arguments by name."""
        self.model = model
        self.config = model.config
        if options is not None:
            self.engine = Engine.from_options(model, options)
        else:
            self.engine = Engine(model, **engine_options)

    @classmethod
    def from_folder(cls, folder, dtype: str | None = None, device=None, options=None,
                    **engine_options) -> "LLM":
        """``options`` (an ``EngineOptions``) also says in which dtype and on which device
        the folder is loaded, unless ``dtype`` / ``device`` are given here."""
        dtype, device = cls._where(dtype, device, options)
        return cls(load_model(folder, dtype=dtype, device=device), options, **engine_options)

    @classmethod
    def from_random(cls, config, seed: int = 0, norm_std: float = 0.0,
                    dtype: str | None = None, device=None, fast: bool = False, options=None,
                    **engine_options) -> "LLM":
        if isinstance(config, dict):
            config = config_from_dict(config)
        dtype, device = cls._where(dtype, device, options)
        return cls(random_model(config, seed, norm_std, dtype, device, fast), options,
                   **engine_options)

    @staticmethod
    def _where(dtype, device, options):
        if options is not None:
            dtype = dtype or options.dtype
            device = device or options.device
        return dtype, device or "cuda:0"

    def generate(self, prompts, max_new_tokens: int = 32, temperature: float = 0.0,
                 seed: int | None = None, eos=None) -> list:
        """New tokens for each prompt (lists of token ids in, lists out).

        All prompts are submitted at once and served by continuous batching.
        Request i draws with the key (seed, i-th id of this engine), so the
        result does not depend on how the requests were batched; ``seed`` None takes
        the engine's (``EngineOptions.seed``).
        """
        reqs = [self.engine.submit(p, max_new_tokens, eos, temperature, seed) for p in prompts]
        self.engine.run_until_done(max_steps=10_000_000)
        return [list(r.generated) for r in reqs]
