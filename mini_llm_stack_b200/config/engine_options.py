"""Options of the engine (not of the model).

The first four carry the names and defaults of the reference's
``Engine.__init__`` arguments (serve/engine.py:163-166): ``num_blocks=256,
block_size=16, max_batch=16, dtype=float32``.  The token budget and portion
size have no counterpart there: the reference prefills every admitted prompt
whole and alone (serve/engine.py:190-206).
"""

from __future__ import annotations

from dataclasses import dataclass

from .model_config import ConfigError, canonical_dtype_name


@dataclass
class EngineOptions:
    num_blocks: int = 256             # pages per cache group
    block_size: int = 16              # tokens per page
    max_batch: int = 16               # most requests running at once
    max_tokens_per_step: int = 2048   # token budget of one step
    chunk_size: int = 2048            # largest prompt portion of one request
    dtype: str | None = None          # None: the model folder's own dtype
    device: str = "cuda:0"
    cuda_graphs: bool = True          # replay pure-decode steps from a graph
    launch_ahead: bool = True         # start the next decode step before the host has this one's tokens

    def __post_init__(self):
        for k in ("num_blocks", "block_size", "max_batch", "max_tokens_per_step",
                  "chunk_size"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"{k} must be a positive integer, got {v!r}")
        if self.dtype is not None:
            self.dtype = canonical_dtype_name(self.dtype)
