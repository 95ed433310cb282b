"""Options of the engine (not of the model).

All knobs of the engine live in this one record, as the reference keeps them in
``Engine.__init__`` (serve/engine.py:163-166): ``num_blocks=256, block_size=16,
max_batch=16, device, dtype`` carry its names and defaults (``dtype`` None means
the model folder's own; the reference's is float32).  The token budget and
portion size have no counterpart there: the reference prefills every admitted
prompt whole and alone (serve/engine.py:190-206).  ``dtype`` and ``device``
say how the model is loaded (``LLM.from_folder(folder, options=...)``) and are
checked against a model that is already loaded (``Engine.from_options``).
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
    kv_dtype: str | None = None       # type of the cached keys and values; None: the run's dtype
    seed: int = 0                     # sampling seed of requests that bring none
    cuda_graphs: bool = True          # replay decode steps (and repeated, host-bound prompt steps) from graphs
    launch_ahead: bool = True         # start the next decode step before the host has this one's tokens

    def __post_init__(self):
        for k in ("num_blocks", "block_size", "max_batch", "max_tokens_per_step",
                  "chunk_size"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"{k} must be a positive integer, got {v!r}")
        if self.dtype is not None:
            self.dtype = canonical_dtype_name(self.dtype)
        if self.kv_dtype is not None:
            self.kv_dtype = canonical_dtype_name(self.kv_dtype)
        if not isinstance(self.seed, int):
            raise ConfigError(f"seed must be an integer, got {self.seed!r}")

    def check_against(self, run_dtype: str, device) -> None:
        """Refuse options a loaded model (its run dtype, its device) contradicts.  The
        cache holds keys and values in the run's dtype: there is no quantised or
        widened cache, so another ``kv_dtype`` is an error, not a silent default."""
        run_dtype = canonical_dtype_name(run_dtype)
        if self.dtype is not None and self.dtype != run_dtype:
            raise ConfigError(f"options ask for dtype {self.dtype}, the model runs in {run_dtype}")
        if self.kv_dtype is not None and self.kv_dtype != run_dtype:
            raise ConfigError(f"kv_dtype {self.kv_dtype} differs from the run's dtype "
                              f"{run_dtype}: the cache is kept in the run's dtype only")
        import torch
        want, have = torch.device(self.device), torch.device(device)
        if want.type != have.type or (want.index or 0) != (have.index or 0):
            raise ConfigError(f"options ask for device {self.device}, the model is on {have}")
