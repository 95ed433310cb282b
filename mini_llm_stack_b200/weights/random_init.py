"""Random weights from a configuration and a seed.

The reference initialises every ``nn.Linear`` and ``nn.Embedding`` weight from
N(0, 0.02^2) and every norm weight to one (train/model.py:232-236, :27).  Here
the tensors are drawn one by one, in the order the model declares them, from a
single seeded CPU generator, so the same (config, seed) gives the same folder
on every machine.
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.model_config import write_config_json
from ..config.registry import build_model
from .loader import WEIGHT_FILE
from .safetensors_io import write_safetensors

INIT_STD = 0.02          # train/model.py:234,236

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def draw_tensor(spec, gen: torch.Generator, norm_std: float) -> torch.Tensor:
    """One tensor in float32 from its spec's initialisation rule."""
    if spec.init == "normal":
        return torch.randn(spec.shape, generator=gen, dtype=torch.float32) * INIT_STD
    if spec.init == "ones":
        t = torch.ones(spec.shape, dtype=torch.float32)
        if norm_std:
            t = t + torch.randn(spec.shape, generator=gen,
                                dtype=torch.float32) * norm_std
        return t
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32)
    raise ValueError(f"unknown initialisation {spec.init!r}")


def random_tensors(config, seed: int, norm_std: float = 0.0,
                   dtype: str | None = None):
    """Yield ``(name, tensor)`` in declaration order, cast to the stored dtype."""
    model = build_model(config)
    store = _TORCH_DTYPES[dtype or config.dtype]
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    for name, spec in model.tensor_specs().items():
        t = draw_tensor(spec, gen, norm_std)
        yield name, (t.to(torch.int32) if spec.kind == "table" else t.to(store))


def write_random_model(folder, config, seed: int, norm_std: float = 0.0,
                       dtype: str | None = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config``."""
    folder = Path(folder)
    model = build_model(config)
    store = _TORCH_DTYPES[dtype or config.dtype]
    specs = model.tensor_specs()
    file_specs = [(n, torch.int32 if s.kind == "table" else store, tuple(s.shape))
                  for n, s in specs.items()]
    stream = random_tensors(config, seed, norm_std, dtype)

    def produce(name):
        got, t = next(stream)
        assert got == name
        return t

    write_config_json(folder, config)
    write_safetensors(folder / WEIGHT_FILE, file_specs, produce,
                      metadata={"seed": seed, "norm_std": norm_std})
    return folder
