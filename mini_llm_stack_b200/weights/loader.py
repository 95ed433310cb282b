"""Weights by tensor name, with one error that says everything that is wrong.

The reference loads with a strict ``load_state_dict`` (serve/api.py:60), which
raises on missing and unexpected keys.  Here the model's parts declare the
tensors they need (name -> shape, kind); the file is checked against that list
before a single byte moves, and every missing name, unexpected name and wrong
shape is reported together.

Device dtypes: in a bfloat16 run, tensors stored in 16 bits are kept in
bfloat16 and tensors stored in 32 bits stay in 32 bits; integer tables become
int32.  In a float32 run every floating tensor is float32.
"""

from __future__ import annotations

from pathlib import Path

import torch

from .safetensors_io import SafetensorsFile

WEIGHT_FILE = "model.safetensors"


class WeightError(ValueError):
    """Missing / unexpected tensors and wrong shapes, all in one message."""

    def __init__(self, path, missing, unexpected, wrong_shape, other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"weights in {str(path)!r} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): "
                         + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): "
                         + "; ".join(f"{n}: expected {list(e)}, file has {list(g)}"
                                     for n, e, g in self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def device_dtype(stored: torch.dtype, kind: str, run_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor has on the device, from how it is stored and run."""
    if kind == "table" or not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored.itemsize >= 4:
        return torch.float32           # stored in 32 bits: stays so
    return torch.bfloat16


def check_against_specs(path, entries: dict, specs: dict, tied: dict) -> None:
    """Raise one WeightError if the file's tensors do not fit ``specs``.

    ``tied`` maps a name that may appear in the file without being needed
    (a tied output head) to the tensor it must then equal in shape.
    """
    missing = [n for n in specs if n not in entries]
    unexpected = [n for n in entries if n not in specs and n not in tied]
    wrong = []
    other = []
    for n, spec in specs.items():
        if n in entries and tuple(entries[n].shape) != tuple(spec.shape):
            wrong.append((n, spec.shape, entries[n].shape))
        if n in entries:
            is_int = not entries[n].dtype.is_floating_point
            if (spec.kind == "table") != is_int:
                other.append(f"{n}: stored as {entries[n].dtype}, but the model "
                             f"needs {'an integer table' if spec.kind == 'table' else 'a floating tensor'}")
    for n, target in tied.items():
        if n in entries and target in specs and \
                tuple(entries[n].shape) != tuple(specs[target].shape):
            wrong.append((n, specs[target].shape, entries[n].shape))
    if missing or unexpected or wrong or other:
        raise WeightError(path, missing, unexpected, wrong, other)


def load_tensors(folder, specs: dict, tied: dict, run_dtype: torch.dtype,
                 device) -> dict:
    """Read every tensor in ``specs`` from ``folder`` onto ``device``."""
    path = Path(folder) / WEIGHT_FILE
    with SafetensorsFile(path) as f:
        check_against_specs(path, f.entries, specs, tied)
        out = {}
        for name, spec in specs.items():
            t = f.read(name)
            out[name] = t.to(device=device,
                             dtype=device_dtype(t.dtype, spec.kind, run_dtype))
        mismatched = []
        for name, target in tied.items():
            if name in f.entries:
                a = f.read(name)
                b = f.read(target)
                if not torch.equal(a, b.to(a.dtype)):
                    mismatched.append(
                        f"{name}: the model ties it to {target}, but the file "
                        f"stores a different tensor")
        if mismatched:
            raise WeightError(path, [], [], [], mismatched)
    return out
