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

import json
from pathlib import Path

import torch

from .safetensors_io import SafetensorsFile, SafetensorsFormatError

WEIGHT_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"     # {"weight_map": {tensor name: file name}}


class WeightShards:
    """The tensors of a folder whose weights are spread over several safetensors
    files, named by ``model.safetensors.index.json``: one ``entries`` table and one
    ``read``, like a single file."""

    def __init__(self, folder: Path):
        self.path = folder / INDEX_FILE
        try:
            weight_map = json.loads(self.path.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError) as exc:
            raise SafetensorsFormatError(f"{self.path}: no \"weight_map\" table") from exc
        self._files = {}
        self.entries = {}
        try:
            for name, fname in weight_map.items():
                if fname not in self._files:
                    self._files[fname] = SafetensorsFile(folder / fname)
                f = self._files[fname]
                if name not in f.entries:
                    raise SafetensorsFormatError(
                        f"{self.path}: says {name!r} is in {fname}, which does not hold it")
                self.entries[name] = f.entries[name]
            self._where = {n: self._files[f] for n, f in weight_map.items()}
        except Exception:
            self.close()
            raise

    def read(self, name: str) -> torch.Tensor:
        return self._where[name].read(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def open_weights(folder):
    """The folder's ``model.safetensors``, or the files its index names."""
    folder = Path(folder)
    if (folder / WEIGHT_FILE).is_file() or not (folder / INDEX_FILE).is_file():
        return SafetensorsFile(folder / WEIGHT_FILE)
    return WeightShards(folder)


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


def resolve_names(entries: dict, wanted, aliases: dict) -> dict:
    """``{name the model uses: name the file uses}`` for the wanted names the file has
    under their own name or, failing that, under one of their ``aliases``."""
    stored = {}
    for name in wanted:
        for cand in (name, *aliases.get(name, ())):
            if cand in entries:
                stored[name] = cand
                break
    return stored


def load_tensors(folder, specs: dict, tied: dict, run_dtype: torch.dtype,
                 device, aliases: dict | None = None) -> dict:
    """Read every tensor in ``specs`` from ``folder`` onto ``device``.

    ``aliases`` maps a name to other spellings the file may use for it; errors name
    tensors as the model does.
    """
    with open_weights(folder) as f:
        path = f.path
        stored = resolve_names(f.entries, list(specs) + list(tied), aliases or {})
        used = set(stored.values())
        # the file's tensors under the model's names; what the model has no name for stays
        entries = {n: f.entries[s] for n, s in stored.items()}
        entries.update({n: e for n, e in f.entries.items() if n not in used and n not in entries})
        check_against_specs(path, entries, specs, tied)
        out = {}
        for name, spec in specs.items():
            t = f.read(stored[name])
            out[name] = t.to(device=device,
                             dtype=device_dtype(t.dtype, spec.kind, run_dtype))
        mismatched = []
        for name, target in tied.items():
            if name in stored:
                a = f.read(stored[name])
                b = f.read(stored[target])
                if not torch.equal(a, b.to(a.dtype)):
                    mismatched.append(
                        f"{name}: the model ties it to {target}, but the file "
                        f"stores a different tensor")
        if mismatched:
            raise WeightError(path, [], [], [], mismatched)
    return out
