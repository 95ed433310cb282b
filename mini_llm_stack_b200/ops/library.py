"""Building and loading the CUDA kernels.

The reference's kernels are Triton functions compiled when first called
(kernels/__init__.py:12-15 even runs them in an interpreter without a GPU).
The kernels here are CUDA sources under ``csrc/``, compiled for sm_100a with
nvcc into shared libraries inside the package (``csrc/_build``) the first time
they are needed, and called through their exported C symbols.  There is no
fallback: if a library cannot be built or loaded, the caller gets the error.

A module is a set of sources plus preprocessor defines; the file name carries a
hash of the sources, headers and flags, so a stale library is never loaded.
The attention module is compiled per head size, so a model builds only what it
needs.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"

# no fast-math: float32 sums, roots and exponentials keep their IEEE meaning
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

MODULES = {
    "core": ["embed.cu", "norm.cu", "rope_store.cu", "swiglu.cu", "gemm_f32.cu",
             "attention_simt.cu", "sampling.cu"],
    "attention": ["attention_mma.cu", "attention_tc.cu"],
    "gemm": ["gemm_tcgen05.cu"],
    "argmax_static": ["argmax_static.cu"],
}


def all_modules(head_sizes=()) -> list:
    """Every (module, defines) pair there is to build, for the given head sizes."""
    out = [("core", {})]
    if (CSRC / "attention_mma.cu").is_file():
        out += [("attention", {"MLS_HEAD_DIM": int(h)}) for h in head_sizes]
    if (CSRC / "gemm_tcgen05.cu").is_file():
        out.append(("gemm", {}))
    out.append(("argmax_static", {}))
    return out


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: dict = {}


def _say(msg: str) -> None:
    print(f"[mini_llm_stack_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDACXX"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise KernelBuildError(
        "nvcc was not found (looked at $CUDACXX, PATH and /usr/local/cuda/bin): "
        "the CUDA kernels cannot be compiled, and there is no other path")


def _build_dir() -> Path:
    """``csrc/_build`` if it can be written, else a per-user folder under tmp."""
    env = os.environ.get("MLS_B200_BUILD_DIR")
    cands = [Path(env)] if env else []
    cands.append(CSRC / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"mini_llm_stack_b200_build_{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe_{os.getpid()}"
            probe.write_text("x")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {cands}")


def _module_key(name: str, defines: dict) -> tuple:
    sources = MODULES[name]
    h = hashlib.sha256()
    own_headers = [CSRC / (Path(s).stem + ".h") for s in sources]
    for f in (sorted(CSRC.glob("*.cuh")) + [h for h in own_headers if h.is_file()]
              + [CSRC / s for s in sources]):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(NVCC_FLAGS).encode())
    tag = "_".join(f"{k}{v}" for k, v in sorted(defines.items()))
    stem = f"libmls_{name}{'_' + tag if tag else ''}_{h.hexdigest()[:12]}"
    return stem, sources


def library_path(name: str, defines: dict | None = None) -> Path:
    """Where the module's library is, or would be built."""
    stem, _ = _module_key(name, defines or {})
    for d in (CSRC / "_build",
              Path(tempfile.gettempdir()) / f"mini_llm_stack_b200_build_{os.getuid()}"):
        if (d / f"{stem}.so").is_file():
            return d / f"{stem}.so"
    return _build_dir() / f"{stem}.so"


def _run(cmd: list, what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            out, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        raise KernelBuildError(f"compiling {what} failed:\n{' '.join(cmd)}\n{out}")


def _drop_stale(fresh: Path) -> None:
    """Remove libraries of the same module and defines built from other sources."""
    prefix = fresh.name[:-len("0123456789ab.so")]
    for other in fresh.parent.glob(prefix + "*.so"):
        rest = other.name[len(prefix):-len(".so")]
        if other != fresh and len(rest) == 12 and all(c in "0123456789abcdef" for c in rest):
            try:
                other.unlink()
            except OSError:
                pass


def build(name: str, defines: dict | None = None, verbose: bool = True) -> Path:
    """Compile module ``name`` if its library does not exist yet; return its path."""
    defines = defines or {}
    stem, sources = _module_key(name, defines)
    out = library_path(name, defines)
    if out.is_file():
        return out
    nvcc = find_nvcc()
    bdir = out.parent
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    if verbose:
        _say(f"compiling kernel module '{name}' {defines or ''} for sm_100a "
             f"({len(sources)} files) into {bdir}")
    objs = []

    def compile_one(src):
        obj = bdir / f"{stem}_{Path(src).stem}.{os.getpid()}.o"
        _run([nvcc, *NVCC_FLAGS, *dflags, "-I", str(CSRC), "-c", str(CSRC / src),
              "-o", str(obj)], src)
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            objs = list(pool.map(compile_one, sources))
        tmp = bdir / f"{stem}.{os.getpid()}.tmp.so"
        _run([nvcc, "-shared", *[str(o) for o in objs], "-o", str(tmp),
              "-lcudart"], f"link {name}")
        os.replace(tmp, out)
        _drop_stale(out)
    finally:
        for o in objs:
            try:
                o.unlink()
            except OSError:
                pass
    if verbose:
        _say(f"built {out.name}")
    return out


def load(name: str, defines: dict | None = None) -> ctypes.CDLL:
    """The module's library, built first if need be.  Raises if that fails."""
    key = (name, tuple(sorted((defines or {}).items())))
    with _lock:
        if key not in _loaded:
            path = build(name, defines)
            try:
                _loaded[key] = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelBuildError(f"cannot load {path}: {exc}") from exc
        return _loaded[key]
