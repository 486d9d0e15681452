"""In-tree build and loading of the sm_100a CUDA extension.

The shared object lives under ``llaminar_b200/ops/_build`` (next to the sources, so a source
snapshot carries it along) together with a hash of the sources it was built from.  ``load()``
imports the existing binary when the hash still matches and rebuilds otherwise.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
from pathlib import Path

NAME = "llaminar_b200_ops"
CSRC = Path(__file__).resolve().parent / "csrc"
BUILD_DIR = Path(__file__).resolve().parent / "_build"
SOURCES = ["binding.cpp", "gemv.cu", "gemv_stream.cu", "gemm_tc.cu", "gemm_tc_small.cu", "attention.cu", "attention_tc.cu", "ops.cu", "gdn.cu", "moe_ep.cu", "no_alloc.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]

_module = None


def _bounds_check() -> bool:
    from ..utils.env import debug_env
    return bool(debug_env().bounds_check)


def _flags() -> list[str]:
    return NVCC_FLAGS + (["-DLLM_BOUNDS_CHECK"] if _bounds_check() else [])


def _build_dir() -> Path:
    """The bounds-check variant is a build of its own (other flags, other directory), selected by LLAMINAR_BOUNDS_CHECK."""
    return BUILD_DIR.with_name("_build_bc") if _bounds_check() else BUILD_DIR


def _existing_sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def source_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.iterdir()):
        if p.suffix in (".cu", ".cuh", ".cpp", ".h", ".inc"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(_flags()).encode())
    return h.hexdigest()


def _so_path() -> Path:
    return _build_dir() / f"{NAME}.so"


def is_built() -> bool:
    hp = _build_dir() / f"{NAME}.hash"
    return _so_path().exists() and hp.exists() and hp.read_text().strip() == source_hash()


def _import_so():
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, str(_so_path()))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[NAME] = mod
    return mod


def build(verbose: bool = False, force: bool = False):
    """Compile every source for sm_100a (cross-compiles without a GPU) and return the module."""
    global _module
    if not force and is_built():
        _module = _import_so()
        return _module
    from torch.utils import cpp_extension
    _build_dir().mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(max(1, (os.cpu_count() or 2))))
    cpp_extension.load(
        name=NAME,
        sources=[str(s) for s in _existing_sources()],
        extra_cflags=["-O2", "-std=c++17"] + (["-DLLM_BOUNDS_CHECK"] if _bounds_check() else []),
        extra_cuda_cflags=_flags(),
        extra_include_paths=[str(CSRC)],
        build_directory=str(_build_dir()),
        with_cuda=True,
        verbose=verbose,
        is_python_module=True,
    )
    (_build_dir() / f"{NAME}.hash").write_text(source_hash())
    _module = sys.modules.get(NAME) or _import_so()
    return _module


def build_bounds_check_variant() -> None:
    """Compile the debug variant with explicit index checks (LLAMINAR_BOUNDS_CHECK=1 loads it) in a child process: the
    variant is chosen by the environment before the extension is first imported."""
    import subprocess
    env = dict(os.environ, LLAMINAR_BOUNDS_CHECK="1")
    code = "from llaminar_b200.ops import build as b; b.build()"
    subprocess.run([sys.executable, "-c", code], check=True, env=env, cwd=str(Path(__file__).resolve().parents[2]))


def load():
    """The extension module; built on first use if the in-tree binary is missing or stale."""
    global _module
    if _module is None:
        _module = build()
    return _module


def so_path() -> str:
    return str(_so_path())


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv)
    print("built", _so_path())
