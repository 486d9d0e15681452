"""In-tree build and loading of the C++ BPE merger (`csrc/bpe_merge.cpp`).

The Python tokenizer works without it; with it, long words and cold caches avoid the quadratic pair rescan.
The reference's tokenizer is C++ throughout (reference: src/v2/utils/Tokenizer.cpp).
"""
from __future__ import annotations

import importlib.util
import pathlib
import subprocess
import sys
import sysconfig

HERE = pathlib.Path(__file__).resolve().parent
SRC = HERE / "csrc" / "bpe_merge.cpp"
BUILD = HERE / "_build"
NAME = "llaminar_b200_bpe"
_mod = None


def _so() -> pathlib.Path:
    return BUILD / f"{NAME}{sysconfig.get_config_var('EXT_SUFFIX') or '.so'}"


def build(force: bool = False):
    """g++ -shared against the CPython and pybind11 headers; returns the module."""
    global _mod
    so = _so()
    if force or not so.exists() or so.stat().st_mtime < SRC.stat().st_mtime:
        import pybind11
        BUILD.mkdir(exist_ok=True)
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", f"-I{pybind11.get_include()}",
               f"-I{sysconfig.get_paths()['include']}", str(SRC), "-o", str(so)]
        subprocess.run(cmd, check=True, capture_output=True)
    spec = importlib.util.spec_from_file_location(NAME, str(so))
    _mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(_mod)
    sys.modules[NAME] = _mod
    return _mod


def load():
    global _mod
    if _mod is None:
        so = _so()
        if not so.exists():
            raise ImportError("the native BPE merger has not been built")
        build()
    return _mod


def make_merger(tokens: list[str], ranks: dict[tuple[str, str], int]):
    """Merger over the tokenizer's vocabulary and merge table (raises ImportError when the helper is not built)."""
    mod = load()
    merges = [pair for pair, _ in sorted(ranks.items(), key=lambda kv: kv[1])]
    return mod.Merger(list(tokens), merges)
