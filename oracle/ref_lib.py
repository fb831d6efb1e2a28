"""Loader for the compiled reference CPU library (TEST INFRASTRUCTURE ONLY).

oracle/_ref/libnocta_ref.so is the UNMODIFIED reference built by oracle/Makefile from its own
sources, plus oracle/ref_shims.c.  It travels with the repository snapshot as a built artefact
(it is git-ignored), so GPU-side tests can call the real reference; the reference sources
themselves are only needed where the library is built.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

from nocta_b200.capi import NoctaAPI, TensorP

HERE = Path(__file__).resolve().parent
REF_SO = HERE / "_ref" / "libnocta_ref.so"
REF_FAST_SO = HERE / "_ref" / "libnocta_ref_fast.so"
# where the reference sources lie when they are available (same variable as oracle/Makefile: make REF=...)
REFERENCE_ROOT = Path(os.environ.get("REF", "/root/reference"))


def build(reference_root: Path = REFERENCE_ROOT) -> bool:
    """Compile the reference into oracle/_ref/ when its sources are present."""
    if not (reference_root / "src" / "nn" / "conv.c").exists():
        return REF_SO.exists()
    subprocess.run(["make", "-C", str(HERE), f"REF={reference_root}"], check=True, capture_output=True)
    return REF_SO.exists()


def build_apps(reference_root: Path = REFERENCE_ROOT) -> list:
    """Compile the reference's example programs against this repository's libraries (oracle/_ref/apps/)."""
    if (reference_root / "examples" / "xor.c").exists():
        subprocess.run(["make", "-C", str(HERE), f"REF={reference_root}", "apps"], check=True, capture_output=True)
    return sorted((HERE / "_ref" / "apps").glob("*")) if (HERE / "_ref" / "apps").exists() else []


def available() -> bool:
    return REF_SO.exists()


class RefAPI(NoctaAPI):
    def __init__(self, path: Path = REF_SO):
        super().__init__(path)
        for name in ("shim_flatten", "shim_gelu"):
            fn = getattr(self.lib, name)
            fn.restype = TensorP
            fn.argtypes = [TensorP]
            setattr(self, name, fn)


_cache = {}


def load(fast: bool = False) -> RefAPI:
    path = REF_FAST_SO if fast else REF_SO
    if path not in _cache:
        _cache[path] = RefAPI(path)
    return _cache[path]
