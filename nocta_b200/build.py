"""Build the native libraries in-tree.

  nocta_b200/lib/libnocta_cuda.so   the sm_100a kernel library behind the nc_cuda_* C ABI
  nocta_b200/lib/libnocta.so        the C host library (nc_* API) on top of it

nvcc cross-compiles for sm_100a without a GPU, so this runs on any box with the CUDA toolkit.
Each source is compiled to an object only when it or a header changed (content hash).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
LIB = PKG / "lib"
OBJ = PKG / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CC = os.environ.get("CC", "gcc")
CFLAGS = ["-std=c11", "-O2", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-D_GNU_SOURCE"]


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _run(cmd, log: Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write(" ".join(map(str, cmd)) + "\n" + proc.stdout + proc.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]}")


def _compile(src: Path, headers, cmd_prefix, flags) -> Path:
    obj = OBJ / (src.name + ".o")
    stamp = OBJ / (src.name + ".sha")
    want = _digest([src, *headers]) + " ".join(flags)
    if obj.exists() and stamp.exists() and stamp.read_text() == want:
        return obj
    _run([cmd_prefix, *flags, "-c", str(src), "-o", str(obj)], log=OBJ / (src.name + ".log"))
    stamp.write_text(want)
    return obj


def build_cuda(verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted((ROOT / "include").glob("*.h"))
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, headers, NVCC, NVCC_FLAGS), srcs))
    out = LIB / "libnocta_cuda.so"
    newest = max(o.stat().st_mtime for o in objs)
    if not out.exists() or out.stat().st_mtime < newest:
        _run([NVCC, "-shared", "-o", str(out), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-lcudart"])
    if verbose:
        for s in srcs:
            log = OBJ / (s.name + ".log")
            if log.exists():
                print(log.read_text())
    return out


def build_host() -> Path | None:
    srcs = sorted(HOST.glob("*.c"))
    if not srcs:
        return None
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    headers = sorted(HOST.glob("*.h")) + sorted((ROOT / "include").rglob("*.h"))
    flags = CFLAGS + ["-I", str(ROOT / "include"), "-I", str(HOST)]
    objs = [_compile(s, headers, CC, flags) for s in srcs]
    out = LIB / "libnocta.so"
    newest = max(o.stat().st_mtime for o in objs)
    cuda_lib = LIB / "libnocta_cuda.so"
    if not out.exists() or out.stat().st_mtime < max(newest, cuda_lib.stat().st_mtime if cuda_lib.exists() else 0):
        _run([CC, "-shared", "-o", str(out), *map(str, objs), "-Wl,-Bsymbolic", f"-L{LIB}", "-lnocta_cuda",
              "-Wl,-rpath,$ORIGIN", "-lm", "-ldl"])
    return out


def build_all(verbose: bool = False):
    cuda = build_cuda(verbose)
    host = build_host()
    return cuda, host


if __name__ == "__main__":
    print(build_all(verbose="-v" in sys.argv))
