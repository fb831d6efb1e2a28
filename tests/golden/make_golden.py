"""Regenerates tests/golden/reference_cpu.npz and the golden .ncta files from the compiled reference CPU library.

Run where the reference sources are available (oracle/Makefile builds oracle/_ref/libnocta_ref.so from
them):   python tests/golden/make_golden.py
The file holds, for every case of tests/golden/cases.py, what the reference's own C code returned.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import cases  # noqa: E402
import ncta_cases  # noqa: E402
from nocta_b200 import configs  # noqa: E402
from oracle import ref_lib  # noqa: E402


def main():
    ref_lib.build()
    r = configs.Runner(ref_lib.load(), on_device=False)
    out = cases.run_all(r)
    path = Path(__file__).resolve().parent / "reference_cpu.npz"
    np.savez_compressed(path, **out)
    print(f"{path}: {len(out)} arrays, {path.stat().st_size} bytes")
    for name, written in ncta_cases.write_all(r, Path(__file__).resolve().parent / "ncta").items():
        print(f"{written}: {written.stat().st_size} bytes")


if __name__ == "__main__":
    main()
