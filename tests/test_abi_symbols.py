"""CPU-side checks of the drop-in boundary: the kernel library loads without a GPU and exports every
entry point that include/nocta_cuda.h declares, and the Python binding table covers the header."""
from nocta_b200 import cuda_abi


def test_library_exports_every_declared_symbol():
    abi = cuda_abi.load()
    declared = cuda_abi.header_symbols()
    assert len(declared) > 80
    missing = [s for s in declared if not hasattr(abi.lib, s)]
    assert not missing, missing


def test_binding_table_matches_header():
    declared = set(cuda_abi.header_symbols())
    bound = set(cuda_abi.SIGNATURES)
    assert declared - bound == set(), sorted(declared - bound)
    assert bound - declared == set(), sorted(bound - declared)


def test_status_api_without_gpu():
    abi = cuda_abi.load()
    abi.nc_cuda_clear_status()
    assert abi.nc_cuda_last_status() == 0
    prev = abi.nc_cuda_set_math_mode(2)
    assert abi.nc_cuda_get_math_mode() == 2
    abi.nc_cuda_set_math_mode(prev)


def test_reference_include_paths_compile(tmp_path):
    """A translation unit written against the reference's include layout (nocta/nn/conv.h, ...)
    compiles against this repository's headers, and the host library exports what it uses."""
    import ctypes
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    fwd = sorted(p.relative_to(root / "include") for p in (root / "include" / "nocta").rglob("*.h"))
    assert len(fwd) > 15
    src = tmp_path / "tu.c"
    src.write_text("".join(f'#include "{p.as_posix()}"\n' for p in fwd) +
                   "int use(void) { nc_tensor* t = nc_tensor_zeros((size_t[]){2, 2}, 2, NC_F32);\n"
                   "  nc_tensor_free(t); return (int)nc_cuda_last_status(); }\n")
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", f"-I{root / 'include'}", "-c", str(src), "-o", str(tmp_path / "tu.o")],
                   check=True)
    host = ctypes.CDLL(str(root / "nocta_b200" / "lib" / "libnocta.so"))
    for sym in ("nc_tensor_zeros", "nc_tensor_free", "nc_conv2d", "nc_batchnorm2d", "nc_cross_entropy_loss", "nc_sgd", "nc_backward"):
        assert hasattr(host, sym), sym
