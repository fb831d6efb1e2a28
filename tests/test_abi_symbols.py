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
