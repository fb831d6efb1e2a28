"""The .ncta writer/reader of this repository's host library on HOST tensors (no GPU needed): files are
byte-identical to the golden files the compiled reference wrote (tests/golden/ncta, made by
tests/golden/make_golden.py), golden files load back to the right values, damaged files are refused."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import ncta_cases as N  # noqa: E402

GOLD = Path(__file__).resolve().parent / "golden" / "ncta"


@pytest.fixture(scope="module")
def host():
    from nocta_b200 import configs
    r = configs.Runner(configs.load_library(), on_device=False)
    N.bind(r.api.lib)
    return r


def test_written_files_equal_the_reference_bytes(host, tmp_path):
    for name, path in N.write_all(host, tmp_path).items():
        assert path.read_bytes() == (GOLD / name).read_bytes(), name
        assert host.api.lib.nc_file_verify(str(path).encode())


def test_header_layout():
    raw = (GOLD / "module.ncta").read_bytes()
    assert raw[:4] == b"NCTA" and int.from_bytes(raw[4:8], "little") == 1 and int.from_bytes(raw[8:12], "little") == 8
    assert raw[16:80].rstrip(b"\0") == b"golden module"
    assert raw[80:144].rstrip(b"\0") == b"features.conv.weight"      # first record: name[64]
    assert int.from_bytes(raw[144:148], "little") == 0 and int.from_bytes(raw[148:152], "little") == 4  # f32, 4-d
    assert [int.from_bytes(raw[152 + 8 * i:160 + 8 * i], "little") for i in range(4)] == [3, 2, 3, 3]
    assert int.from_bytes(raw[216:224], "little") == 3 * 2 * 3 * 3 * 4


def test_golden_files_load(host):
    lib, a = host.api.lib, host.api
    t = lib.nc_tensor_load(str(GOLD / "tensor.ncta").encode())
    v = a.to_numpy(t)
    assert v.shape == (2, 2) and abs(v[0, 0] - 1.23) < 1e-6 and abs(v[1, 1] - 4.56) < 1e-6 and v[0, 1] == 0  # reference tests/test_io.c
    root, mods = N.build_model(host)
    assert lib.nc_module_load(root, str(GOLD / "module.ncta").encode()) == 0
    for name, w in N.weights().items():
        mod, pname = name.rsplit(".", 1)
        assert np.array_equal(a.to_numpy(a.nc_module_get_param(mods[mod], pname.encode())), w), name
    ck = lib.nc_checkpoint_load(str(GOLD / "checkpoint.ncta").encode())
    assert ck and ck.contents.epoch == 7 and ck.contents.loss == 0.123456
    model, opt = N.read_state_dict(host, ck.contents.model_state), N.read_state_dict(host, ck.contents.optimizer_state)
    assert list(model) == list(N.weights())
    for k, w in N.weights().items():
        assert np.array_equal(model[k], w)
    for k, w in N.optimizer_arrays().items():
        assert np.array_equal(opt[k], w) and opt[k].dtype == w.dtype
    lib.nc_checkpoint_free(ck)


def test_damaged_files_are_refused(host, tmp_path):
    lib = host.api.lib
    raw = (GOLD / "module.ncta").read_bytes()
    cases = {
        "truncated": raw[:-10],
        "bad_magic": b"XXXX" + raw[4:],
        "bad_size": raw[:216] + (10 ** 9).to_bytes(8, "little") + raw[224:],  # data_size of the first record
        "bad_ndim": raw[:148] + (99).to_bytes(4, "little") + raw[152:],
    }
    for name, data in cases.items():
        p = tmp_path / f"{name}.ncta"
        p.write_bytes(data)
        assert not lib.nc_file_verify(str(p).encode()), name
        assert not lib.nc_state_dict_load(str(p).encode()), name
    assert not lib.nc_checkpoint_load(str(GOLD / "module.ncta").encode())  # not a checkpoint (flags != 1)
    assert not lib.nc_tensor_load(str(tmp_path / "missing.ncta").encode())
