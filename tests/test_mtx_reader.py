"""CPU test: the Matrix Market loader of the library against upstream's mmio_allinone (goldens made by the unmodified
upstream loader, tests/golden/make_golden.py): file order inside rows, repeated entries, symmetric expansion,
pattern and integer fields."""
import ctypes as C
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "tiling_golden.json")))["mtx"]


def read(path):
    from tilespmm_b200 import api
    L = api.lib()
    L.tsp_read_mtx.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_longlong), C.POINTER(C.c_int),
                               C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_int)), C.POINTER(C.POINTER(C.c_float))]
    L.tsp_free_host.argtypes = [C.c_void_p]
    m, n, sym, nnz = C.c_int(), C.c_int(), C.c_int(), C.c_longlong()
    rp, ci, va = C.POINTER(C.c_int)(), C.POINTER(C.c_int)(), C.POINTER(C.c_float)()
    rc = L.tsp_read_mtx(path.encode(), C.byref(m), C.byref(n), C.byref(nnz), C.byref(sym), C.byref(rp), C.byref(ci), C.byref(va))
    if rc:
        return rc, L.tsp_last_error().decode()
    out = {"m": m.value, "n": n.value, "nnz": nnz.value, "symmetric": sym.value, "rowptr": [rp[i] for i in range(m.value + 1)],
           "colidx": [ci[i] for i in range(nnz.value)], "val": [float(va[i]) for i in range(nnz.value)]}
    for p in (rp, ci, va):
        L.tsp_free_host(C.cast(p, C.c_void_p))
    return 0, out


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_reader_matches_upstream_loader(name):
    rc, got = read(os.path.join(HERE, "golden", "mtx", name))
    assert rc == 0, got
    assert got == GOLDEN[name]


def test_reader_rejects_bad_files(tmp_path):
    bad = tmp_path / "bad.mtx"
    bad.write_text("%MatrixMarket matrix coordinate real general\n2 2 1\n1 1 1.0\n")      # one percent sign (src/mmio.h:19)
    rc, msg = read(str(bad))
    assert rc != 0 and "banner" in msg
    short = tmp_path / "short.mtx"
    short.write_text("%%MatrixMarket matrix coordinate real general\n3 3 4\n1 1 1.0\n2 2 2.0\n")
    rc, msg = read(str(short))
    assert rc != 0 and "ends after" in msg
    rc, msg = read(str(tmp_path / "missing.mtx"))
    assert rc != 0 and "cannot open" in msg
