"""GPU test of the two drop-in executables: arguments, exit codes, the 19-field CSV row without header and the
check message of upstream's main (src/main.cu:136-352)."""
import os
import subprocess

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def write_mtx(path, rows, cols, seed):
    rng = np.random.default_rng(seed)
    ents = {(int(rng.integers(1, rows + 1)), int(rng.integers(1, cols + 1))) for _ in range(rows * 9)}
    with open(path, "w") as f:
        f.write("%" + "%MatrixMarket matrix coordinate real general\n")
        f.write("%d %d %d\n" % (rows, cols, len(ents)))
        for i, j in sorted(ents, key=lambda e: (e[1], e[0])):      # column-major file order: rows come out unsorted
            f.write("%d %d %.3f\n" % (i, j, rng.normal()))
    return len(ents)


@pytest.mark.parametrize("exe,colB,csv", [("tilespmm_fp16", 32, "TileSpMM-FP16.csv"), ("tilespmm_tf32", 100, "TileSpMM-TF32.csv")])
def test_cli_row_and_check(tmp_path, exe, colB, csv):
    path = os.path.join(ROOT, "tilespmm_b200", "bin", exe)
    mtx = str(tmp_path / "m.mtx")
    nnz = write_mtx(mtx, 777, 640, 5)
    for _ in range(2):                                             # rows are appended, never a header
        r = subprocess.run([path, "-d", "0", mtx, str(colB)], cwd=tmp_path, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "Check... PASS!" in r.stdout
        assert "padded colB = %d" % (32 if colB <= 32 else (colB + 63) // 64 * 64) in r.stdout
    lines = open(tmp_path / csv).read().splitlines()
    assert len(lines) == 2
    f = lines[0].split(",")
    assert len(f) == 19
    assert f[0] == mtx and [int(x) for x in f[1:5]] == [777, 640, nnz, colB]
    assert sum(int(x) for x in f[5:8]) > 0                          # tilenum64, tilenum16, tilenum8
    assert all(float(x) > 0 for x in f[13:19])                      # pre_time, time, tflops, cusparse pre, time, tflops


def test_cli_usage_and_bad_width(tmp_path):
    path = os.path.join(ROOT, "tilespmm_b200", "bin", "tilespmm_fp16")
    r = subprocess.run([path, "-x", "0"], capture_output=True, text=True)
    assert r.returncode == 1 and r.stdout.startswith("Usage:")
    mtx = str(tmp_path / "m.mtx")
    write_mtx(mtx, 64, 64, 1)
    r = subprocess.run([path, "-d", "0", mtx, "0"], cwd=tmp_path, capture_output=True, text=True)
    assert r.returncode == 1 and "colB must be positive" in r.stderr
