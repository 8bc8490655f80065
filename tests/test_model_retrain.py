"""CPU tests of the threshold-model refit (tilespmm_b200/retrain_model.py): tree growth on sweep records, the emitted
table in upstream's node format, and the table walk."""
import json
import re

import numpy as np
import pytest

from tilespmm_b200 import retrain_model as rm


def _records():
    from tilespmm_b200 import retrain_model as r
    n = len(r.CANDIDATES)
    dense, sparse = r.CANDIDATES.index((0.0, 1.5)), r.CANDIDATES.index((3.8, 2.0))
    recs = []
    rng = np.random.default_rng(0)
    for i in range(12):
        heavy = i % 2 == 0                       # rows with many entries want 64-row tiles in this fabricated corpus
        avg = 200.0 + i if heavy else 8.0 + i
        ms = np.full(n, 1.0) + rng.uniform(0, 0.01, n)
        ms[dense if heavy else sparse] = 0.5
        feats = [0, 0, 65536, 65536, 65536 * avg, 1 - avg / 65536, avg, avg * 3, 1, 10.0, 128.0]
        recs.append({"name": f"case{i}", "precision": i % 4 // 2, "colB": 128, "features": feats, "ms": ms.tolist()})
    return recs, dense, sparse


def test_fit_splits_where_the_winner_changes_and_the_table_reproduces_it(tmp_path):
    from tilespmm_b200 import retrain_model as r
    recs, dense, sparse = _records()
    src = tmp_path / "sweep.jsonl"
    src.write_text("\n".join(json.dumps(x) for x in recs) + "\n")
    table = tmp_path / "model_table.inc"
    trees = r.fit([str(src)], depth=3, table_path=str(table))
    text = table.read_text()
    rows = re.findall(r"^\s*\{(-?\d+), (-?\d+), (-?\d+), (-?\d+), (-?\d+), (-?\d+), (-?\d+), (\d+), ([-0-9.e+]+)f, ([-0-9.e+]+)f, ([-0-9.e+]+)f\},", text, flags=re.M)
    roots = {0: int(re.search(r"kPolicyRootFp16 = (-?\d+);", text).group(1)), 1: int(re.search(r"kPolicyRootTf32 = (-?\d+);", text).group(1))}
    nodes = [{"feature": int(a), "left_feature": int(b), "right_feature": int(c), "child": [int(d), int(e), int(f), int(g)], "mask": int(h),
              "cut": float(i), "left_cut": float(j), "right_cut": float(k)} for a, b, c, d, e, f, g, h, i, j, k in rows]
    assert nodes and all(t[0] == "node" for t in trees.values())
    for x in recs:
        got = r.walk(nodes, roots[x["precision"]], x["features"])
        assert got == (dense if x["features"][6] > 100 else sparse)
    # NaN features follow missing_left_mask (0 here: to the right), like upstream's walk
    f = list(recs[0]["features"])
    f[nodes[roots[0]]["feature"] + 2] = float("nan")
    assert r.walk(nodes, roots[0], f) in (dense, sparse)


def test_no_gain_no_split(tmp_path):
    from tilespmm_b200 import retrain_model as r
    recs, _, sparse = _records()
    for x in recs:                                # every candidate equally good: the default pair must be kept
        x["ms"] = [1.0] * len(x["ms"])
    src = tmp_path / "flat.jsonl"
    src.write_text("\n".join(json.dumps(x) for x in recs) + "\n")
    trees = r.fit([str(src)], depth=3, table_path=str(tmp_path / "t.inc"))
    assert trees == {0: ("leaf", sparse), 1: ("leaf", sparse)}


def test_shipped_table_answers_a_candidate_through_the_c_abi():
    from tilespmm_b200 import api, retrain_model as r
    f = [0, 0, 4096.0, 4096.0, 65536.0, 1 - 16 / 4096, 16.0, 16.0, 16.0, 10.0, 32.0]
    for prec in (0, 1):
        g, d = api.predict(prec, f)
        assert (round(g, 1), round(d, 1)) in r.CANDIDATES


# ---------------------------------------------------------------- the C walker (csrc/model.cu) itself

def _c_walk(nodes, root, features):
    """tsp_policy_walk over a table given as a list of node dicts (retrain_model's format) -> candidate number or None."""
    import ctypes as C
    from tilespmm_b200 import api
    L = api.lib()
    L.tsp_policy_walk.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    raw = np.zeros((max(len(nodes), 1), 11), dtype=np.int32)
    for i, n in enumerate(nodes):
        raw[i, :8] = [n["feature"], n["left_feature"], n["right_feature"], *n["child"], n["mask"]]
        raw[i, 8:] = np.array([n["cut"], n["left_cut"], n["right_cut"]], dtype=np.float32).view(np.int32)
    f = np.ascontiguousarray(features, dtype=np.float64)
    g, d = C.c_float(0), C.c_float(0)
    rc = L.tsp_policy_walk(raw.ctypes.data_as(C.c_void_p), len(nodes), root, f.ctypes.data_as(C.c_void_p), C.byref(g), C.byref(d))
    if rc != 0:
        return None
    cands = [(np.float32(a), np.float32(b)) for a, b in rm.CANDIDATES]
    return cands.index((np.float32(g.value), np.float32(d.value)))


def _random_table(rng, nnodes):
    """A well-formed table in upstream's node format: children point to earlier nodes or leaves; about half of the sides
    carry a second feature; every missing_left_mask combination occurs."""
    nodes = []
    for i in range(nnodes):
        def child():
            return int(rng.integers(0, i)) if (i > 0 and rng.random() < 0.6) else -1 - int(rng.integers(0, 66))
        nodes.append({"feature": int(rng.integers(0, 9)), "left_feature": int(rng.integers(0, 9)) if rng.random() < 0.5 else -1,
                      "right_feature": int(rng.integers(0, 9)) if rng.random() < 0.5 else -1, "child": [child(), child(), child(), child()],
                      "mask": int(rng.integers(0, 8)), "cut": float(rng.normal()), "left_cut": float(rng.normal()), "right_cut": float(rng.normal())})
    return nodes


def test_c_walker_matches_the_python_walk_on_random_tables_with_second_levels_and_nans():
    rng = np.random.default_rng(123)
    checked = nan_routes = second = 0
    for _ in range(40):
        nodes = _random_table(rng, int(rng.integers(1, 40)))
        root = len(nodes) - 1
        for _ in range(60):
            f = np.concatenate([[0.0, 0.0], rng.normal(size=9)])
            f[2 + rng.integers(0, 9, size=int(rng.integers(0, 4)))] = np.nan          # missing features take the mask's side
            f[2 + int(rng.integers(0, 9))] = nodes[root]["cut"]                            # a value exactly on a cut goes right
            want = rm.walk(nodes, root, f)
            assert _c_walk(nodes, root, f) == want
            checked += 1
            nan_routes += int(np.isnan(f).any())
            second += int(nodes[root]["left_feature"] >= 0 or nodes[root]["right_feature"] >= 0)
    assert checked == 2400 and nan_routes > 500 and second > 500


def test_c_walker_refuses_malformed_tables():
    ok = {"feature": 0, "left_feature": -1, "right_feature": -1, "child": [-1, -1, -2, -2], "mask": 0, "cut": 0.0, "left_cut": 0.0, "right_cut": 0.0}
    f = np.zeros(11)
    assert _c_walk([ok], 0, f) == 1                                                     # 0.0 < 0.0 is false: right side, leaf 1
    assert _c_walk([dict(ok, child=[0, 0, 0, 0])], 0, f) is None                        # a loop
    assert _c_walk([dict(ok, child=[5, 5, 5, 5])], 0, f) is None                        # a child outside the table
    assert _c_walk([dict(ok, child=[-100, -100, -100, -100])], 0, f) is None            # a leaf outside the candidates
    assert _c_walk([dict(ok, feature=12)], 0, f) is None                                # a feature outside the vector
    assert _c_walk([], -4, f) == 3                                                      # a bare leaf as the root


def test_c_walker_reproduces_upstream_on_upstreams_own_table():
    """The 800 golden answers were produced by upstream's tilespmm_policy_select (src/model.h:3463-3491) on upstream's table.
    The product's walker, run over that same table (read from oracle/_ref, which compiles upstream's model.h where it
    lies), must give the same answers -- this pins the walk semantics on a 3421-node table with second-level tests."""
    import ctypes as C
    import json
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    lib = os.path.join(os.path.dirname(here), "oracle", "_ref", "libref_model_table.so")
    if not os.path.exists(lib):
        pytest.skip("oracle/_ref/libref_model_table.so is not built (needs the upstream checkout)")
    from tilespmm_b200 import api
    R = C.CDLL(lib)
    R.ref_model_nodes.restype = C.c_void_p
    n, nb, r16, r32 = C.c_int(0), C.c_int(0), C.c_int(0), C.c_int(0)
    table = R.ref_model_nodes(C.byref(n), C.byref(nb), C.byref(r16), C.byref(r32))
    assert nb.value == 44 and n.value > 3000
    L = api.lib()
    L.tsp_policy_walk.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    golden = json.load(open(os.path.join(here, "golden", "tiling_golden.json")))["model"]
    assert len(golden) == 800
    answers = set()
    for rec in golden:
        f = np.array(rec["features"], dtype=np.float64)
        g, d = C.c_float(0), C.c_float(0)
        rc = L.tsp_policy_walk(C.c_void_p(table), n.value, r32.value if rec["precision"] else r16.value, f.ctypes.data_as(C.c_void_p), C.byref(g), C.byref(d))
        assert rc == 0 and (g.value, d.value) == (np.float32(rec["gamma"]), np.float32(rec["delta"])), rec
        answers.add((g.value, d.value))
    assert len(answers) >= 5                                                            # not a constant function


@pytest.mark.gpu
def test_sweep_leg_times_candidates_on_the_gpu_and_the_fit_consumes_its_records(tmp_path):
    """The measuring half of the refit: two small corpus cases, four candidates (one per class mix), real conversions,
    tuning and timed loops on the GPU; the records it writes are what `fit` reads."""
    out = tmp_path / "sweep.jsonl"
    picks = [rm.CANDIDATES.index(c) for c in ((0.0, 1.5), (5.0, 0.0), (5.0, 3.0), (2.0, 1.2))]
    rm.sweep(str(out), iters=5, cases={"fixed_4096x16", "stencil_32"}, candidates=picks)
    recs = [json.loads(l) for l in open(out)]
    assert [r["name"] for r in recs] == ["fixed_4096x16", "stencil_32"]
    for r in recs:
        assert len(r["ms"]) == len(rm.CANDIDATES) and all(t > 0 for t in r["ms"]) and len(r["features"]) == 11
        assert len({r["ms"][i] for i in picks}) >= 2                 # different tilings were really timed
    table = tmp_path / "table.inc"
    trees = rm.fit([str(out)], depth=2, table_path=str(table))
    assert set(trees) == {0, 1} and "kPolicyNodes" in table.read_text()
