"""CPU tests of the threshold-model refit (tilespmm_b200/retrain_model.py): tree growth on sweep records, the emitted
table in upstream's node format, and the table walk."""
import json
import re

import numpy as np


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
