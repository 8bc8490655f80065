"""Refit of the threshold model on the current GPU: corpus -> sweep of the 66 candidate pairs -> decision table.

Upstream ships a frozen table (src/model.h: 3421 nodes fitted to its kernels on other GPUs) and nothing that could
produce another one.  This tool is that missing half for THESE kernels:

  sweep   times every (gamma, delta) candidate of upstream's candidate set (src/model.h:14-38) on a seeded synthetic
          corpus (fixed-degree, stencil, R-MAT, mixed-density matrices; both precisions; several dense widths) with
          GPU conversion, threshold tuning and a timed SpMM loop, and writes one JSON record per case.  Candidates
          that produce the same tiling share one measurement.
  fit     grows a small decision tree over the 9 live features of upstream's 11-slot feature vector
          (src/model_features.h:31-57) that minimises the summed regret t(chosen) / t(best) over the corpus, and
          writes it in upstream's node format ({feature, left_feature, right_feature, child0..3, missing_left_mask,
          cut, left_cut, right_cut}, negative child = leaf -1-index into the candidate table) as
          csrc/model_table.inc, which csrc/model.cu walks.

    python -m tilespmm_b200.retrain_model sweep --out sweep.jsonl        # needs the GPU
    python -m tilespmm_b200.retrain_model fit sweep.jsonl                # CPU only; rewrites csrc/model_table.inc
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

# upstream's candidate table in upstream's order (src/model.h:14-38): index = leaf number
GAMMAS = [1.0, 1.4, 1.8, 2.0, 2.4, 2.8, 3.0, 3.4, 3.8, 4.0]
DELTAS = [1.0, 1.2, 1.4, 1.5, 1.8, 2.0]
CANDIDATES = [(0.0, 1.5), (5.0, 0.0), (5.0, 3.0)] + [(g, d) for g in GAMMAS for d in DELTAS] + [(2.5, 1.0), (2.5, 1.2), (3.5, 1.0)]

HERE = os.path.dirname(os.path.abspath(__file__))
TABLE = os.path.join(HERE, "csrc", "model_table.inc")
DEFAULT_LEAF = CANDIDATES.index((3.8, 2.0))
FEATURE_NAMES = ["rowA", "colA", "nnzA", "sparsity", "avg_row_nnz", "max_row_nnz", "min_row_nnz", "capability", "colB"]


def corpus():
    """(name, generator call, precision, colB) of the seeded training cases."""
    from . import synth
    c = []
    c.append(("fixed_4096x16", lambda: synth.fixed_nnz_per_row(4096, 16, seed=21), 0, 32))
    c.append(("fixed_65536x8", lambda: synth.fixed_nnz_per_row(65536, 8, seed=22), 1, 64))
    c.append(("fixed_16384x64", lambda: synth.fixed_nnz_per_row(16384, 64, seed=23), 0, 128))
    c.append(("fixed_8192x160", lambda: synth.fixed_nnz_per_row(8192, 160, seed=24), 1, 128))
    c.append(("stencil_32", lambda: synth.stencil27(32, seed=25), 1, 128))
    c.append(("stencil_48", lambda: synth.stencil27(48, seed=26), 0, 64))
    c.append(("rmat_16", lambda: synth.rmat_symmetric(16, seed=27), 0, 64))
    c.append(("rmat_17", lambda: synth.rmat_symmetric(17, seed=28), 1, 128))
    c.append(("mixed_65536_d10", lambda: synth.mixed_density(65536, seed=29, dense_fraction=0.1), 1, 256))
    c.append(("mixed_65536_d50", lambda: synth.mixed_density(65536, seed=30, dense_fraction=0.5), 0, 128))
    c.append(("mixed_32768_d90", lambda: synth.mixed_density(32768, seed=31, dense_fraction=0.9, blocks_per_panel=8), 1, 128))
    c.append(("mixed_32768_dense_fp16", lambda: synth.mixed_density(32768, seed=32, dense_fraction=0.9, blocks_per_panel=8, density=0.9), 0, 256))
    # the same families at the sizes of the benchmark configurations
    c.append(("fixed_262144x16", lambda: synth.fixed_nnz_per_row(262144, 16, seed=33), 1, 128))
    c.append(("stencil_64", lambda: synth.stencil27(64, seed=34), 1, 128))
    c.append(("stencil_64_fp16", lambda: synth.stencil27(64, seed=35), 0, 256))
    c.append(("rmat_19", lambda: synth.rmat_symmetric(19, seed=36), 0, 64))
    c.append(("rmat_19_tf32", lambda: synth.rmat_symmetric(19, seed=37), 1, 128))
    c.append(("mixed_262144_d10", lambda: synth.mixed_density(262144, seed=38, dense_fraction=0.1), 1, 256))
    c.append(("mixed_262144_d50", lambda: synth.mixed_density(262144, seed=39, dense_fraction=0.5), 0, 128))
    c.append(("mixed_131072_d90", lambda: synth.mixed_density(131072, seed=40, dense_fraction=0.9, blocks_per_panel=8), 1, 128))
    c.append(("mixed_131072_dense_fp16", lambda: synth.mixed_density(131072, seed=41, dense_fraction=0.9, blocks_per_panel=8, density=0.9), 0, 64))
    # banded and block-diagonal structure (rows that share their columns), more dense widths
    c.append(("banded_131072_hb12", lambda: synth.banded(131072, 12, 0.6, seed=42), 1, 128))
    c.append(("banded_131072_hb40_fp16", lambda: synth.banded(131072, 40, 0.5, seed=43), 0, 64))
    c.append(("banded_262144_hb4", lambda: synth.banded(262144, 4, 0.9, seed=44), 1, 32))
    c.append(("blockdiag_65536_b64", lambda: synth.block_diagonal(65536, 64, 0.3, seed=45), 1, 256))
    c.append(("blockdiag_131072_b32_fp16", lambda: synth.block_diagonal(131072, 32, 0.5, seed=46), 0, 128))
    c.append(("blockdiag_32768_b128", lambda: synth.block_diagonal(32768, 128, 0.15, seed=47), 1, 64))
    c.append(("stencil_40_c32", lambda: synth.stencil27(40, seed=48), 1, 32))
    c.append(("rmat_17_fp16_c256", lambda: synth.rmat_symmetric(17, seed=49), 0, 256))
    return c


def sweep(out_path: str, iters: int, cases=None, candidates=None):
    """Times the candidates on the corpus.  `cases` (names) and `candidates` (indices into CANDIDATES) restrict the sweep;
    a candidate that is not timed gets the time of the default pair."""
    import torch
    from . import api, synth
    picked = set(range(len(CANDIDATES))) if candidates is None else set(candidates) | {DEFAULT_LEAF}
    with open(out_path, "w") as out:
        for name, gen, prec, colB in corpus():
            if cases is not None and name not in cases:
                continue
            rp, ci, v, shape = gen()
            cb = api.padded_width(colB)
            B = synth.dense_b(shape[1], cb, 1, "uniform")
            Bv = api.to_values(B, prec).reshape(shape[1], cb)
            dB = torch.from_numpy(Bv.view(np.float16) if prec == 0 else Bv).cuda()
            vv = api.to_values(v, prec)
            d_rp, d_ci = torch.from_numpy(rp).cuda(), torch.from_numpy(ci).cuda()
            d_v = torch.from_numpy(vv.view(np.float16) if prec == 0 else vv).cuda()
            feats = api.features_from_csr(rp, shape, 10.0, colB)
            m = api.TileMatrix(prec)
            seen, times = {}, []
            t_case = time.perf_counter()
            for index, (g, d) in enumerate(CANDIDATES):
                if index not in picked:
                    times.append(None)
                    continue
                m.convert_device(shape, d_rp, d_ci, d_v, ci.size, g, d)
                info = m.info()
                key = tuple(int(x) for x in info[:, [0, 3]].ravel())   # rows and tiles per class
                if key not in seen:
                    dC = torch.empty((m.c_rows(), cb), dtype=torch.float32, device="cuda")
                    m.tune(dB, dC, cb)
                    # best of three loops: one disturbed loop (another tenant of the machine, a clock event) must not reach the fit
                    seen[key] = min(m.time(dB, dC, cb, iters) for _ in range(3))
                    del dC
                times.append(seen[key])
            times = [t if t is not None else times[DEFAULT_LEAF] for t in times]
            m.close()
            rec = {"name": name, "precision": prec, "colB": colB, "features": [float(x) for x in feats], "ms": times}
            out.write(json.dumps(rec) + "\n")
            out.flush()
            best = int(np.argmin(times))
            print(f"{name}: prec {prec} colB {colB}: {len(seen)} distinct tilings, best {CANDIDATES[best]} {times[best]:.4f} ms, "
                  f"default {times[DEFAULT_LEAF]:.4f} ms ({time.perf_counter() - t_case:.1f} s)", flush=True)


# ---------------------------------------------------------------- fit

def _regret(cases, leaf):
    return sum(c["ms"][leaf] / min(c["ms"]) for c in cases)


def _best_leaf(cases):
    tot = np.zeros(len(CANDIDATES))
    for c in cases:
        tot += np.asarray(c["ms"]) / min(c["ms"])
    # ties and near-ties (candidates with the same tiling on every case, or within the 0.5 % run-to-run noise of the
    # timings) go to the default pair, then to the lowest index
    best = int(np.argmin(tot))
    if tot[DEFAULT_LEAF] <= tot[best] * 1.005:
        best = DEFAULT_LEAF
    return best, float(tot[best])


def grow(cases, depth, min_gain=0.005, min_leaf=2):
    """Binary tree as nested tuples: ("leaf", index) or ("node", feature, cut, left, right); value < cut goes left.
    A split must buy `min_gain` of mean regret and leave at least `min_leaf` cases on either side: one matrix is no
    evidence for a rule."""
    leaf, cost = _best_leaf(cases)
    if depth == 0 or len(cases) < 2:
        return ("leaf", leaf), cost
    best = None
    for f in range(len(FEATURE_NAMES)):
        vals = sorted({np.float32(c["features"][f + 2]) for c in cases})
        for lo, hi in zip(vals, vals[1:]):
            cut = np.float32((float(lo) + float(hi)) / 2)
            left = [c for c in cases if np.float32(c["features"][f + 2]) < cut]
            right = [c for c in cases if not np.float32(c["features"][f + 2]) < cut]
            if len(left) < min_leaf or len(right) < min_leaf:
                continue
            cl = _best_leaf(left)[1] + _best_leaf(right)[1]
            if best is None or cl < best[0]:
                best = (cl, f, float(cut), left, right)
    if best is None or best[0] > cost - min_gain * len(cases):     # a split must buy min_gain of mean regret
        return ("leaf", leaf), cost
    lt, lc = grow(best[3], depth - 1, min_gain, min_leaf)
    rt, rc = grow(best[4], depth - 1, min_gain, min_leaf)
    if lc + rc > cost - min_gain * len(cases):
        return ("leaf", leaf), cost
    return ("node", best[1], best[2], lt, rt), lc + rc


def flatten(tree):
    """Nodes in upstream's format, children before parents; returns (nodes, index of the root or a negative leaf)."""
    nodes = []

    def emit(t):
        if t[0] == "leaf":
            return -1 - t[1]
        l, r = emit(t[3]), emit(t[4])
        # a plain binary node: no second-level features, so child0 serves the left side and child2 the right side
        nodes.append({"feature": t[1], "left_feature": -1, "right_feature": -1, "child": [l, l, r, r], "mask": 0,
                      "cut": t[2], "left_cut": 0.0, "right_cut": 0.0})
        return len(nodes) - 1

    root = emit(tree)
    return nodes, root


def walk(nodes, index, features):
    """The same walk as csrc/model.cu, for checking a table on the CPU."""
    while index >= 0:
        n = nodes[index]
        v = np.float32(features[n["feature"] + 2])
        left = (n["mask"] & 1) != 0 if np.isnan(v) else bool(v < np.float32(n["cut"]))
        if left:
            if n["left_feature"] < 0:
                index = n["child"][0]
            else:
                v = np.float32(features[n["left_feature"] + 2])
                l2 = (n["mask"] & 2) != 0 if np.isnan(v) else bool(v < np.float32(n["left_cut"]))
                index = n["child"][0] if l2 else n["child"][1]
        else:
            if n["right_feature"] < 0:
                index = n["child"][2]
            else:
                v = np.float32(features[n["right_feature"] + 2])
                l2 = (n["mask"] & 4) != 0 if np.isnan(v) else bool(v < np.float32(n["right_cut"]))
                index = n["child"][2] if l2 else n["child"][3]
    return -1 - index


def _lit(v) -> str:
    """C float literal that round-trips a float32."""
    t = f"{np.float32(v):.9g}"
    if not any(ch in t for ch in ".en"):
        t += ".0"
    return t + "f"


def write_table(path, trees, note):
    """trees: {precision: tree}.  One shared node array, one root per precision (like upstream's shared table)."""
    nodes, roots = [], {}
    for prec in (0, 1):
        n, r = flatten(trees[prec])
        off = len(nodes)
        for x in n:
            x["child"] = [c + off if c >= 0 else c for c in x["child"]]
        nodes += n
        roots[prec] = r + off if r >= 0 else r
    L = ["// Generated by `python -m tilespmm_b200.retrain_model fit`; do not edit by hand.", f"// {note}",
         "// Node format of upstream's table (src/model.h:9-13): feature f reads features[f + 2] as float; value < cut goes",
         "// left; a side with a second feature tests it too; a negative child is leaf -1-index into the candidate table.",
         "static const TspPolicyNode kPolicyNodes[] = {"]
    for x in nodes:
        c = x["child"]
        L.append(f"    {{{x['feature']}, {x['left_feature']}, {x['right_feature']}, {c[0]}, {c[1]}, {c[2]}, {c[3]}, {x['mask']}, "
                 f"{_lit(x['cut'])}, {_lit(x['left_cut'])}, {_lit(x['right_cut'])}}},")
    if not nodes:
        L.append("    {0, -1, -1, -1, -1, -1, -1, 0, 0.0f, 0.0f, 0.0f},   // placeholder: both roots are leaves")
    L += ["};", f"static const int kPolicyRootFp16 = {roots[0]};", f"static const int kPolicyRootTf32 = {roots[1]};", ""]
    with open(path, "w") as fh:
        fh.write("\n".join(L))
    return nodes, roots


def fit(paths, depth: int, table_path: str = TABLE):
    cases = []
    for p in paths:
        cases += [json.loads(l) for l in open(p) if l.strip()]
    trees, report = {}, []
    for prec in (0, 1):
        sub = [c for c in cases if c["precision"] == prec]
        if sub:
            tree, cost = grow(sub, depth)
            base = _regret(sub, DEFAULT_LEAF)
            report.append(f"precision {prec}: {len(sub)} cases, mean regret {cost / len(sub):.4f} (single rule (3.8, 2.0): {base / len(sub):.4f})")
        else:
            tree = ("leaf", DEFAULT_LEAF)
            report.append(f"precision {prec}: no cases, leaf (3.8, 2.0)")
        trees[prec] = tree
    note = "Fitted on " + ", ".join(sorted({c["name"] for c in cases})) if cases else "No sweep data: both roots answer (3.8, 2.0)."
    nodes, roots = write_table(table_path, trees, note[:400])
    for prec in (0, 1):       # the emitted table must reproduce the tree's answers
        for c in (x for x in cases if x["precision"] == prec):
            want = trees[prec]
            while want[0] == "node":
                want = want[3] if np.float32(c["features"][want[1] + 2]) < np.float32(want[2]) else want[4]
            assert walk(nodes, roots[prec], c["features"]) == want[1]
    print("\n".join(report))
    print(f"wrote {table_path}: {len(nodes)} nodes, roots {roots}")
    return trees


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("sweep")
    s.add_argument("--out", default="sweep.jsonl")
    s.add_argument("--iters", type=int, default=30)
    f = sub.add_parser("fit")
    f.add_argument("records", nargs="*")
    f.add_argument("--depth", type=int, default=3)
    args = ap.parse_args()
    if args.cmd == "sweep":
        sweep(args.out, args.iters)
    else:
        fit(args.records, args.depth)


if __name__ == "__main__":
    sys.exit(main())
