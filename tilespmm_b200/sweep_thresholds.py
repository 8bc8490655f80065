"""Sweep of the (gamma, delta) candidate pairs on the current GPU -- the measurement behind the rule in csrc/model.cu.

Upstream ships a frozen decision table (src/model.h) and no way to refit it.  This tool times every candidate pair of
upstream's candidate set (or a subset) on one or more benchmark configurations with THESE kernels: conversion on the
GPU, threshold tuning, then the mean of `--iters` SpMM passes.  It prints one line per candidate and the winner per
configuration; refit the rule in csrc/model.cu from its output when kernels or hardware change.

    python -m tilespmm_b200.sweep_thresholds c1 c2 c3 c4 [--scale S] [--iters 50] [--all]
"""
from __future__ import annotations

import argparse
import time

import numpy as np

GAMMAS = [1.0, 1.4, 1.8, 2.0, 2.4, 2.8, 3.0, 3.4, 3.8, 4.0]
DELTAS = [1.0, 1.2, 1.4, 1.5, 1.8, 2.0]
ALL = [(0.0, 1.5), (5.0, 0.0), (5.0, 3.0)] + [(g, d) for g in GAMMAS for d in DELTAS] + [(2.5, 1.0), (2.5, 1.2), (3.5, 1.0)]
SHORT = [(0.0, 1.5), (5.0, 0.0), (5.0, 3.0), (1.0, 1.0), (1.4, 1.0), (2.0, 1.0), (2.0, 1.2), (2.0, 2.0), (3.0, 1.0), (3.0, 1.5),
         (3.8, 1.0), (3.8, 2.0), (4.0, 1.0), (4.0, 1.5), (4.0, 2.0)]


def main():
    import torch
    from tilespmm_b200 import api, synth
    ap = argparse.ArgumentParser()
    ap.add_argument("configs", nargs="+", choices=sorted(synth.CONFIGS))
    ap.add_argument("--scale", type=int, default=None, help="R-MAT scale override for c3/c5")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--all", action="store_true", help="all 66 upstream candidates instead of the short list")
    args = ap.parse_args()
    for name in args.configs:
        kw = {"scale": args.scale} if (args.scale and name in ("c3", "c5")) else {}
        rp, ci, v, shape, cfg = synth.make_config(name, **kw)
        prec = 0 if cfg["precision"] == "fp16" else 1
        colB = cfg["colB"]
        cb = api.padded_width(colB)
        B = synth.dense_b(shape[1], cb, 1, cfg["b_dist"])
        Bv = api.to_values(B, prec).reshape(shape[1], cb)
        dB = torch.from_numpy(Bv.view(np.float16) if prec == 0 else Bv).cuda()
        vv = api.to_values(v, prec)
        d_rp, d_ci = torch.from_numpy(rp).cuda(), torch.from_numpy(ci).cuda()
        d_v = torch.from_numpy(vv.view(np.float16) if prec == 0 else vv).cuda()
        print(f"{name}: {shape[0]} x {shape[1]}, nnz {ci.size}, {cfg['precision']}, colB {colB}", flush=True)
        m = api.TileMatrix(prec)
        best = None
        for (g, d) in (ALL if args.all else SHORT):
            torch.cuda.synchronize()
            t = time.perf_counter()
            m.convert_device(shape, d_rp, d_ci, d_v, ci.size, g, d)
            conv_ms = (time.perf_counter() - t) * 1e3
            info = m.info()
            dC = torch.empty((m.c_rows(), cb), dtype=torch.float32, device="cuda")
            th, _ = m.tune(dB, dC, cb)
            ms = m.time(dB, dC, cb, args.iters)
            tf = 2.0 * ci.size * colB / ms / 1e9
            print(f"  gamma={g:<4} delta={d:<4} tiles(64/16/8)={info[:, 3].tolist()} th={th.tolist()} convert_ms={conv_ms:.1f} "
                  f"ms={ms:.4f} TFLOPS={tf:.2f}", flush=True)
            if best is None or ms < best[0]:
                best = (ms, g, d, tf)
            del dC
        print(f"  -> best for {name}: gamma={best[1]} delta={best[2]} ({best[0]:.4f} ms, {best[3]:.2f} TFLOPS)", flush=True)
        m.close()


if __name__ == "__main__":
    main()
