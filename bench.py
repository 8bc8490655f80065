#!/usr/bin/env python
"""Benchmark of the TileSpMM hot path on B200: SpMM TFLOPS = 2*nnz*colB/t (upstream src/csr2tile.h:1057).

    python bench.py --gpus N --steps K --warmup W            this library (CUDA, C ABI)
    python bench.py --impl reference ...                      CPU CSR SpMM of the checker on the host cores

One "step" is one SpMM pass (all tile classes) over the resident converted matrix.  The loop of K steps is repeated
back to back (at least 5 times and for at least 1.5 s, so that clocks and power settle and can be sampled while it
runs) and the reported time is the median loop.

Workloads (`--workload`, default `auto`):
  auto  on one GPU of a one-GPU box: benchmark configuration 2 (27-point stencil on 64^3, TF32, colB=128) as the
        headline, with configurations 1, 3 and 4 measured the same way under `per_config`.  With more than one GPU --
        `--gpus N` > 1, or `--gpus 1` on a box that shows several GPUs, i.e. the first point of a scaling run --
        configuration 5 (symmetric R-MAT scale 24, FP16, colB=128, generated on the GPU): ONE matrix whose panels
        are cut across the N ranks ("strong" scaling), B replicated once over NCCL, C row-partitioned.
  c1..c5  that configuration; `c2` on N > 1 ranks stacks the stencil N times along z (fixed work per GPU, "weak").
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tilespmm_b200 import synth  # noqa: E402

PREC = {"fp16": 0, "tf32": 1}
MIN_TIMED_S = 1.5
C5_CPU_SAMPLE = 8          # the CPU arm multiplies every 8th block of 1024 rows of configuration 5

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the class kernel that dominates the workload, from
# the ncu captures summarised under profiles/ (key: workload, tile class).  Only used when the live run picked the
# same tiling as the capture (`tiles` must match), otherwise the roofline falls back to the compulsory bytes.
TRAFFIC = {
    ("c2", 2): {"bytes": 363.8e6, "tiles": 376872, "source": "profiles/c2_spmm_8row_tf32.md"},
    ("c2", 0): {"bytes": 281.4e6, "tiles": 144400, "source": "profiles/c2_spmm_64row_tf32_tcgen05.md"},
    ("c3", 2): {"bytes": 1019.6e6, "tiles": 1849624, "source": "profiles/c3_spmm_8row_fp16.md"},
    ("c4", 2): {"bytes": 2210.4e6, "tiles": 235936, "source": "profiles/c4_spmm_8row_64row_tf32.md"},
}


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def describe(name: str, world: int, scale=None) -> str:
    if name == "c1":
        return "c1: 4096^2, 16 nnz/row, FP16, colB=32"
    if name == "c2":
        return f"c2: 27-point stencil 64x64x{64 * world}, TF32, colB=128"
    if name == "c3":
        return f"c3: symmetric R-MAT scale {scale or 20}, FP16, colB=64"
    if name == "c4":
        return "c4: mixed density 524288^2, TF32, colB=256"
    return f"c5: symmetric R-MAT scale {scale or 24}, FP16, colB=128 (generated on the GPU)"


def make_workload(name: str, n_gpus: int, scale=None):
    """Host CSR (float32 values) and shape of one benchmark configuration (c1..c4)."""
    if name == "c2":
        return synth.stencil27(64, 1002) if n_gpus == 1 else stencil_stacked(64, 64 * n_gpus, 1002)
    if name == "c1":
        return synth.fixed_nnz_per_row(4096, 16, 1001)
    if name == "c3":
        return synth.rmat_symmetric(scale or 20, 16, 1003)
    if name == "c4":
        return synth.mixed_density(524288, 1004)
    raise SystemExit(f"workload {name} is generated on the device")


def stencil_stacked(g: int, gz: int, seed: int):
    """27-point stencil on a g x g x gz grid (x fastest), same value law as configuration 2."""
    rng = np.random.Generator(np.random.Philox(seed))
    n = g * g * gz
    idx = np.arange(n, dtype=np.int64)
    x, y, z = idx % g, (idx // g) % g, idx // (g * g)
    rows, cols, diag = [], [], []
    for dz in (-1, 0, 1):
        for dy in (-1, 0, 1):
            for dx in (-1, 0, 1):
                ok = (x + dx >= 0) & (x + dx < g) & (y + dy >= 0) & (y + dy < g) & (z + dz >= 0) & (z + dz < gz)
                r = idx[ok]
                rows.append(r); cols.append(r + dx + dy * g + dz * g * g)
                diag.append(np.full(r.shape, dx == 0 and dy == 0 and dz == 0))
    rows, cols, diag = np.concatenate(rows), np.concatenate(cols), np.concatenate(diag)
    order = np.lexsort((cols, rows))
    rows, cols, diag = rows[order], cols[order], diag[order]
    vals = np.where(diag, 26.0, -1.0) + rng.uniform(-1e-3, 1e-3, size=rows.size)
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(rowptr, rows + 1, 1)
    return np.cumsum(rowptr).astype(np.int32), cols.astype(np.int32), vals.astype(np.float32), (n, n)


def resolve_workload(requested: str, world: int) -> str:
    if requested != "auto":
        return requested
    visible = 1
    try:
        import torch
        visible = torch.cuda.device_count()
    except Exception:
        pass
    return "c5" if (world > 1 or visible > 1) else "c2"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.stop_flag, self.thread = index, [], False, None

    def _loop(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=10)
        sm = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        pw = [float(s[2]) for s in self.samples if len(s) > 2 and s[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(s) > 3 + i and s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "power_w_max": max(pw) if pw else None, "samples": len(self.samples), "sampled": "during the timed loops"}


# ----------------------------------------------------------------------------------------------------------------
# baselines that run beside the product (never inside its timed region)

def _checker():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import _orc
    _orc.Orc.lib().orc_set_threads(os.cpu_count() or 1)      # torchrun sets OMP_NUM_THREADS=1; use every host core
    return _orc


def cpu_csr_spmm_timed(prec, shape, rp, ci, vv, Bv, colB, budget_s=12.0):
    """The CPU baseline: the checker's OpenMP CSR SpMM on all host threads, best of a few passes."""
    _orc = _checker()
    best, t_total, n = None, 0.0, 0
    while n < 2 or (t_total < budget_s and n < 8):
        t0 = time.perf_counter()
        _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, colB)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        t_total += dt
        n += 1
    return best, n, int(_orc.Orc.lib().orc_num_threads())


def upstream_gpu_leg(name, prec, shape, rp, ci, vv, Bv, colB, cb, device):
    """Upstream's own kernels (its unmodified sources compiled for sm_100a under oracle/_ref) on the same GPU, in a child
    process, through upstream's call_tilespmm_cuda: its model, its conversion, its tuning, its 1000-pass timed loop."""
    lib = os.path.join(ROOT, "oracle", "_ref", f"libref_{'tf32' if prec else 'fp16'}.so")
    if not os.path.exists(lib):
        return {"unavailable": "oracle/_ref is not built (needs the upstream checkout at build time)"}
    with tempfile.TemporaryDirectory() as tmp:
        np.save(os.path.join(tmp, "rp.npy"), rp); np.save(os.path.join(tmp, "ci.npy"), ci)
        np.save(os.path.join(tmp, "vv.npy"), vv); np.save(os.path.join(tmp, "b.npy"), Bv)
        cmd = [sys.executable, os.path.join(ROOT, "oracle", "upstream_gpu_leg.py"), tmp, str(prec), str(shape[0]), str(shape[1]),
               str(colB), str(cb), str(device)]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        except subprocess.TimeoutExpired:
            return {"unavailable": "upstream's driver did not finish within 600 s"}
    if r.returncode != 0:
        return {"unavailable": f"upstream's driver exited with {r.returncode}: {r.stderr.strip()[-200:]}"}
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {"unavailable": "upstream's driver printed no result"}


def cusparse_leg(api, prec, shape, rp, ci, vv, Bv, colB, device):
    out3, _ = api.cusparse_baseline(prec, shape, rp, ci, vv, Bv, colB, device=device, warmup=20, repeat=100, want_c=False)
    cus = {"time_ms": float(out3[1]), "tflops": float(out3[2]), "alg": "CUSPARSE_SPMM_ALG_DEFAULT"}
    others = {}   # a stronger cuSPARSE baseline, reported beside upstream's choice: the best of CSR_ALG1..3
    for alg in (1, 2, 3):
        try:
            o3, _ = api.cusparse_baseline(prec, shape, rp, ci, vv, Bv, colB, device=device, warmup=20, repeat=100, want_c=False, alg=alg)
            others[f"CUSPARSE_SPMM_CSR_ALG{alg}"] = float(o3[2])
        except api.TileSpMMError:
            pass
    if others:
        best_alg = max(others, key=others.get)
        cus["best_other_alg"] = {"alg": best_alg, "tflops": others[best_alg]}
    return cus


# ----------------------------------------------------------------------------------------------------------------
# the reference arm

def c5_row_sample(scale: int):
    """Configuration 5 for the CPU arm: the matrix is generated on the GPU (the host generator needs minutes at this
    size), then every C5_CPU_SAMPLE-th block of 1024 rows is brought to the host together with the whole of B."""
    import torch
    d_rp, d_ci, d_v, shape = synth.rmat_symmetric_device(scale, 16, 1005, values="u01")
    n = shape[0]
    # R-MAT rows are heaviest where the index has many zero bits, so a regular stride would favour heavy (or light) blocks:
    # the blocks are drawn by a fixed multiplicative hash instead, about one in C5_CPU_SAMPLE
    allb = torch.arange(0, n // 1024, device="cuda", dtype=torch.int64)
    blocks = allb[((allb * 2654435761) >> 13) % C5_CPU_SAMPLE == 0]
    rows = (blocks[:, None] * 1024 + torch.arange(1024, device="cuda")[None, :]).reshape(-1)
    rp64 = d_rp.to(torch.int64)
    lens = rp64[rows + 1] - rp64[rows]
    out_rp = torch.zeros(rows.numel() + 1, dtype=torch.int64, device="cuda")
    out_rp[1:] = torch.cumsum(lens, 0)
    total = int(out_rp[-1].item())
    src = torch.repeat_interleave(rp64[rows] - out_rp[:-1], lens) + torch.arange(total, device="cuda")
    ci, v = d_ci[src].cpu().numpy(), d_v[src].to(torch.float16).cpu().numpy().view(np.uint16)
    gB = torch.Generator(device="cuda")
    gB.manual_seed(7)
    B = (torch.rand((shape[1], 128), generator=gB, device="cuda", dtype=torch.float32) * 2 - 1).to(torch.float16).cpu().numpy().view(np.uint16)
    return out_rp.to(torch.int32).cpu().numpy(), ci, v, (int(rows.numel()), shape[1]), B


def run_reference(args):
    """--impl reference: upstream has no CPU SpMM (its check compares against cuSPARSE, src/main.cu:315-335), so
    the reference arm is the checker's CPU CSR SpMM (FP32 accumulate) on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    name = resolve_workload(args.workload, max(world, args.gpus))
    from tilespmm_b200 import api
    cfg = synth.CONFIGS[name]
    prec, colB = PREC[cfg["precision"]], cfg["colB"]
    cb = api.padded_width(colB)
    if name == "c5":
        rp, ci, vv, shape, Bv = c5_row_sample(args.scale or 24)
        sample = (f"one in {C5_CPU_SAMPLE} blocks of 1024 rows, drawn by a fixed hash ({shape[0]} rows, {ci.size} entries) against the whole B; "
                  "matrix and B generated on GPU 0, the product runs on the host cores")
    else:
        rp, ci, v, shape = make_workload(name, 1, args.scale)
        B = synth.dense_b(shape[1], cb, 1, cfg["b_dist"])
        Bv = api.to_values(B, prec).reshape(shape[1], cb)
        vv = api.to_values(v, prec)
        sample = "whole workload, one pass per step"
    _orc = _checker()
    for _ in range(args.warmup):
        _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, colB)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _orc.spmm_csr(prec, shape, rp, ci, vv, Bv, colB)
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 2.0 * ci.size * colB / dt / 1e12
    threads = int(_orc.Orc.lib().orc_num_threads())
    line = {"impl": "reference", "metric": "spmm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong" if name != "c2" else "weak",
            "vs_baseline": None, "dtype": cfg["precision"], "data": "synthetic",
            "config": {"workload": describe(name, 1, args.scale)},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------------
# this library

class Ctx:
    pass


def measure(name: str, cx, headline: bool):
    """Converts, tunes and times one configuration on this rank's GPU.  Returns the record of the configuration."""
    import torch
    from tilespmm_b200 import api, multi
    args, world, rank, local, dist = cx.args, cx.world, cx.rank, cx.local, cx.dist
    cfg = synth.CONFIGS[name]
    prec, colB = PREC[cfg["precision"]], cfg["colB"]
    cb = api.padded_width(colB)
    tdt = torch.float16 if prec == 0 else torch.float32
    on_device = name == "c5"            # ~500 M nonzeros: generated on the GPU, converted from device memory

    if on_device:
        d_rp, d_ci, d_v, shape = synth.rmat_symmetric_device(args.scale or 24, 16, 1005, values="u01")
        d_v = d_v.to(torch.float16) if prec == 0 else d_v
        rp = d_rp.cpu().numpy()
        ci = vv = None
        nnz = int(d_ci.numel())
    else:
        rp, ci, v, shape = make_workload(name, world, args.scale)
        nnz = int(ci.size)
        vv = api.to_values(v, prec)

    # threshold model (upstream src/main.cu:226-247), conversion on the GPU
    cap = torch.cuda.get_device_capability(local)
    gamma, delta = api.predict(prec, api.features_from_csr(rp, shape, cap[0] + cap[1] / 10.0, colB))
    if args.gamma is not None:
        gamma = args.gamma
    if args.delta is not None:
        delta = args.delta
    sm = multi.ShardedTileMatrix(prec, dist, local)
    torch.cuda.synchronize()
    convert_ms = []
    if not on_device:
        # the CSR as a performance-minded caller holds it: in pinned host memory, so that its upload runs at PCIe speed
        pinned = [torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in (rp, ci, vv.view(np.int16) if prec == 0 else vv)]
        rp_p, ci_p = pinned[0].numpy(), pinned[1].numpy()
        vv_p = pinned[2].numpy().view(np.uint16) if prec == 0 else pinned[2].numpy()
    for _ in range(1 if on_device else 3):   # the first conversion also creates the library's workspace
        t0 = time.perf_counter()
        if on_device:
            sm.convert_device(shape, d_rp, d_ci, d_v, nnz, gamma, delta)
        else:
            sm.convert_host(shape, rp_p, ci_p, vv_p, gamma, delta)
        torch.cuda.synchronize()
        convert_ms.append((time.perf_counter() - t0) * 1e3)
    if on_device:
        del d_ci, d_v
        torch.cuda.empty_cache()
    m, info = sm.m, sm.info
    row0, row1 = sm.row_range

    # B: generated on rank 0, replicated once over NCCL; C: this rank's row slab
    B_pinned = Bv = None
    if rank == 0 and on_device:
        gB = torch.Generator(device="cuda")
        gB.manual_seed(7)
        dB = (torch.rand((shape[1], cb), generator=gB, device="cuda", dtype=torch.float32) * 2 - 1).to(tdt)
    elif rank == 0:
        Bh = synth.dense_b(shape[1], cb, 1, cfg["b_dist"])
        Bh[:, colB:] = 0
        Bv = api.to_values(Bh, prec).reshape(shape[1], cb)
        B_pinned = torch.from_numpy(Bv.view(np.float16) if prec == 0 else Bv).pin_memory()
        dB = B_pinned.to("cuda", non_blocking=True)
    else:
        dB = torch.empty((shape[1], cb), dtype=tdt, device="cuda")
    bcast_ms = None
    if world > 1:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        e0.record()
        multi.broadcast_dense(dB, dist, src=0)
        e1.record()
        torch.cuda.synchronize()
        bcast_ms = e0.elapsed_time(e1)
    dC = torch.empty((m.c_rows(), cb), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()

    if args.th:
        best_th, tune_ms = [int(x) for x in args.th.split(",")], 0.0
        for cls in range(3):
            if info[cls, 2] > 0:
                m.schedule(cls, best_th[cls])
    else:
        best_th, tune_ms = m.tune(dB, dC, cb)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed loops: `repeats` loops of K steps back to back, median loop reported
    stream = torch.cuda.current_stream().cuda_stream
    K = args.steps
    ew0, ew1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ew0.record()
    for _ in range(args.warmup):
        m.spmm(dB, dC, cb, stream)
    ew1.record()
    barrier()
    est_ms = multi.max_over_ranks(max(ew0.elapsed_time(ew1) / args.warmup, 1e-3), dist, "cuda")
    min_s = args.min_seconds if headline else min(0.4, args.min_seconds)
    repeats = int(min(max(5, math.ceil(min_s * 1e3 / (est_ms * K))), 5000))
    launches0 = m.launch_count()
    sampler = ClockSampler(local) if (headline and rank == 0) else None
    if sampler:
        sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
    barrier()
    for a, b in evs:
        a.record()
        for _ in range(K):
            m.spmm(dB, dC, cb, stream)
        b.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    loop_ms = sorted(a.elapsed_time(b) for a, b in evs)
    launches = m.launch_count() - launches0
    ms_step = multi.max_over_ranks(float(np.median(loop_ms)), dist, "cuda") / K
    tflops = 2.0 * nnz * colB / (ms_step * 1e-3) / 1e12

    # ---- per-class kernel timing and the roofline of the dominant kernel (CUDA events on the launching stream)
    cls_ms, cls_bytes = {}, {}
    for cls in range(3):
        if info[cls, 2] > 0:
            cls_ms[cls] = m.time(dB, dC, cb, max(20, min(200, K * repeats // 4)), cls)
            cls_bytes[cls] = m.algorithmic_bytes(cb, cls)
    peak, peak_kind = measured_peak_gbs()
    roofline = None
    if cls_ms:
        dom = max(cls_ms, key=lambda c: cls_ms[c])
        b3 = cls_bytes[dom]
        vsz = 2 if prec == 0 else 4
        # what HBM has to move at least: the class's tiles and indices once, the rows of B it touches once (at most
        # the gathered bytes, at most all of B), its rows of C once
        compulsory = float(m.tile_bytes(dom) + min(b3[1], float(shape[1]) * cb * vsz) + b3[2])
        tr = TRAFFIC.get((name, dom))
        traffic = tr["bytes"] if (tr and world == 1 and int(info[dom, 3]) == tr["tiles"]) else None
        basis = traffic if traffic else compulsory
        ach = basis / (cls_ms[dom] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": f"{api.CLASSES[dom]}-row tiles", "kernel_ms": cls_ms[dom], "achieved": ach, "peak": peak,
                    "peak_kind": peak_kind, "unit": "GB/s", "frac": ach / peak, "frac_of_nominal_8TBs": ach / 8000.0,
                    "basis": (f"DRAM bytes of one launch measured with ncu ({tr['source']})" if traffic else
                              "compulsory bytes: tile data as stored + indices once, touched rows of B once, C once"),
                    "traffic": traffic, "compulsory_bytes": compulsory,
                    "algorithmic": {"a_tiles": float(b3[0]), "b_gathered": float(b3[1]), "c": float(b3[2]),
                                    "gbs": float(b3.sum()) / (cls_ms[dom] * 1e-3) / 1e9,
                                    "note": "upstream tile format; the gathered rows of B are mostly L2 hits, so this rate is not bounded by HBM"},
                    "class_ms": {str(api.CLASSES[c]): cls_ms[c] for c in cls_ms}}

    rec = {"workload": describe(name, world, args.scale), "precision": cfg["precision"], "rows": int(shape[0]), "nnz": nnz, "colB": colB,
           "ms": ms_step, "tflops": tflops, "loops": repeats, "loop_ms_min_median_max": [loop_ms[0] / K, float(np.median(loop_ms)) / K, loop_ms[-1] / K],
           "gamma": gamma, "delta": delta, "tiles_64_16_8": [int(x) for x in info[:, 3]], "best_th": [int(x) for x in best_th],
           "tune_ms": tune_ms, "broadcast_b_ms": bcast_ms, "roofline": roofline, "gpu_launches": int(launches),
           "slab_rows": [int(row0), int(row1)]}
    csr_bytes = (shape[0] + 1) * 4.0 + nnz * (4.0 + (2 if prec == 0 else 4))
    tile_bytes = float(m.tile_bytes()) + float(info[:, 2].sum() + info[:, 3].sum()) * 4.0
    conv_ms = min(convert_ms)
    rec["convert"] = {"ms": conv_ms, "first_call_ms": convert_ms[0], "includes": "device CSR" if on_device else "upload of the host CSR from pinned memory",
                      "algorithmic_bytes": csr_bytes + tile_bytes, "frac": (csr_bytes + tile_bytes) / (conv_ms * 1e-3) / 1e9 / peak}

    # ---- end to end with host buffers: upload of B, kernels, download of C inside the timed region
    if headline and world == 1:
        # one GPU: the C ABI's host-buffer entry points; consecutive steps use the library's two staging slots, so that
        # one step's download overlaps the next step's upload
        import ctypes as C
        if B_pinned is None:
            B_pinned = dB.cpu().pin_memory()
        Bnp = B_pinned.numpy()
        outs = [torch.empty((row1 - row0, cb), dtype=torch.float32).pin_memory() for _ in range(2)]
        L = api.lib()

        def e2e_steps(n):
            for i in range(n):
                slot = i & 1
                if i >= 2:
                    api._check(L.tsp_spmm_host_wait(m.h, slot), "tsp_spmm_host_wait")
                api._check(L.tsp_spmm_host_async(m.h, C.c_void_p(Bnp.ctypes.data), C.c_void_p(outs[slot].data_ptr()), cb, slot),
                           "tsp_spmm_host_async")
            for slot in (0, 1):
                api._check(L.tsp_spmm_host_wait(m.h, slot), "tsp_spmm_host_wait")

        h2d, path = int(Bnp.nbytes), "tsp_spmm_host_async / tsp_spmm_host_wait (C ABI, pinned host buffers, two staging slots)"
    elif headline:
        # N GPUs: every rank uploads only its own 1/N row block of B from pinned host memory, the ranks all-gather the
        # blocks over NCCL, multiply and download their slab of C; consecutive steps alternate between two streams
        # and two buffer sets
        per = multi.b_block_rows(shape[1], world)
        lo, hi = sm.b_block()
        Bblk = torch.empty((per, cb), dtype=tdt).pin_memory()
        Bblk[:hi - lo].copy_(dB[lo:hi])
        outs = [torch.empty((row1 - row0, cb), dtype=torch.float32).pin_memory() for _ in range(2)]
        streams = [torch.cuda.Stream(), torch.cuda.Stream()]
        torch.cuda.synchronize()

        def e2e_steps(n):
            for i in range(n):
                with torch.cuda.stream(streams[i & 1]):
                    sm.spmm_host(Bblk, outs[i & 1], cb, slot=i & 1)
            torch.cuda.synchronize()

        h2d, path = int((hi - lo) * cb * (2 if prec == 0 else 4)), ("ShardedTileMatrix.spmm_host: pinned row block of B -> H2D -> all-gather "
                                                                     "over NCCL -> tsp_spmm -> D2H of the C slab")
    if headline:
        e2e_steps(2)
        n_e2e = args.e2e_steps if nnz < 100_000_000 else max(4, args.e2e_steps // 2)
        barrier()
        t0 = time.perf_counter()
        e2e_steps(n_e2e)
        torch.cuda.synchronize()
        dt = multi.max_over_ranks((time.perf_counter() - t0) / n_e2e, dist, "cuda")
        rec["e2e"] = {"value": 2.0 * nnz * colB / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": int((row1 - row0) * cb * 4), "ms_per_step": dt * 1e3, "steps": n_e2e,
                      "bytes_are": "per rank" if world > 1 else "total", "path": path}
        del outs

    # ---- baselines beside it, outside every timed region (one GPU, host-generated workloads)
    if rank == 0 and world == 1 and not on_device:
        if not args.no_cusparse:
            rec["cusparse"] = cusparse_leg(api, prec, shape, rp, ci, vv, Bv, colB, local)
        if not args.no_upstream:
            rec["upstream_gpu"] = upstream_gpu_leg(name, prec, shape, rp, ci, vv, Bv, colB, cb, local)
            # the same matrix through THIS library under upstream's own protocol (tsp_run = call_tilespmm_cuda: clock-stabilised
            # warm-up, tuning, then 1000 passes timed as one interval), so that the two times are like for like
            out6, _ = m.run(Bv, cb, colB, repeat=1000, want_c=False)
            rec["upstream_protocol"] = {"time_ms": float(out6[4]), "tflops": float(out6[5]), "best_th": [int(x) for x in out6[:3]]}
            if rec["upstream_gpu"].get("time_ms"):
                rec["upstream_protocol"]["speedup_vs_upstream_gpu"] = rec["upstream_gpu"]["time_ms"] / float(out6[4])
        if headline and not args.no_cpu:
            best, n, threads = cpu_csr_spmm_timed(prec, shape, rp, ci, vv, Bv, colB)
            rec["cpu_baseline"] = {"value": 2.0 * nnz * colB / best / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                   "sample": f"whole workload, best of {n} passes ({best * 1e3:.1f} ms)"}
    rec["clocks"] = clocks
    sm.close()
    del dB, dC
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--scale", type=int, default=None, help="R-MAT scale override for c3/c5")
    ap.add_argument("--gamma", type=float, default=None)
    ap.add_argument("--delta", type=float, default=None)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-cusparse", action="store_true")
    ap.add_argument("--no-upstream", action="store_true", help="skip the leg that runs upstream's own kernels")
    ap.add_argument("--no-per-config", action="store_true", help="headline workload only")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_S,
                    help="shortest total length of the timed loops of the headline workload (0: five loops; for profiling runs)")
    ap.add_argument("--th", default=None, help="th64,th16,th8: fixed thresholds, skips the on-GPU tuning (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    cx = Ctx()
    cx.args = args
    cx.world = int(os.environ.get("WORLD_SIZE", "1"))
    cx.rank = int(os.environ.get("RANK", "0"))
    cx.local = int(os.environ.get("LOCAL_RANK", "0"))
    if cx.world != args.gpus and cx.world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={cx.world}")
    torch.cuda.set_device(cx.local)
    cx.dist = None
    if cx.world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", cx.local))
        cx.dist = dist

    name = resolve_workload(args.workload, cx.world)
    head = measure(name, cx, headline=True)
    per_config = {}
    if cx.world == 1 and name == "c2" and args.workload == "auto" and not args.no_per_config:
        for other in ("c1", "c3", "c4"):
            per_config[other] = measure(other, cx, headline=False)

    if cx.rank == 0:
        cfg = synth.CONFIGS[name]
        scaling = "weak" if name == "c2" else "strong"
        config = {"workload": head["workload"], "rows": head["rows"], "nnz": head["nnz"], "colB": head["colB"], "gamma": head["gamma"],
                  "delta": head["delta"], "tiles_64_16_8": head["tiles_64_16_8"], "best_th": head["best_th"],
                  "l2": "working set (A tiles + B + C) larger than L2; no flush", "tune_ms": head["tune_ms"],
                  "broadcast_b_ms": head["broadcast_b_ms"], "convert": head["convert"],
                  "timing": f"median of {head['loops']} back-to-back loops of {args.steps} steps (CUDA events, max over ranks)",
                  "loop_ms_per_step_min_median_max": head["loop_ms_min_median_max"]}
        line = {"metric": "spmm_tflops", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": cx.world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
                "dtype": cfg["precision"], "data": "synthetic", "config": config, "roofline": head["roofline"],
                "cpu_baseline": head.get("cpu_baseline"), "cusparse": head.get("cusparse"), "upstream_gpu": head.get("upstream_gpu"),
                "upstream_protocol": head.get("upstream_protocol"),
                "clocks": head["clocks"], "e2e": head.get("e2e"), "gpu_launches": head["gpu_launches"],
                "per_config": {k: {kk: vv for kk, vv in v.items() if kk not in ("clocks",)} for k, v in per_config.items()} or None}
        print(json.dumps(line))
    if cx.world > 1:
        cx.dist.barrier()
        cx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
