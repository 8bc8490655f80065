"""CPU tests of bench.py's contract: the reference arm prints one JSON line with the agreed keys, and the workload rule."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_agreed_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-800:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "spmm_tflops" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["steps"] == 2 and d["warmup"] == 1 and d["n_gpus"] == 1 and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"].startswith("c1")
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_workload_rule():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.resolve_workload("c3", 1) == "c3" and bench.resolve_workload("c2", 8) == "c2"
    assert bench.resolve_workload("auto", 2) == "c5"
    # one rank on a box without several GPUs: the headline configuration
    import torch
    if torch.cuda.device_count() <= 1:
        assert bench.resolve_workload("auto", 1) == "c2"
    # every captured traffic figure names the summary it comes from
    for key, rec in bench.TRAFFIC.items():
        assert os.path.exists(os.path.join(ROOT, rec["source"])), rec["source"]
        assert rec["bytes"] > 0 and rec["tiles"] > 0


def test_every_profile_summary_names_its_command():
    """profiles/ holds text summaries only, each with the command that produced it (committed files only)."""
    pdir = os.path.join(ROOT, "profiles")
    names = sorted(os.listdir(pdir))
    assert names and all(n.endswith((".md", ".txt")) for n in names), names
    for n in names:
        text = open(os.path.join(pdir, n)).read()
        assert "Command" in text and ("bench.py" in text), n
        assert "_work" not in text and "gpurun" not in text, n
