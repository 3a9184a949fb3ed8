"""The benchmark's reference arm runs on CPU and prints one JSON line with the contract's keys."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def test_reference_arm_prints_the_contract_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                           "--warmup", "1", "--cpu-seconds", "1"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"].startswith("paged KV append+gather")
    assert line["unit"] == "GB/s" and line["higher_is_better"] is True and line["value"] > 0
    assert line["steps"] == 2 and line["warmup"] == 1 and line["n_gpus"] == 1 and line["vs_baseline"] is None
    assert line["config"]["workload"] == "llama3-8b-decode"
    import bench

    assert line["config"] == bench.decode_config(1)          # the words the GPU arm's line uses too
    base = line["cpu_baseline"]
    from oracle import ref_python

    # the reference's own byte-compiled CPU path when oracle/_ref holds it, else the oracle's restatement
    assert base["kind"] == ("reference" if ref_python.built() else "port")
    assert base["cores"] >= 1 and base["value"] == line["value"] and "sample" in base
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_other_ranks_of_the_reference_arm_exit_quietly():
    import os

    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2"],
                          capture_output=True, text=True, timeout=120, env=env)
    assert proc.returncode == 0 and proc.stdout.strip() == ""
