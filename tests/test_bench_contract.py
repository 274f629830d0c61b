"""The benchmark's output contract, checked on the CPU through its reference arm (the reference's
CPU operator on a tiny sample) and through the byte arithmetic both arms share."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_contract_line():
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3",
           "--cpu-prefill-seqs", "4", "--cpu-decode-seqs", "2", "--cpu-decode-steps", "1"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, "exactly one JSON line on stdout"
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["metric"] == "attn_algorithmic_bytes_per_s" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["vs_baseline"] is None and d["n_gpus"] == 1 and d["warmup"] >= 3
    assert "workload" in d["config"] and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"]
    assert abs(cb["value"] - d["value"]) <= 1e-9 * max(1.0, d["value"])
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["unit"] == d["unit"]
    assert d["value"] > 0 and d["ms_per_step"] > 0


def test_job_byte_arithmetic():
    sys.path.insert(0, str(ROOT))
    import bench
    rows, batch, steps = 1000, 8, 3
    E = bench.E
    # prefill: Q, K, V read once and O written once per packed row
    assert bench.prefill_bytes(rows) == 4 * rows * E * 4
    # a decode launch: K and V of every visible row (cache + the new block) once, q read, out written
    base = 512
    want = 2 * batch * (base + bench.N_NEW) * E * 4 + 2 * batch * bench.N_NEW * E * 4
    assert bench.decode_bytes(batch, base) == want
    total = bench.prefill_bytes(rows) + sum(bench.decode_bytes(batch, bench.BASE_LEN + bench.N_NEW * t) for t in range(steps))
    assert bench.job_bytes(rows, batch, steps) == total
    assert np.isfinite(total)


def test_reference_arm_on_other_ranks_does_nothing():
    import os
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(ROOT), env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
