"""The benchmark's reference arm (`bench.py --impl reference`): the reference's CPU path timed on the host cores.
Checked here on a reduced shape: exactly one JSON line on stdout with the keys the contract names, and under a
multi-rank launch only rank 0 works and prints."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
SMALL = ["--steps", "1", "--warmup", "0", "--ctx", "1024", "--layers", "1", "--batch", "2"]


def _run(extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference"] + SMALL, capture_output=True,
                       text=True, cwd=str(ROOT), env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return [ln for ln in r.stdout.splitlines() if ln.strip()]


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    lines = _run()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "decode_attn_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1 and d["vs_baseline"] is None
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("torch-restatement", "port", "reference") and cb["cores"] >= 1 and cb["sample"]
    assert cb["value"] == d["value"]
    assert d["config"]["workload"].startswith("config1")


def test_reference_arm_other_ranks_exit_without_work():
    lines = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert lines == []
