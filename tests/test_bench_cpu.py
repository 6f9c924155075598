"""CPU: the reference arm of bench.py (the reference's PyTorch path where an unpacked copy of the reference is present,
else its CPU restatement, timed on host cores) prints exactly one JSON line on stdout with the contract's keys, also
when a library writes to file descriptor 1 behind Python's back."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_json_line():
    env = dict(os.environ, OMP_NUM_THREADS="4")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "decode_e32",
                        "--steps", "1", "--warmup", "0"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["value"] > 0 and d["higher_is_better"] is True and d["n_gpus"] == 1
    # "reference" = the reference's own binding.py ran (baseline/_ref is present), "port" = the C restatement
    has_ref = (ROOT / "baseline" / "_ref" / "solution" / "cuda" / "binding.py").is_file()
    assert d["cpu_baseline"]["kind"] == ("reference" if has_ref else "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0
