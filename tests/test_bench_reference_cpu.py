"""CPU: the reference arm of bench.py (the torch CPU path of the same workload) runs without a
GPU, prints the contract's JSON line, and maps none of this repository's native libraries."""
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_line_and_no_native_libraries():
    code = r"""
import runpy, sys
sys.argv = ["bench.py", "--impl", "reference", "--steps", "1", "--warmup", "0"]
try:
    runpy.run_path(%r, run_name="__main__")
except SystemExit as e:
    assert not e.code, e.code
mapped = [l.split()[-1] for l in open("/proc/self/maps") if l.rstrip().endswith(".so")]
ours = [p for p in mapped if "libiex_" in p or "iex_oracle" in p]
print("NATIVE", ours)
""" % os.path.join(REPO, "bench.py")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    res = subprocess.run([sys.executable, "-c", code], cwd=REPO, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "spmm_sddmm_gflops" and d["unit"] == "GFLOP/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1 and d["gpu_launches"] == 0
    assert d["value"] > 0 and d["e2e"]["value"] == d["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert "cfg2" in d["config"]["workload"]
    assert "NATIVE []" in res.stdout, res.stdout[-500:]
