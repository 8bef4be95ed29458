"""The bench's own bookkeeping, checked without a GPU: the reference arm prints one JSON line with the contract's
keys (it times the CPU path of the reference, through the oracle, on a declared row sample), and the DRAM-traffic
figure the bench reports is the committed ncu capture scaled the way the summary says."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "dot_tflops" and line["unit"] == "TFLOP/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert "1/16 row sample" in line["config"]["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_recorded_traffic_scales_reads_and_row_sized_writes():
    sys.path.insert(0, ROOT)
    import bench
    small, full = bench.recorded_traffic(8192), bench.recorded_traffic(65536)
    assert small["traffic"] and full["traffic"]
    rec = None
    for ln in open(os.path.join(ROOT, "profiles", "mlp_step_gemm_dram_traffic.md")):
        if ln.startswith("TRAFFIC_JSON "):
            rec = json.loads(ln[len("TRAFFIC_JSON "):])
    total = sum(g["read"] + g["write"] for g in rec["launches"])
    assert abs(small["traffic"] - total / 8) < 1.0                       # the capture itself, per launch
    fixed = sum(g["write"] for g in rec["launches"] if g["rows_are"] == "K")
    assert abs(full["traffic"] - (8 * (total - fixed) + fixed) / 8) < 8.0   # dW results do not grow with the rows
    # algorithmic bytes of the eight GEMMs at the benchmark's size: each operand and result once
    assert abs(full["algorithmic_bytes_per_launch"] / 1e9 - 1.891) < 0.01
