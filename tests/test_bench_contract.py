"""Host-side checks of bench.py that need no GPU: the reference arm prints one JSON line with the keys the contract names, and the
clock summary reads NVML (a fake one here) as documented."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_reference_arm_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["cpu_baseline"]["value"] == d["value"] and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and "sample" in d["cpu_baseline"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_other_ranks_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"], capture_output=True, text=True,
                       timeout=120, cwd=ROOT, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_clock_summary():
    """the sampler against a fake NVML (read-only queries; nothing is ever set): median clock, reasons seen at any sample, sample count"""
    class FakeNvml:
        NVML_CLOCK_SM = 1
        def __init__(self):
            self.i = 0
            self.clocks = [1800, 1750, 1700]
            self.reasons = [0x4, 0x4, 0x0]           # sw_power_cap on two of three samples
        def nvmlDeviceGetClockInfo(self, h, which):
            return self.clocks[self.i % 3]
        def nvmlDeviceGetPowerUsage(self, h):
            return 900000
        def nvmlDeviceGetCurrentClocksEventReasons(self, h):
            r = self.reasons[self.i % 3]; self.i += 1
            return r
    c = bench.ClockSampler(0)
    c.nvml, c.handle, c.max_mhz = FakeNvml(), object(), 1965.0
    c.sm, c.power, c.reason_bits = [], [], 0
    for _ in range(3):
        c.sample_nvml()
    s = c.summary()
    assert s["sm_mhz"] == 1750.0 and s["sm_min_mhz"] == 1700.0 and s["sm_max_mhz"] == 1965.0 and s["reasons"] == ["sw_power_cap"] and s["samples"] == 3
    assert s["power_w_max"] == 900.0
    c.reason_bits |= 0x40
    assert "hw_thermal_slowdown" in c.summary()["reasons"]
    c.sm = []
    assert c.summary()["sm_mhz"] is None


def test_algorithmic_bytes_constants():
    # one expert: gate|up 3 145 728 codes + 768 scale bytes, down 1 572 864 + 384
    assert bench.GU_BYTES == 3145728 + 768 and bench.DN_BYTES == 1572864 + 384
    assert np.isclose(128 * (bench.GU_BYTES + bench.DN_BYTES) + 2 * 256 * 2048 * 2, 606224384)
