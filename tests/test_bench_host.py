"""Host-side pieces of bench.py that need no GPU: the clock record and the reference arm's JSON line."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_clock_record_counts_only_lines_from_the_timed_region():
    bench = load_bench()
    s = bench.ClockSampler(0)
    line = "{}, 1965, 900.0, Not Active, Not Active, Not Active, {}"
    s.lines = [(10.0, line.format(1200, "Not Active")),      # warm-up
               (11.1, line.format(1650, "Active")), (11.2, line.format(1670, "Active")), (11.3, line.format(1660, "Active")),
               (12.5, line.format(1965, "Not Active")),      # after the timed region: idle boost clock
               (11.25, "garbage")]
    s.t0, s.t1 = 11.0, 11.4
    got = s.summary()
    assert got == {"sm_mhz": 1660.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    s.t0 = s.t1 = None                                       # never marked: everything counts
    assert s.summary()["samples"] == 5


def test_reference_arm_prints_the_contract_line_without_a_gpu():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["metric"] == "nanolab_gpt_124m_train_tokens_per_s" and line["value"] > 0
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and "sample" in line["cpu_baseline"]
