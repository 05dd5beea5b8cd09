"""Collects the reference's own golden vectors for the training-step path into tests/golden/.

Run once where the reference checkout is mounted (it is not present where the
GPU tests run):  python tests/golden/make_golden.py <path to the ojas checkout>

Sources (all are test data of the reference, not code):
  ojas-cpu/tests/exact_golden.rs:206-276      FNV-1a digests of Exact outputs -> exact_golden_digests.json
  ojas-core/src/exp_exact_pins.txt            correctly rounded exp pins       -> exp_exact_pins.txt
  ojas-oracle/fixtures/tiny/*.safetensors     torch goldens of the tiny model  -> tiny/
  ojas-oracle/fixtures/tiny/{tokens.bin,batch_starts.json,lr_schedules.json,autocast_gap.json}
                                              inputs and side gates of the 40-step trainer traces -> tiny/
  ojas-oracle/fixtures/variants/*.safetensors GQA / sliding-window variants    -> variants/
  ojas-cpu/tests/torch_ref/data.rs            torch-2.13 bits, one-head step   -> torch_ref.json
"""
import json
import re
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def digests(ref: Path) -> None:
    text = (ref / "ojas-cpu/tests/exact_golden.rs").read_text()
    body = text[text.index("const GOLDEN"):]
    rows = re.findall(r'\("([^"]+)",\s*0x([0-9a-f]{16})\)', body)
    assert len(rows) == 69, len(rows)
    (HERE / "exact_golden_digests.json").write_text(json.dumps({k: v for k, v in rows}, indent=1) + "\n")


def torch_ref(ref: Path) -> None:
    text = (ref / "ojas-cpu/tests/torch_ref/data.rs").read_text()
    out = {}
    for name, body in re.findall(r"pub static (\w+): LazyLock<\[f32; \d+\]> = LazyLock::new\(\|\| \{\s*\[(.*?)\]\s*\}\);", text, re.S):
        out[name] = [int(b, 16) for b in re.findall(r"from_bits\(0x([0-9a-fA-F]+)\)", body)]
    for name, body in re.findall(r"pub static (\w+): \[u32; \d+\] = \[(.*?)\];", text, re.S):
        out[name] = [int(v) for v in re.findall(r"\d+", body)]
    for name, val in re.findall(r"pub static (\w+): LazyLock<f\d+> = LazyLock::new\(\|\| f\d+::from_bits\(0x([0-9a-fA-F]+)\)\);", text):
        out[name] = int(val, 16)
    (HERE / "torch_ref.json").write_text(json.dumps(out) + "\n")


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the ojas checkout>")
    ref = Path(sys.argv[1])
    digests(ref)
    shutil.copyfile(ref / "ojas-core/src/exp_exact_pins.txt", HERE / "exp_exact_pins.txt")
    (HERE / "tiny").mkdir(exist_ok=True)
    for name in ("init", "forward", "grads_init", "grads_step5", "trace_ns5_f32", "trace_ns5_bf16", "muon_step_bf16"):
        shutil.copyfile(ref / f"ojas-oracle/fixtures/tiny/{name}.safetensors", HERE / "tiny" / f"{name}.safetensors")
    # the trainer traces' inputs and side gates: the token stream and the sampler's window starts the 40 steps read, the
    # schedule multipliers, torch's own autocast gap on the trace, and the f64 RMSNorm fixture
    for name in ("tokens.bin", "batch_starts.json", "lr_schedules.json", "autocast_gap.json"):
        shutil.copyfile(ref / f"ojas-oracle/fixtures/tiny/{name}", HERE / "tiny" / name)
    (HERE / "variants").mkdir(exist_ok=True)
    for name in ("gqa", "swa"):
        shutil.copyfile(ref / f"ojas-oracle/fixtures/variants/{name}.safetensors", HERE / "variants" / f"{name}.safetensors")
    torch_ref(ref)


if __name__ == "__main__":
    main()
