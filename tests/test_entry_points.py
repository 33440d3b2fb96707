"""The repository's command-line entry points byte-compile and start on a machine without a
GPU (the driver imports them there), and the benchmark's helpers keep their contract."""
import json
import py_compile
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SCRIPTS = ["bench.py", "__graft_entry__.py", "baseline/compare_triton.py",
           "baseline/train_step_ab.py", "fast-attnres_b200/build.py", "tests/golden/make_golden.py"]


@pytest.mark.parametrize("script", SCRIPTS)
def test_script_compiles(script):
    py_compile.compile(str(ROOT / script), doraise=True)


def test_bench_help_lists_the_contract_flags():
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True,
                          text=True, timeout=300)
    assert done.returncode == 0, done.stderr
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--strong"):
        assert flag in done.stdout


def test_bench_algorithmic_bytes_and_peak():
    sys.path.insert(0, str(ROOT))
    import bench
    forward, backward = bench.algorithmic_bytes(49, 16384, 4096)
    assert forward == 16384 * (2 * 49 * 4096 + 2 * 4096)
    assert backward == 16384 * (4 * 49 * 4096 + 2 * 4096)
    assert forward + backward == 16384 * 1220608          # 6SD + 4D bytes per position
    peak, kind = bench.measured_peak_gbs()
    assert peak > 1000 and kind in ("measured", "fallback")
    ratios = bench.traffic_ratios()
    assert ratios and all(0.5 < ratio < 2.0 for ratio in ratios.values())
    assert set(ratios) <= {"stream", "stash", "ring"}
    assert json.loads((ROOT / "profiles" / "dram_traffic.json").read_text())["backward"]
    assert bench.backward_family(2, False) == "ring"
    assert bench.backward_family(9, False) == "stash"
    assert bench.backward_family(49, True) == "stream"
