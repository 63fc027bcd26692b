"""GPU test of the C++ host harness: golden files from oracle/make_ref.py (fp32 SDPA autograd on the CPU)
-> hopper_jeni_b200/gqa_bench -> loadBin / reportPrecision / checkResult gate / determinism probe / timing.
The binary must exit 0 when every gate holds and non-zero when the reference files are wrong."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "hopper_jeni_b200", "gqa_bench")


def _run(args, data):
    return subprocess.run([BENCH, *map(str, args), "--data", data, "--iters", "3", "--warmup", "1", "--runs", "1"],
                          capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("dims", [(1, 6, 2, 256, 64, 0), (1, 4, 2, 256, 128, 1)])
def test_cpp_harness_gates_against_fp32_sdpa(gqa_lib, tmp_path, dims):
    assert os.path.exists(BENCH), "build the harness with `python -m hopper_jeni_b200.build`"
    data = str(tmp_path / "data")
    subprocess.check_call([sys.executable, os.path.join(ROOT, "oracle", "make_ref.py"), *map(str, dims), "--out", data])
    out = _run(dims, data)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith('{"harness"')][-1])
    assert line["gate_pass"] is True and line["dkdv_bit_identical"] is True
    assert all(0 < line["rel_rms"][k] < 2e-2 for k in ("O", "dQ", "dK", "dV")), line["rel_rms"]
    # a corrupted reference must fail the gate and the exit code
    dv = np.fromfile(os.path.join(data, "gqa_dv.bin"), dtype=np.float32)
    (dv + 1.0).astype(np.float32).tofile(os.path.join(data, "gqa_dv.bin"))
    bad = _run(dims, data)
    assert bad.returncode == 4, bad.returncode


def test_cpp_harness_synthetic_mode_reports_no_gate(gqa_lib):
    """Without golden files nothing is compared: the JSON line must say so (gate_pass null, no rel_rms)."""
    out = subprocess.run([BENCH, "1", "4", "2", "256", "64", "0", "--synthetic", "--iters", "2", "--warmup", "1",
                          "--runs", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith('{"harness"')][-1])
    assert line["gate_pass"] is None and "rel_rms" not in line and line["outputs_finite"] is True
