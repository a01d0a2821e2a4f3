"""Builds and runs the global-to-shared copy probe (tests/probes/bulk_copy_issue_cost.cu): what a
page-sized chunk costs its issuing warp as one `cp.async.bulk` against 16-byte `cp.async` from 32
lanes. The decode kernel's ring uses the second; this keeps the measurement that decision rests
on reproducible. The test checks that every copy completed (status 0) and prints the table."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def test_probe_runs_and_every_copy_completes(tmp_path, capsys):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found on this machine")
    exe = str(tmp_path / "bulk_probe")
    src = os.path.join(HERE, "probes", "bulk_copy_issue_cost.cu")
    subprocess.run([nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a",
                    "-o", exe, src], check=True, capture_output=True, text=True, timeout=600)
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    with capsys.disabled():
        print("\n" + run.stdout)
    assert run.returncode == 0, run.stdout + run.stderr
    lines = [l for l in run.stdout.splitlines() if l.startswith("chunk")]
    assert len(lines) == 12
    for line in lines:
        assert line.rstrip().endswith("status 0")
        assert float(line.split("grid")[1].split("GB/s")[0]) > 100.0
