"""The GDN decode-step kernel source compiled as host C++20 and run thread-per-lane against a float64 reference."""

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_gdn_step_kernel_body_on_the_host(tmp_path):
    exe = tmp_path / "gdn_step_emu"
    build = subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-DB200_EMU", "-I", str(ROOT / "tests/emu"), "-x", "c++",
                            str(ROOT / "tests/emu/gdn_step_emu.cpp"), "-o", str(exe)], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.startswith("OK"), run.stdout + run.stderr


def test_router_row_body_on_the_host(tmp_path):
    """``ops/cuda/moe_route.cuh`` (softmax, top-k with ties to the lower id, renormalised bf16 weights, expert map,
    counts) compiled as host C++: one std::thread per lane, shuffles through the shim, against float64."""
    exe = tmp_path / "route_emu"
    build = subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-DB200_EMU", "-I", str(ROOT / "tests/emu"), "-x", "c++",
                            str(ROOT / "tests/emu/route_emu.cpp"), "-o", str(exe)], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.startswith("OK"), run.stdout + run.stderr
