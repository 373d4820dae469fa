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


def test_conv_step_kernel_body_on_the_host(tmp_path):
    """``gdn_conv_step_kernel<4>``: window, weights, SiLU, the state left in the slot and the per-row state ring."""
    exe = tmp_path / "gdn_conv_emu"
    build = subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-DB200_EMU", "-I", str(ROOT / "tests/emu"), "-x", "c++",
                            str(ROOT / "tests/emu/gdn_conv_emu.cpp"), "-o", str(exe)], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.startswith("OK"), run.stdout + run.stderr


def test_expert_plan_kernels_on_the_host(tmp_path):
    """``ops/cuda/moe_plan.cuh``: 1024-thread CTAs (shared-memory histogram, two-level scans over warp shuffles,
    scatter through per-expert cursors, the ticket by which the last CTA of a grid builds the plan) as host C++."""
    exe = tmp_path / "plan_emu"
    build = subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-DB200_EMU", "-I", str(ROOT / "tests/emu"), "-x", "c++",
                            str(ROOT / "tests/emu/plan_emu.cpp"), "-o", str(exe)], capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and run.stdout.startswith("OK"), run.stdout + run.stderr


def _tsan_build(src, exe, defines=()):
    return subprocess.run(["g++", "-std=c++20", "-O1", "-g", "-pthread", "-fsanitize=thread", *defines, "-I", str(ROOT / "tests/emu"),
                           "-x", "c++", str(src), "-o", str(exe)], capture_output=True, text=True, timeout=600)


def test_emulated_kernels_have_no_data_race_and_a_missing_barrier_would_show(tmp_path):
    """The host builds of the device kernels under ThreadSanitizer (one std::thread per CUDA thread): no race in the
    GDN step kernel or in the router's row body. The control program shows what the check is worth: the same shim
    with a barrier left out is reported, with it is not."""
    import pytest

    control = tmp_path / "race_control"
    b = _tsan_build(ROOT / "tests/emu/race_control.cpp", control)
    if b.returncode != 0:
        pytest.skip("this toolchain has no ThreadSanitizer: " + b.stderr[-300:])
    ok = subprocess.run([str(control), "with-barrier"], capture_output=True, text=True, timeout=300)
    assert ok.returncode == 0 and "ThreadSanitizer" not in ok.stderr
    bad = subprocess.run([str(control), "without-barrier"], capture_output=True, text=True, timeout=300)
    assert "ThreadSanitizer: data race" in bad.stderr
    for name in ("gdn_step_emu", "gdn_conv_emu", "route_emu", "plan_emu"):
        exe = tmp_path / (name + "_tsan")
        b = _tsan_build(ROOT / f"tests/emu/{name}.cpp", exe, ("-DB200_EMU",))
        assert b.returncode == 0, b.stderr[-3000:]
        run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
        assert run.returncode == 0 and run.stdout.startswith("OK") and "ThreadSanitizer" not in run.stderr, run.stderr[-3000:]
