"""CPU check of the tensor-core engine's host-side plans: compiles tests/tc_emulator.cpp (an emulation of what TMA writes
to shared memory and what the tensor core reads from the canonical UMMA layouts) against the planner and runs every plan."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plans_reproduce_direct_convolution_and_gemm(tmp_path):
    exe = str(tmp_path / "tc_emulator")
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-o", exe, os.path.join(ROOT, "tests", "tc_emulator.cpp"),
                           os.path.join(ROOT, "lantern_b200", "csrc", "tc_plan.cpp")])
    out = subprocess.run([exe], stdout=subprocess.PIPE, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:]
    assert "0 failures" in out.stdout
