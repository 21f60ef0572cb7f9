"""Tensor-core base conversion, host side: the planner's byte images and group tables (bconv_tc_plan.h) and the
kernel's reduction, emulated on the CPU against 128-bit integer arithmetic (tests/bconv_tc_emul.cpp)."""
import os
import subprocess
import tempfile

import pytest

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("seed", [1, 2026])
def test_planner_and_reduction_match_big_integer_arithmetic(seed):
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "bconv_tc_emul")
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-I" + os.path.join(_ROOT, "phantom-fhe_b200", "csrc"),
                               os.path.join(_ROOT, "tests", "bconv_tc_emul.cpp"), "-o", exe])
        out = subprocess.run([exe, str(seed)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.startswith("ok"), out.stdout + out.stderr
