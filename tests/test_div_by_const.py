"""scores / sqrtf(head_dim) in the attention kernels is a product and two FMAs (div_by_const, csrc/mma_common.cuh)
instead of an IEEE division; the claim that both give the same bits is checked here on the CPU with the same
operations in C (fmaf is exact in glibc), over every 61st float by default and over every float with
LLMB_DIV_CHECK_ALL=1."""
import os
import shutil
import subprocess

from conftest import ROOT


def test_division_by_sqrt_head_dim_is_bit_exact(tmp_path):
    exe = os.path.join(str(tmp_path), "div_check")
    src = os.path.join(ROOT, "tests", "c_driver", "div_check.c")
    r = subprocess.run([shutil.which("gcc") or "gcc", "-O2", "-ffp-contract=off", "-Wall", "-Werror", src, "-o", exe, "-lm"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    stride = "1" if os.environ.get("LLMB_DIV_CHECK_ALL") == "1" else "61"
    r = subprocess.run([exe, stride], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count(" 0 mismatches") == 4, r.stdout
