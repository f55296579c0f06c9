"""The packers' division for fp16 / bf16 weights (a correctly rounded reciprocal and one fused
correction instead of the division instruction sequence) gives the same 4-bit codes as IEEE division
for every operand pair: enumerated on the host by tests/exact_division_check.c."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("arg", [[], ["bf16"]], ids=["fp16", "bf16"])
def test_every_operand_pair(tmp_path, arg):
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    try:
        has_fma = " fma " in open("/proc/cpuinfo").read()
    except OSError:
        has_fma = False
    if not has_fma:
        pytest.skip("the host CPU has no fused multiply-add: a software fmaf makes the enumeration take too long")
    exe = str(tmp_path / "exact_division_check")
    subprocess.run([gcc, "-O2", "-mfma", "-o", exe, os.path.join(HERE, "exact_division_check.c"), "-lm"], check=True)
    r = subprocess.run([exe, *arg], stdout=subprocess.PIPE, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-400:]
    assert " 0 mismatches" in r.stdout
