"""The quantizers divide by the block scale through its correctly rounded reciprocal and two fused residual corrections
(delta_matching_b200/csrc/dm_quant.cu, quotient_rn).  That sequence must carry the bits of the IEEE division the
reference's quantizers perform (producers.py:149-204 divide element by element); tests/quotient_identity.c checks it on
the host with the C library's fmaf, over every bf16 significand against a stride of the scale's significands and over
random 24-bit operands."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_reciprocal_quotient_equals_division(tmp_path):
    exe = str(tmp_path / "quotient_identity")
    # -ffp-contract=off: the division and the products must not be fused by the compiler; fmaf is the only fusion
    subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-o", exe, os.path.join(HERE, "quotient_identity.c"), "-lm"])
    out = subprocess.run([exe, "61", "20000000"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:]
    assert "mismatches 0" in out.stdout
