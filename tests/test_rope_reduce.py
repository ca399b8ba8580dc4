"""CPU check: the closed-form sin/cos range reduction used by the append
kernel (wayruntime_b200/csrc/rope_reduce.h, plain C on the host side) returns
the bits of the reference's float loop (src/core/mathx.c:124-127) for every
RoPE angle of positions 0..39999 at theta 1e4 / 5e5 / 1e6, a stride through
all floats in [3, 2^18) and every binade edge."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_closed_form_reduction_matches_float_loop():
    exe = os.path.join(tempfile.mkdtemp(prefix="wr_rrc_"), "rope_reduce_check")
    subprocess.run(
        ["gcc", "-std=c11", "-O2", "-ffp-contract=off",
         "-I", os.path.join(ROOT, "wayruntime_b200", "csrc"), "-I", os.path.join(ROOT, "oracle"),
         os.path.join(ROOT, "tests", "rope_reduce_check.c"), os.path.join(ROOT, "oracle", "wr_oracle.c"),
         "-fopenmp", "-o", exe], check=True)
    res = subprocess.run([exe], stdout=subprocess.PIPE, text=True)
    assert res.returncode == 0, res.stdout
    assert "mismatches 0" in res.stdout
