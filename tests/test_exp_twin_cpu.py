"""The device exp's algorithm, restated in C with the same constants and operation order, against glibc expf on the
host: at most 1 ulp apart on every sampled float32 (every 61st bit pattern here; `exp_sweep 1` checks all 2.2e9 and
finds the same bound with 99.5 % of the inputs bit-equal).  The constants are read back out of the kernel generator so
that the twin cannot drift away from what the device runs."""
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_exp_twin_stays_within_one_ulp_of_glibc_and_uses_the_generators_constants(tmp_path):
    exe = tmp_path / "exp_sweep"
    subprocess.check_call(["gcc", "-O2", "-o", str(exe), os.path.join(ROOT, "tests", "exp_sweep.c"), "-lm"])
    out = subprocess.run([str(exe), "61"], capture_output=True, text=True, timeout=600, check=True).stdout.splitlines()
    fields = out[0].split()
    stats = dict(zip(fields[0::2], (int(v) for v in fields[1::2])))
    assert stats["max_ulp"] == 1 and stats["worse"] == 0 and stats["specials_ok"] == 1
    assert stats["equal"] / (stats["equal"] + stats["off_by_one"]) > 0.99
    generator = open(os.path.join(ROOT, "pytorch-rs_b200", "csrc", "pointwise_plan.cpp")).read()
    fast = generator[generator.index("__device__ __forceinline__ float trs_exp(float x)"):]
    fast = fast[:fast.index("\n}\n")]
    for hexword in out[1].split()[5:]:
        assert f"__uint_as_float({hexword}u)" in fast, hexword
    for literal in ("1.44269502f", "12582912.0f", "-0.693145752f", "-1.42860677e-06f", "87.0f", "<< 23"):
        assert literal in fast, literal
    assert len(re.findall(r"__fmaf_rn", fast)) == 9          # one rounding step, two reduction steps, six Horner steps
