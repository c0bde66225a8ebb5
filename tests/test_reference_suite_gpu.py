"""The reference's OWN tests/test_matmul.cpp, compiled unmodified against the C++ shim
(laplace_b200/csrc/shim) so that every quantized matmul in it runs through the CUDA library
behind the reference's back-end interface. The binary is built where the reference checkout
is present (`make -C oracle ref_cuda`) and travels with oracle/_ref."""
import os
import re
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
EXE = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "test_matmul_cuda"


@pytest.mark.skipif(not EXE.exists(), reason="oracle/_ref/test_matmul_cuda not built (needs the reference checkout)")
def test_reference_test_matmul_passes_on_the_cuda_backend():
    env = dict(os.environ, LAPLACE_CUDA_VERBOSE="1")
    env.pop("LAPLACE_NOSIMD", None)
    r = subprocess.run([str(EXE)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "test_matmul: OK (1048 checks)" in r.stdout
    assert "failed" not in r.stderr
    m = re.search(r"(\d+) matmul calls ran on the GPU", r.stderr)
    # 4 int8-path types x 4 N at K=512, Q4_K/Q6_K x 4 N at K=2816, plus the batched-rows test
    assert m and int(m.group(1)) >= 24, r.stderr
