"""Register budgets that a decode step depends on.  Kernels launched with programmatic dependent launch share the SMs
with their neighbours in the stream; two of them were measured to fall off a cliff when they grow by a few registers
(the step, not the kernel alone, gets 14 % slower), so the compiler's report is checked here."""
import os
import re
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "mini_inference_b200", "csrc")


def registers(source):
    """{mangled kernel name: registers per thread} from ptxas for one source file."""
    from mini_inference_b200.ops.build import NVCC_FLAGS
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    r = subprocess.run([nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-c", os.path.join(CSRC, source), "-o", os.devnull],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    out, name = {}, None
    for line in r.stderr.splitlines():
        m = re.search(r"Compiling entry function '(\S+)'", line)
        if m:
            name = m.group(1)
        m = re.search(r"Used (\d+) registers", line)
        if m and name:
            out[name] = int(m.group(1))
            name = None
    return out


def test_stream_gemm_register_budget():
    regs = registers("gemm_stream.cu")
    eight_tokens = {k: v for k, v in regs.items() if "gemm_stream_kernelILi1E" in k}
    assert len(eight_tokens) == 2, sorted(regs)
    assert all(v <= 112 for v in eight_tokens.values()), eight_tokens


def test_deferred_norm_register_budget():
    regs = registers("deferred_sum.cu")
    norm = {k: v for k, v in regs.items() if "deferred_add_rmsnorm_kernel" in k}
    assert len(norm) == 2, sorted(regs)
    assert all(v <= 32 for v in norm.values()), norm
