"""Compile-time properties of the kernels that the GPU tests cannot see.  CPU only (nvcc cross-compiles)."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "voxcpm.cpp_b200", "csrc")


def _ptxas_report(source, tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    out = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
                          "-Xptxas", "-v", "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", os.path.join(CSRC, source),
                          "-o", str(tmp_path / "out.o")], capture_output=True, text=True, check=True)
    report = {}
    name = None
    for line in (out.stdout + out.stderr).splitlines():
        m = re.search(r"Compiling entry function '(\S+)'", line)
        if m:
            name = m.group(1)
        m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m and name:
            report[name] = tuple(int(x) for x in m.groups())
    return report


def test_prefill_kernels_do_not_spill(tmp_path):
    """The tcgen05 prefill kernel lets its warpgroups trade registers after launch (setmaxnreg) and sizes each role's share
    by hand.  A role that no longer fits spills silently; an experimental build in which the 40- and 56-register roles
    spilled produced wrong results without any fault.  Every instantiation must compile without spills."""
    report = _ptxas_report("prefill_attn.cu", tmp_path)
    kernels = {k: v for k, v in report.items() if "prefill_tc_kernel" in k}
    assert len(kernels) == 5, sorted(report)
    for name, (stack, stores, loads) in kernels.items():
        assert (stack, stores, loads) == (0, 0, 0), f"{name}: {stack} bytes of stack, {stores} spilled"


def test_decode_kernels_do_not_spill(tmp_path):
    """The decode kernels run three (f16) and four (q8_0) CTAs per SM on fixed register budgets; spills would put
    local-memory traffic into a kernel that is bound by memory bandwidth."""
    report = _ptxas_report("decode_attn.cu", tmp_path)
    kernels = {k: v for k, v in report.items() if "decode_kernel" in k}
    assert len(kernels) >= 2, sorted(report)
    for name, (stack, stores, loads) in kernels.items():
        assert stores == 0 and loads == 0, f"{name}: {stores} bytes spilled"
