"""The fused decode kernel keeps compiling for sm_100a within its register and spill limits (nvcc cross-compiles
without a GPU): 512 threads per CTA leave 128 registers per thread, and the two streaming loops, where the kernel
spends its time, must not spill at all."""
import os
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "blok_b200", "csrc")
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "-Xptxas", "-v", "-cubin"]


def _properties(stderr, name):
    """(spill store bytes, spill load bytes) ptxas reports for the first function whose mangled name holds `name`."""
    lines = stderr.splitlines()
    idx = [i for i, l in enumerate(lines) if "Function properties for" in l and name in l]
    assert idx, stderr[-2000:]
    spill = lines[idx[0] + 1]
    stores = int(spill.split("bytes spill stores")[0].split(",")[-1])
    loads = int(spill.split("bytes spill loads")[0].split(",")[-1])
    return stores, loads, lines[idx[0]:idx[0] + 4]


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not on PATH")
def test_fused_kernel_registers_and_spills(tmp_path):
    out = str(tmp_path / "moe_fused.cubin")
    p = subprocess.run(["nvcc"] + FLAGS + ["moe_fused.cu", "-o", out], cwd=CSRC, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert os.path.getsize(out) > 0
    for loop in ("consume_i4", "consume_bf16", "collect_row_block", "routing_from_scores"):
        stores, loads, _ = _properties(p.stderr, loop)
        assert stores == 0 and loads == 0, (loop, stores, loads)
    # the kernel body (the chunk dispatcher around those loops) may keep a few words on the stack
    stores, _, around = _properties(p.stderr, "moe_decode_fused_kernel")
    assert stores <= 128, around
    regs = [l for l in around if "registers" in l][0]
    assert int(regs.split("Used")[1].split("registers")[0]) <= 128, regs   # 512 threads per CTA: more cannot launch
