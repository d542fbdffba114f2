"""The streaming kernels keep compiling for sm_100a within their register and spill limits (nvcc cross-compiles
without a GPU).  Fused decode kernel: 512 threads per CTA leave 128 registers per thread, and the two streaming loops,
where the kernel spends its time, must not spill at all.  Small-group kernel, weight-streaming bf16 kernel and the
tcgen05 grouped GEMM: the registers their CTAs per SM allow, and next to nothing on the stack."""
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


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not on PATH")
@pytest.mark.parametrize("source,kernel,max_regs,max_spill", [
    # 512 threads per CTA: 128 registers at most; the token-count instances of the streaming loop are inlined into
    # the kernel, a few words of its task bookkeeping may live on the stack
    ("wgemv_small.cu", "wgemv_small_kernel", 128, 64),
    # 256 threads and two CTAs per SM at 32 tokens: 128 registers at most, and the eight accumulator tiles of the
    # 64-token instance must stay in registers
    ("wgemm_stream.cu", "wgemm_stream_kernel", 128, 16),
    # 288 threads, two CTAs per SM (tensor memory and shared memory are sized for two): 113 registers at most
    ("wgemm_tc.cu", "wgemm_tc_kernel", 112, 16),
])
def test_streaming_kernels_registers_and_spills(tmp_path, source, kernel, max_regs, max_spill):
    out = str(tmp_path / (source + ".cubin"))
    p = subprocess.run(["nvcc"] + FLAGS + [source, "-o", out], cwd=CSRC, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = p.stderr.splitlines()
    idx = [i for i, l in enumerate(lines) if "Function properties for" in l and kernel in l]
    assert idx, p.stderr[-2000:]
    for i in idx:  # every instance of the template
        stores = int(lines[i + 1].split("bytes spill stores")[0].split(",")[-1])
        regs = [l for l in lines[i:i + 4] if "registers" in l][0]
        assert stores <= max_spill, lines[i:i + 4]
        assert int(regs.split("Used")[1].split("registers")[0]) <= max_regs, regs
