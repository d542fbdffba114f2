"""The compile-time variants of the fused decode kernel keep compiling for sm_100a (nvcc cross-compiles without a GPU).
The defaults are what the library is built with; the variants exist for tuning runs (BLOK_NVCC_EXTRA, blok_b200/build.py)."""
import os
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "blok_b200", "csrc")
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "-Xptxas", "-v", "-cubin"]


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not on PATH")
@pytest.mark.parametrize("defines,max_spill_bytes", [
    ([], 0),                                                    # the measured configuration: no spills
    (["-DBLOK_FUSED_C1_BLOCKS=2"], 0),
    (["-DBLOK_FUSED_C1_BLOCKS=4", "-DBLOK_I4_ACC_CHAINS=2"], 0),
    (["-DBLOK_FUSED_STAGE_UNITS=4", "-DBLOK_FUSED_COLLECT=8"], 400),   # these trade a few spilled registers per chunk
    (["-DBLOK_FUSED_I4_IMMA=1"], 0),                            # the integer consumer for the routed experts
])
def test_fused_kernel_variants_compile(tmp_path, defines, max_spill_bytes):
    out = str(tmp_path / "moe_fused.cubin")
    p = subprocess.run(["nvcc"] + FLAGS + defines + ["moe_fused.cu", "-o", out], cwd=CSRC, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert os.path.getsize(out) > 0
    # ptxas reports per function; the kernel's own line follows its "Function properties" line
    lines = p.stderr.splitlines()
    idx = [i for i, l in enumerate(lines) if "Function properties for" in l and "moe_decode_fused_kernel" in l]
    assert idx, p.stderr[-2000:]
    spill = lines[idx[0] + 1]
    stores = int(spill.split("bytes spill stores")[0].split(",")[-1])
    assert stores <= max_spill_bytes, spill
    regs = [l for l in lines[idx[0]:idx[0] + 4] if "registers" in l][0]
    assert int(regs.split("Used")[1].split("registers")[0]) <= 128, regs   # 512 threads per CTA: more cannot launch


def test_bad_variant_is_refused_at_compile_time(tmp_path):
    if shutil.which("nvcc") is None:
        pytest.skip("nvcc not on PATH")
    p = subprocess.run(["nvcc"] + FLAGS + ["-DBLOK_FUSED_C1_BLOCKS=3", "moe_fused.cu", "-o", str(tmp_path / "x.cubin")], cwd=CSRC,
                       capture_output=True, text=True, timeout=600)
    assert p.returncode != 0 and "BLOK_FUSED_C1_BLOCKS must be 1, 2 or 4" in p.stderr
