"""In-tree build of the CUDA library (sm_100a only).

    python -m blok_b200.build            # builds blok_b200/libblok_b200.so if stale
    python -m blok_b200.build --force

nvcc cross-compiles without a GPU.  Objects go to blok_b200/build/, the shared
library next to this file so that it travels with the source tree.
"""
import argparse
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libblok_b200.so")
OBJ = os.path.join(HERE, "build")
CLI = os.path.join(HERE, "blok-kimi-exec")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


# Extra nvcc flags for a one-off build, e.g. BLOK_NVCC_EXTRA="-Xptxas -warn-spills" python -m blok_b200.build --force
EXTRA = os.environ.get("BLOK_NVCC_EXTRA", "").split()


def _deps():
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    hdrs.append(os.path.join(HERE, "..", "include", "blok_b200.h"))
    return hdrs


def _compile(src, verbose_ptxas):
    obj = os.path.join(OBJ, os.path.basename(src) + ".o")
    deps = [src] + _deps()
    if os.path.exists(obj) and all(os.path.getmtime(d) <= os.path.getmtime(obj) for d in deps):
        return obj, ""
    cmd = ["nvcc"] + NVCC_FLAGS + EXTRA + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-c", src, "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, p.stdout, p.stderr))
    return obj, p.stderr


def build(force=False, verbose_ptxas=False):
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    if force:
        for o in glob.glob(os.path.join(OBJ, "*.o")):
            os.remove(o)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose_ptxas), srcs))
    objs = [r[0] for r in results]
    log = "".join(r[1] for r in results)
    if force or not os.path.exists(OUT) or any(os.path.getmtime(o) > os.path.getmtime(OUT) for o in objs):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT] + objs + ["-lcudart", "-ldl"]
        subprocess.check_call(cmd)
    cli_src = os.path.join(HERE, "cli", "blok_kimi_exec.cpp")
    if os.path.exists(cli_src) and (force or not os.path.exists(CLI) or os.path.getmtime(cli_src) > os.path.getmtime(CLI)
                                    or os.path.getmtime(OUT) > os.path.getmtime(CLI)):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-I", os.path.join(HERE, "..", "include"), cli_src, "-o", CLI,
                               "-L", HERE, "-lblok_b200", "-Wl,-rpath,$ORIGIN"])
    return OUT, log


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args()
    out, log = build(a.force, a.ptxas)
    if a.ptxas:
        sys.stderr.write(log)
    print(out)
