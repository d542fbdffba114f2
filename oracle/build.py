"""Build recipe for the checker libraries (test infrastructure).

  oracle/libblok_oracle.so   the CPU restatement (oracle/blok_oracle.cpp), g++ + OpenMP.
  oracle/_ref/libblok_ref.so the reference executor's own translation unit, compiled from
                             where it lies (never copied) together with oracle/ref_shim/,
                             for sm_100a.  Only built when the reference checkout is
                             present; the prebuilt file travels to the GPU box.

Run: python oracle/build.py [--reference /path/to/reference]
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _stale(out, srcs):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def build_oracle(force=False):
    src = os.path.join(HERE, "blok_oracle.cpp")
    out = os.path.join(HERE, "libblok_oracle.so")
    if force or _stale(out, [src]):
        cmd = ["g++", "-O2", "-std=c++17", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-march=x86-64-v2",
               src, "-o", out]
        subprocess.check_call(cmd)
    return out


def build_ref(reference, force=False):
    ref_src = os.path.join(reference, "src", "kimi_exec.cu")
    if not os.path.exists(ref_src):
        return None
    shim = os.path.join(HERE, "ref_shim", "ref_shim.cu")
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "libblok_ref.so")
    if force or _stale(out, [shim, ref_src, os.path.join(HERE, "ref_shim", "ugds.h")]):
        cmd = ["nvcc", "-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler",
               "-fPIC", "-I", os.path.join(HERE, "ref_shim"), "-I", os.path.join(reference, "src"),
               "-DCUDART_INF_F=(__builtin_huge_valf())", "-DCUDART_PI_F=3.141592654f", shim, "-o", out]
        subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("BLOK_REFERENCE") or
                    os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"),
                    help="the reference checkout (default: BLOK_REFERENCE, else a `reference` folder beside this repository)")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    r = build_ref(a.reference, a.force)
    print(r if r else "reference checkout absent: oracle/_ref not built", file=sys.stderr if not r else sys.stdout)
