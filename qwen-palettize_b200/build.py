"""Build libplz.so (the C-ABI library of the PalettizedLinear hot path) in place with nvcc for sm_100a.

Usage: python build.py [--force] [--verbose]
The library lands next to this file so that it travels with the source tree.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["api.cu", "lut_gemm.cu", "lut_gemm_pair.cu", "tn_gemm.cu", "elementwise.cu", "gemv.cu", "smallm_mma.cu", "train_ops.cu", "soft_tensors.cu", "attention.cu", "attention_decode.cu", "layer_ops.cu"]
HEADERS = ["plz_sm100.cuh", "plz_host.h", "plz_launch.h", "soft_math.cuh", os.path.join("..", "..", "include", "plz.h")]
LIB = os.path.join(HERE, "libplz.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v"]
if os.environ.get("PLZ_DIAGNOSTICS") == "1":   # cycle counters inside the kernels + the plz_debug_* entry points
    FLAGS.append("-DPLZ_DIAGNOSTICS")


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every .cu into an object (in parallel) and link the shared library."""
    if not force and not _stale():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for s in SOURCES:
        src = os.path.join(CSRC, s)
        if not os.path.exists(src):
            continue
        obj = os.path.join(objdir, s.replace(".cu", ".o"))
        cmd = [NVCC] + FLAGS + ["-c", src, "-o", obj]
        procs.append((s, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    log = []
    for s, obj, p in procs:
        out, _ = p.communicate()
        log.append(out)
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"nvcc failed on {s}")
        objs.append(obj)
    with open(os.path.join(objdir, "ptxas.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-lcudart"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    return LIB


def spill_report():
    """{kernel name: (spill store bytes, spill load bytes, registers)} parsed from the ptxas log of the last build."""
    import re
    path = os.path.join(HERE, "build", "ptxas.log")
    out, name = {}, None
    if not os.path.exists(path):
        return out
    for line in open(path):
        m = re.search(r"Compiling entry function '([^']+)'", line)
        if m:
            name = m.group(1)
        m = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m and name:
            out[name] = [int(m.group(1)), int(m.group(2)), None]
        m = re.search(r"Used (\d+) registers", line)
        if m and name and name in out:
            out[name][2] = int(m.group(1))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
