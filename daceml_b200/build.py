"""Builds ``libdaceml_b200.so`` (the CUDA kernels plus their C ABI) in-tree with nvcc for sm_100a.

Run as ``python -m daceml_b200.build``.  The library is rebuilt only when a source is newer than it.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdaceml_b200.so")

SOURCES = ["api.cu", "gemm_tc.cu", "gemm_tc2.cu", "gemm_ln.cu", "gemm_simt.cu", "gemm_tf32.cu", "rowwise.cu", "elementwise.cu", "indexing.cu", "conv.cu", "conv1x1_tc.cu", "conv_igemm.cu", "attention.cu", "diagnostics.cu", "peer.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcudafe", "--diag_suppress=177",
]


def find_nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _deps():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    files.append(os.path.join(HERE, "..", "include", "daceml_b200.h"))
    return files


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > built for f in _deps())


def build(force=False, verbose=False, ptxas_info=False):
    """Compiles every ``.cu`` under ``csrc/`` into one shared library.  Returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = find_nvcc()
    os.makedirs(LIB_DIR, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(LIB_DIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src} ---\n{out}\n")
        elif out.strip() and (verbose or ptxas_info):
            print(f"--- {src} ---\n{out}")
    if failed:
        raise RuntimeError("nvcc failed; see messages above")
    link = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart_static",
            "-ldl", "-lrt", "-lpthread"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.run(link, check=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
