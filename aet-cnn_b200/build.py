"""Builds libaet_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python aet-cnn_b200/build.py`` or through ``__graft_entry__.build()``.  nvcc
cross-compiles without a GPU.  The library links the CUDA runtime statically and resolves the
driver's tensor-map encoder and NCCL at run time, so it loads on machines without a GPU
(every compute entry point then fails with AET_E_CUDA)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libaet_b200.so")
SOURCES = ["tensor.cu", "elementwise.cu", "conv.cu", "layers.cu", "network.cu"]
HEADERS = ["common.h", "umma.cuh", "activation.cuh", "conv_tma.cuh", "conv_tma_rows.cuh", "conv_thin.cuh", "stem.cuh", "conv_s2d.cuh", os.path.join("..", "..", "include", "aet_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xptxas", "-v"]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    hdrs = [os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + ["-c", s, "-o", o]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed on %s" % src)
            with open(o + ".ptxas.txt", "w") as f:
                f.write(r.stderr)
    if force or _stale(OUT, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT] + objs + ["-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
