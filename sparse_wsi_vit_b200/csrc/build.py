"""Builds libswv_b200.so (sm_100a only) in-tree with nvcc.

    python sparse_wsi_vit_b200/csrc/build.py [--force] [--verbose] [--checks]

--checks builds libswv_b200_checked.so with -DSWV_CHECKS (indices read from caller-supplied lists
are range-checked on the device and reported through the status word); run the tests against it
with SWV_B200_LIB=<that file>.

(run it by path: importing it through the package would first try to load the library)

nvcc cross-compiles without a GPU; the library links only the CUDA runtime and
loads on a machine without a driver (the TMA descriptor encoder is resolved at
call time).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libswv_b200.so")
SOURCES = ["indexer.cu", "dsa_attn.cu", "dsa_gather.cu", "block_sparse.cu", "nsa.cu", "capi.cu"]
HEADERS = ["ptx.cuh", "common.cuh", os.path.join("..", "..", "include", "swv_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Wno-deprecated-gpu-targets",
]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(HERE, f)) > t for f in SOURCES + HEADERS + ["build.py"])


def build(force: bool = False, verbose: bool = False, checks: bool = False) -> str:
    lib = LIB.replace(".so", "_checked.so") if checks else LIB
    if not checks and not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(HERE, src.replace(".cu", "_checked.o" if checks else ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *(["-DSWV_CHECKS"] if checks else []), "-c", os.path.join(HERE, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out)
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    subprocess.check_call([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", lib, *objs])
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, checks="--checks" in sys.argv))
