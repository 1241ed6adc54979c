"""Builds libswv_b200.so (sm_100a only) in-tree with nvcc.

    python sparse_wsi_vit_b200/csrc/build.py [--force] [--verbose] [--checks] [--profile]

--checks builds libswv_b200_checked.so with -DSWV_CHECKS (indices read from caller-supplied lists
are range-checked on the device and reported through the status word); run the tests against it
with SWV_B200_LIB=<that file>.  --profile builds libswv_b200_prof.so with -DSWV_PROFILE (phase
timers inside dsa_attn_masked_kernel, read with swv_debug_attn_profile).

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
SOURCES = ["indexer.cu", "dsa_attn.cu", "dsa_attn_lists.cu", "dsa_gather.cu", "dsa_bwd.cu", "block_sparse.cu", "nsa.cu", "capi.cu"]
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


def build(force: bool = False, verbose: bool = False, checks: bool = False, defines=(), suffix: str = "") -> str:
    """`checks`: the range-checked library; `defines` + `suffix`: any other variant, e.g. the phase-timer
    build `build(defines=["SWV_PROFILE"], suffix="_prof")` -> libswv_b200_prof.so."""
    if checks:
        defines, suffix = [*defines, "SWV_CHECKS"], suffix + "_checked"
    lib = LIB.replace(".so", suffix + ".so")
    if not suffix and not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(HERE, src.replace(".cu", suffix + ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", os.path.join(HERE, src), "-o", obj]
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
    if "--profile" in sys.argv:
        print(build(defines=["SWV_PROFILE"], suffix="_prof", verbose="--verbose" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, checks="--checks" in sys.argv))
