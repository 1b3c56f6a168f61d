"""Compiles the CUDA sources under nnforge_b200/csrc into nnforge_b200/libnnf_b200.so (sm_100a only).

    python -m nnforge_b200.build

-fmad=false for every file whose kernels are held to nnForge's plain (CPU) backend bit for bit: there products
and sums must be rounded separately. The single-launch training batch norm (nnf_bn_chain.cu) is a tolerance
row - the reference's arithmetic there is cuDNN's - and is built with contraction: its launches are bound by
how instruction issue and memory overlap, and every fused multiply-add is an instruction less.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libnnf_b200.so")
HOST_LIB = os.path.join(HERE, "libnnf_b200_host.so")
HOST_SRC = os.path.join(CSRC, "host", "nnf_layers.cpp")
HOST_SOURCES = [HOST_SRC, os.path.join(CSRC, "host", "nnf_fusion.cpp"), os.path.join(CSRC, "host", "nnf_fused_layers.cpp")]
SOURCES = ["nnf_api.cu", "nnf_elementwise.cu", "nnf_softmax.cu", "nnf_loss.cu", "nnf_maxpool.cu", "nnf_avgpool.cu", "nnf_optimizer.cu", "nnf_bn_train.cu", "nnf_bn_chain.cu", "nnf_peer.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
CONTRACTING = {"nnf_bn_chain.cu"}   # sources built with FMA contraction; all others get -fmad=false


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _deps_mtime():
    newest = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for name in os.listdir(root):
            if name.endswith((".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def _compile(job):
    src, obj, hdr_mtime, verbose = job
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_mtime):
        return
    fmad = [] if os.path.basename(src) in CONTRACTING else ["-fmad=false"]
    cmd = [_nvcc()] + NVCC_FLAGS + fmad + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    subprocess.check_call(cmd)


def build(verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr = _deps_mtime()
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    jobs = [(os.path.join(CSRC, s), os.path.join(OBJ, s[:-3] + ".o"), hdr, verbose) for s in sources]
    with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
        list(pool.map(_compile, jobs))
    objs = [j[1] for j in jobs]
    if not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        subprocess.check_call([_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    build_host()
    build_ceilings()
    return LIB


CEILINGS = os.path.join(HERE, "nnf_ceilings")


def build_ceilings():
    """The stand-alone program that measures the device's memory ceilings for this path's access patterns (bench.py --ceilings)."""
    src = os.path.join(CSRC, "probe", "nnf_ceilings.cu")
    if os.path.exists(CEILINGS) and os.path.getmtime(CEILINGS) >= os.path.getmtime(src):
        return CEILINGS
    subprocess.check_call([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", src, "-o", CEILINGS])
    return CEILINGS


def build_host():
    """C++ host-side layer objects (nnForge-shaped testers / updaters over the C ABI)."""
    deps = HOST_SOURCES + [os.path.join(CSRC, "host", "nnf_layers.h"), os.path.join(CSRC, "host", "nnf_fusion.h"),
            os.path.join(CSRC, "host", "nnf_layers_detail.h"), os.path.join(os.path.dirname(HERE), "include", "nnf_b200.h"), LIB]
    if os.path.exists(HOST_LIB) and os.path.getmtime(HOST_LIB) >= max(os.path.getmtime(d) for d in deps):
        return HOST_LIB
    cuda_home = os.path.dirname(os.path.dirname(_nvcc())) if os.path.sep in _nvcc() else "/usr/local/cuda"
    # the CUDA runtime is linked statically (weights upload, mailbox allocation): no libcudart.so is needed at run time
    subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-I", os.path.join(cuda_home, "include")] + HOST_SOURCES
                          + ["-o", HOST_LIB, "-L", HERE, "-lnnf_b200", "-Wl,-rpath,$ORIGIN",
                             "-L", os.path.join(cuda_home, "lib64"), "-lcudart_static", "-ldl", "-lrt", "-lpthread", "-Wl,--exclude-libs,ALL"])
    return HOST_LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
