"""Build the native extension in-tree: ``python -m odc_b200.build``.

Kernel files are compiled with nvcc for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``);
host files with g++; everything is linked into ``odc_b200/_C.so`` with a static CUDA runtime.
No GPU is needed to build.  Objects are cached under ``odc_b200/csrc/build`` by source hash.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CUDA_SOURCES = ["kernels/comm.cu", "kernels/elementwise.cu", "kernels/gemm_tcgen05.cu", "kernels/gemm_tcgen05_2cta.cu", "kernels/attention_tcgen05.cu",
                "kernels/fused_comm_gemm.cu", "kernels/no_alloc.cu", "kernels/device_prims.cu"]
CPP_SOURCES = ["heap/symm_heap.cpp", "kernels/tensor_map.cpp"]
BINDING_SOURCES = ["bindings/bindings.cpp"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce
    inc = ce.include_paths("cuda") if hasattr(ce, "include_paths") else []
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, lib, abi


def _digest(path: str, extra: str) -> str:
    h = hashlib.sha1(extra.encode())
    with open(path, "rb") as f:
        h.update(f.read())
    # headers next to the source take part in the hash
    d = os.path.dirname(path)
    for name in sorted(os.listdir(d)):
        if name.endswith((".h", ".cuh")):
            with open(os.path.join(d, name), "rb") as f:
                h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd, log):
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    inc, torch_lib, abi = _torch_paths()
    py_inc = sysconfig.get_paths()["include"]
    cuda_inc = os.path.join(CUDA_HOME, "include")
    jobs = []
    for rel in CUDA_SOURCES:
        src = os.path.join(CSRC, rel)
        if not os.path.exists(src):
            continue
        cmd_tail = NVCC_FLAGS + [f"-I{os.path.dirname(src)}"]
        tag = _digest(src, " ".join(cmd_tail))
        obj = os.path.join(OBJ, os.path.basename(rel) + "." + tag + ".o")
        jobs.append((obj, [NVCC] + cmd_tail + ["-c", src, "-o", obj]))
    cxx_common = ["-O2", "-std=c++17", "-fPIC", f"-I{cuda_inc}", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    for rel in CPP_SOURCES:
        src = os.path.join(CSRC, rel)
        tag = _digest(src, " ".join(cxx_common))
        obj = os.path.join(OBJ, os.path.basename(rel) + "." + tag + ".o")
        jobs.append((obj, ["g++"] + cxx_common + ["-c", src, "-o", obj]))
    for rel in BINDING_SOURCES:
        src = os.path.join(CSRC, rel)
        flags = cxx_common + [f"-I{p}" for p in inc] + [f"-I{py_inc}", "-DTORCH_EXTENSION_NAME=_C",
                                                      "-DTORCH_API_INCLUDE_EXTENSION_H"]
        hdrs = "".join(open(os.path.join(CSRC, h)).read() for h in ("kernels/api.h", "heap/symm_heap.h"))
        tag = _digest(src, " ".join(flags) + hashlib.sha1(hdrs.encode()).hexdigest())
        obj = os.path.join(OBJ, os.path.basename(rel) + "." + tag + ".o")
        jobs.append((obj, ["g++"] + flags + ["-c", src, "-o", obj]))

    def compile_one(job):
        obj, cmd = job
        if force or not os.path.exists(obj):
            out = _run(cmd, obj + ".log")
            if verbose:
                print(out)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        objs = list(ex.map(compile_one, jobs))
    so = os.path.join(HERE, "_C.so")
    link = ["g++", "-shared", "-o", so] + objs + [
        f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-ltorch_python", "-lc10", "-lc10_cuda",
        f"-L{os.path.join(CUDA_HOME, 'lib64')}", "-lcudart_static", "-lrt", "-ldl", "-lpthread",
        f"-Wl,-rpath,{torch_lib}"]
    _run(link, os.path.join(OBJ, "link.log"))
    # drop objects of older source revisions
    keep = set(objs)
    for name in os.listdir(OBJ):
        p = os.path.join(OBJ, name)
        if name.endswith(".o") and p not in keep:
            os.remove(p)
            if os.path.exists(p + ".log"):
                os.remove(p + ".log")
    return so


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last build (registers, spills, shared memory)."""
    out = []
    for name in sorted(os.listdir(OBJ)):
        if name.endswith(".o.log") and ".cu." in name:
            out.append(open(os.path.join(OBJ, name)).read())
    return "\n".join(out)


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built", path)
