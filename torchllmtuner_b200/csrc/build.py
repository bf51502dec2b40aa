"""In-tree build of the sm_100a kernel library and its Python bindings.

`build()` compiles every `.cu` with `nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`, the bindings with
g++ against the installed torch headers, and links `torchllmtuner_b200/_C.so`. Objects are cached under
`csrc/build/` keyed by a hash of the source (and shared headers), so a rebuild only recompiles what changed.
The built `.so` carries the combined source hash in `_C.stamp`; `is_stale()` compares it with the tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
BUILD = os.path.join(HERE, "build")
SO_PATH = os.path.join(PKG, "_C.so")
STAMP = os.path.join(PKG, "_C.stamp")
CU_SOURCES = ("gemm.cu", "elementwise.cu", "attention.cu", "attention_fwd_pair.cu", "attention_bwd.cu", "moe.cu", "comm.cu", "ep_comm.cu", "vocab_parallel.cu", "noalloc.cu")
HEADERS = ("common.cuh", "comm.cuh", "attn_common.cuh", "kernels.h", "noalloc.h")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--use_fast_math", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _hash(paths) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _sources():
    return [s for s in CU_SOURCES if os.path.exists(os.path.join(HERE, s))]


def tree_hash() -> str:
    files = [os.path.join(HERE, s) for s in _sources()] + [os.path.join(HERE, h) for h in HEADERS] + [os.path.join(HERE, "bindings.cpp")]
    return _hash(files)


def is_stale() -> bool:
    if not (os.path.exists(SO_PATH) and os.path.exists(STAMP)):
        return True
    with open(STAMP) as f:
        return f.read().strip() != tree_hash()


def _run(cmd, log):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout[-4000:])
    return r.stdout


def build(verbose: bool = False, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(BUILD, exist_ok=True)
    if not force and not is_stale():
        return SO_PATH
    hdr = [os.path.join(HERE, h) for h in HEADERS]
    log: list[str] = []
    objs = []

    # LLMT_DEBUG=1 in the environment builds every kernel with -DLLMT_DEBUG: device-side argument and bounds checks
    # that report through the status word (the release build keeps only the checks that guard peer memory).
    debug = os.environ.get("LLMT_DEBUG") == "1"
    extra = ["-DLLMT_DEBUG"] if debug else []
    # LLMT_NVCC_FLAGS: extra nvcc flags (e.g. "-DNAME" for an experiment); they are part of the object cache key.
    user_flags = os.environ.get("LLMT_NVCC_FLAGS", "").split()
    extra += user_flags
    tag = ("." + hashlib.sha256(" ".join(user_flags).encode()).hexdigest()[:8]) if user_flags else ""

    def compile_cu(src):
        path = os.path.join(HERE, src)
        obj = os.path.join(BUILD, f"{os.path.splitext(src)[0]}.{_hash([path] + hdr)}{'.dbg' if debug else ''}{tag}.o")
        if not os.path.exists(obj):
            _run([_nvcc(), *NVCC_FLAGS, *extra, "-I", HERE, "-c", path, "-o", obj], log)
        return obj

    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as ex:
        objs = list(ex.map(compile_cu, _sources()))

    bsrc = os.path.join(HERE, "bindings.cpp")
    bobj = os.path.join(BUILD, f"bindings.{_hash([bsrc] + hdr)}.{torch.__version__.replace('+', '_')}.o")
    if not os.path.exists(bobj):
        incs = []
        for p in ce.include_paths("cuda"):
            incs += ["-isystem", p]
        incs += ["-isystem", sysconfig.get_paths()["include"]]
        abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-I", HERE, *incs, "-c", bsrc, "-o", bobj], log)
    libs = []
    for p in ce.library_paths("cuda"):
        libs += ["-L", p, f"-Wl,-rpath,{p}"]
    tmp = SO_PATH + ".tmp"
    _run(["g++", "-shared", "-o", tmp, bobj, *objs, *libs, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
          "-ltorch_python", "-lcudart"], log)
    os.replace(tmp, SO_PATH)
    with open(STAMP, "w") as f:
        f.write(tree_hash())
    with open(os.path.join(BUILD, "build.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    return SO_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
