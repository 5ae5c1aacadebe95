"""Compiles the reference's own C++/CUDA sources into oracle/_ref/libnpc_ref.so.

Test infrastructure only: the library built here is the UNMODIFIED reference
(kaihaoma/APT, src/*.cc, src/ops/collective.cc, src/cuda/*.cu), compiled from
where its sources lie (``APT_REFERENCE_DIR``, default ``/root/reference``) with
nvcc for sm_100 against the installed PyTorch headers. Nothing is copied into
this repository; the one file written besides objects is a two-line
``glog/logging.h`` stand-in that includes ``c10/util/Logging.h`` (c10's own glog
replacement), because glog is not installed. The reference's CMake build is not
run (it also wants MPI and googletest for its unit tests, which are absent).

    python oracle/build_ref.py [--force] [-j N]

The result is loaded with ``torch.classes.load_library`` by
``tests/golden/make_ref_golden.py`` on a machine with a GPU, which records the reference
operators' outputs as golden vectors under tests/golden/. Only tests/ and that
script use it; the product never does.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "libnpc_ref.so")
REF = os.environ.get("APT_REFERENCE_DIR", "/root/reference")

SOURCES = [
    "src/cache_feats.cc", "src/cache_graphs.cc", "src/core.cc", "src/feat_shuffle.cc", "src/load_subtensor.cc",
    "src/pybind.cc", "src/relabel.cc", "src/sampling.cc", "src/sddmm.cc", "src/spmm.cc", "src/ops/collective.cc",
    "src/cuda/npc_kernel.cu", "src/cuda/relabel.cu", "src/cuda/sddmm.cu", "src/cuda/spmm.cu",
]


def _paths():
    import sysconfig

    import torch

    tdir = os.path.dirname(torch.__file__)
    site = os.path.dirname(tdir)
    inc = [os.path.join(tdir, "include"), os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           os.path.join(site, "nvidia", "nccl", "include"), sysconfig.get_paths()["include"]]
    libdirs = [os.path.join(tdir, "lib"), os.path.join(site, "nvidia", "nccl", "lib")]
    return inc, libdirs, int(torch._C._GLIBCXX_USE_CXX11_ABI)


def available():
    return os.path.exists(LIB)


def build(force=False, jobs=None):
    if available() and not force:
        return LIB
    if not os.path.isdir(os.path.join(REF, "src")):
        raise RuntimeError(f"reference sources not found under {REF}")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    inc, libdirs, abi = _paths()
    shim = os.path.join(OUT, "shim", "glog")
    os.makedirs(shim, exist_ok=True)
    with open(os.path.join(shim, "logging.h"), "w") as f:
        f.write("// stand-in for glog: c10 provides LOG/CHECK with the same spelling\n#pragma once\n"
                "#include <c10/util/Logging.h>\n")
    obj_dir = os.path.join(OUT, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    flags = ["-gencode", "arch=compute_100,code=sm_100", "-O2", "-std=c++17", "-x", "cu", "-Xcompiler", "-fPIC",
             "-w", "--expt-relaxed-constexpr", "--expt-extended-lambda", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
             "-I", os.path.join(OUT, "shim"), "-I", os.path.join(REF, "src")]
    for d in inc:
        flags += ["-I", d]

    # src/cuda/npc_kernel.cu calls thrust::sequence and relied on older thrust headers pulling its
    # declaration in; CUDA 12.9's do not, so that header is force-included (the source stays as it is)
    extra = {"src/cuda/npc_kernel.cu": ["-include", "thrust/sequence.h"]}

    def one(src):
        obj = os.path.join(obj_dir, src.replace("/", "_").rsplit(".", 1)[0] + ".o")
        if os.path.exists(obj) and not force:
            return obj, 0, ""
        p = subprocess.run([nvcc, *flags, *extra.get(src, []), "-c", os.path.join(REF, src), "-o", obj],
                           stdout=subprocess.PIPE,
                           stderr=subprocess.STDOUT, text=True)
        return obj, p.returncode, p.stdout

    jobs = jobs or max(1, min(8, (os.cpu_count() or 2)))
    with ThreadPoolExecutor(jobs) as ex:
        results = list(ex.map(one, SOURCES))
    bad = [(o, out) for o, rc, out in results if rc != 0]
    if bad:
        for o, out in bad:
            sys.stderr.write(f"--- failed: {o}\n{out[-4000:]}\n")
        raise RuntimeError("the reference did not compile; see the messages above")
    link = [nvcc, "-shared", "-o", LIB, *[o for o, _, _ in results]]
    for d in libdirs:
        link += ["-L", d, "-Xlinker", f"-rpath={d}"]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-l:libnccl.so.2", "-lcudart"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    j = None
    if "-j" in sys.argv:
        j = int(sys.argv[sys.argv.index("-j") + 1])
    print(build(force="--force" in sys.argv, jobs=j))
