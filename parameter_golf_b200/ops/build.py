"""In-tree build of the native extension ``parameter_golf_b200/_C*.so`` for sm_100a.

Every ``csrc/*.cu`` is compiled by nvcc (``-gencode arch=compute_100a,code=sm_100a -lineinfo``; no torch
headers, a few seconds each, in parallel), ``csrc/bindings.cpp`` by g++ against the torch headers, and the
objects are linked into one shared object next to the package so it travels with the source tree.
A content hash of the sources is stored beside the library; `ensure_built` rebuilds only on change.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")
BUILD = os.path.join(PKG, "csrc", "build")
LIB = os.path.join(PKG, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))
STAMP = os.path.join(PKG, "_C.hash")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    hdr = sorted(f for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inc")))
    return cu, cpp, hdr


def source_hash() -> str:
    h = hashlib.sha256()
    for group in _sources():
        for f in group:
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def is_current() -> bool:
    return os.path.exists(LIB) and os.path.exists(STAMP) and open(STAMP).read().strip() == source_hash()


def _run(cmd, log):
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{r.stdout[-4000:]}\n{r.stderr[-4000:]}")


def build(force: bool = False, verbose: bool = True) -> str:
    if not force and is_current():
        return LIB
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(BUILD, exist_ok=True)
    cu, cpp, _ = _sources()
    extra = os.environ.get("PGB_EXTRA_NVCC_FLAGS", "").split()     # development aid, e.g. -DPGB_WAIT_LIMIT_NS=50000000ull
    cuda_home = ce.CUDA_HOME or "/usr/local/cuda"
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    objs = []
    jobs = []
    for f in cu:
        o = os.path.join(BUILD, f + ".o")
        objs.append(o)
        jobs.append(([nvcc, *NVCC_FLAGS, *extra, f"-I{CSRC}", "-c", os.path.join(CSRC, f), "-o", o], os.path.join(BUILD, f + ".log")))
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for f in cpp:
        o = os.path.join(BUILD, f + ".o")
        objs.append(o)
        jobs.append((["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                      f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, "-c", os.path.join(CSRC, f), "-o", o], os.path.join(BUILD, f + ".log")))
    if verbose:
        print(f"[build] compiling {len(jobs)} translation units for sm_100a", file=sys.stderr)
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        list(ex.map(lambda j: _run(*j), jobs))
    libdirs = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", LIB, *objs, *[f"-L{d}" for d in libdirs], *[f"-Wl,-rpath,{d}" for d in libdirs],
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    _run(link, os.path.join(BUILD, "link.log"))
    with open(STAMP, "w") as f:
        f.write(source_hash())
    return LIB


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the saved nvcc logs."""
    out = []
    for f in sorted(os.listdir(BUILD)) if os.path.isdir(BUILD) else []:
        if f.endswith(".cu.log"):
            lines = open(os.path.join(BUILD, f)).read().splitlines()
            for i, l in enumerate(lines):
                if "Compiling entry function" in l:
                    name = l.split("'")[1]
                    info = " ".join(x.strip() for x in lines[i + 1:i + 4] if "ptxas info" in x)
                    out.append(f"{f[:-7]}: {name}: {info}")
    return "\n".join(out)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
