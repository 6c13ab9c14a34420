"""Builds libmoe_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python gpt-oss-amd_b200/build.py [--force] [--verbose]

The CUDA runtime is linked statically, so the library depends only on the
driver and on NCCL (libnccl.so.2, found through the embedded run path in the
Python environment's nvidia/nccl directory or on the system)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libmoe_b200.so")
SOURCES = ["moe_b200.cu"]


def _nccl_dirs():
    cands = []
    for base in {sysconfig.get_paths().get("purelib"), sysconfig.get_paths().get("platlib")}:
        if base:
            cands.append(os.path.join(base, "nvidia", "nccl"))
    for c in cands:
        if os.path.isfile(os.path.join(c, "include", "nccl.h")) and os.path.isfile(
                os.path.join(c, "lib", "libnccl.so.2")):
            return os.path.join(c, "include"), os.path.join(c, "lib")
    if os.path.isfile("/usr/include/nccl.h"):
        for lib in ("/usr/lib/x86_64-linux-gnu", "/usr/lib64", "/usr/local/lib"):
            if os.path.isfile(os.path.join(lib, "libnccl.so.2")):
                return "/usr/include", lib
    raise RuntimeError("NCCL headers / libnccl.so.2 not found")


def _stale() -> bool:
    if not os.path.isfile(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "moe_b200.h"))
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines: tuple = ()) -> str:
    if not force and not defines and not _stale():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise RuntimeError("nvcc not found; the library cannot be built on this machine")
    inc, lib = _nccl_dirs()
    cmd = [
        nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++",
        "-I", inc, "-L", lib, "-l:libnccl.so.2",
        "-Xlinker", f"-rpath={lib}",
        "-o", OUT,
    ]
    cmd += [f"-D{d}" for d in defines]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed")
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
          defines=tuple(a[2:] for a in sys.argv[1:] if a.startswith("-D")))
    print(OUT)
