"""Builds libmoe_b200.so (the C-ABI library) in-tree with nvcc for sm_100a, and
libmoe_b200_testaids.so, the same sources compiled with -DMOE_B200_TEST_AIDS (adds
the plain warp-MMA cross-check GEMM the parity tests compare the tcgen05 kernels
with; never shipped).

    python gpt-oss-amd_b200/build.py [--force] [--verbose] [--no-test-aids]

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
OUT_TEST_AIDS = os.path.join(HERE, "libmoe_b200_testaids.so")
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


def _stale(out: str) -> bool:
    if not os.path.isfile(out):
        return True
    t = os.path.getmtime(out)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "moe_b200.h"))
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(out: str, defines: tuple, verbose: bool) -> None:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise RuntimeError("nvcc not found; the library cannot be built on this machine")
    inc, lib = _nccl_dirs()
    cmd = [
        nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
        "-shared", "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++",
        "-I", inc, "-L", lib, "-l:libnccl.so.2",
        "-Xlinker", f"-rpath={lib}",
        "-o", out,
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


def build(force: bool = False, verbose: bool = False, defines: tuple = (), test_aids: bool = True) -> str:
    """Compiles the library (and, unless ``test_aids`` is False, the test-aids
    variant) when a source is newer than the built file.  Extra ``defines`` go
    to both."""
    jobs = [(OUT, tuple(defines))]
    if test_aids:
        jobs.append((OUT_TEST_AIDS, tuple(defines) + ("MOE_B200_TEST_AIDS",)))
    todo = [(o, d) for o, d in jobs if force or defines or _stale(o)]
    if len(todo) > 1:  # the two compilations are independent
        import concurrent.futures

        with concurrent.futures.ThreadPoolExecutor(len(todo)) as ex:
            for f in [ex.submit(_compile, o, d, verbose) for o, d in todo]:
                f.result()
    else:
        for o, d in todo:
            _compile(o, d, verbose)
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
          defines=tuple(a[2:] for a in sys.argv[1:] if a.startswith("-D")),
          test_aids="--no-test-aids" not in sys.argv)
    print(OUT)
