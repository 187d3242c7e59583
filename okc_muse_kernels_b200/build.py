"""Builds csrc/*.cu into okc_muse_kernels_b200/libokc_moe_b200.so for sm_100a with nvcc.

    python -m okc_muse_kernels_b200.build            # build if sources are newer than the library
    python -m okc_muse_kernels_b200.build --force

nvcc cross-compiles without a GPU.  The library is built in-tree and loaded with ctypes; there is
no JIT and no fallback: if the library is missing, importing the operators fails.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libokc_moe_b200.so")
SOURCES = ("abi.cu", "route.cu", "repack.cu", "gemm.cu", "ep.cu", "router_mma.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(PKG, "..", "include", "okc_moe.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str) -> tuple[str, str]:
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    cmd = [nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False, wait_profile: bool = False, variant: str | None = None,
          defines: tuple[str, ...] = ()) -> str:
    """Compiles and links the library; returns its path.  ``wait_profile`` builds the instrumented
    variant libokc_moe_b200_prof.so (-DOKC_WAIT_PROFILE: per-role wait cycles, read back with
    okc_moe_debug_wait_profile); load it by pointing OKC_MOE_LIB at it.  ``variant`` + ``defines`` build
    libokc_moe_b200_<variant>.so with extra -D switches (tuning experiments: the kernels' compile-time
    knobs), to be compared against the default build through OKC_MOE_LIB."""
    global OBJ
    lib_path = LIB
    if variant:
        lib_path = LIB.replace(".so", f"_{variant}.so")
        OBJ = os.path.join(PKG, "build", variant)
        NVCC_FLAGS.extend(f"-D{d}" for d in defines)
    elif wait_profile:
        lib_path = LIB.replace(".so", "_prof.so")
        OBJ = os.path.join(PKG, "build", "prof")
        NVCC_FLAGS.append("-DOKC_WAIT_PROFILE")
    elif not force and not _stale():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(_compile, SOURCES))
    log = "\n".join(r[1] for r in results)
    with open(os.path.join(OBJ, "ptxas.log"), "w") as f:
        f.write(log)
    if verbose:
        print(log)
    cmd = [nvcc(), "-shared", "-o", lib_path, *[r[0] for r in results], "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    # python -m okc_muse_kernels_b200.build [--force] [-v] [--wait-profile] [--variant NAME -DKNOB=VALUE ...]
    name = sys.argv[sys.argv.index("--variant") + 1] if "--variant" in sys.argv else None
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, wait_profile="--wait-profile" in sys.argv,
                variant=name, defines=tuple(a[2:] for a in sys.argv if a.startswith("-D"))))
