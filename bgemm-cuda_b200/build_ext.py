"""Build libbgemm_b200.so (nvcc, sm_100a) and the `lowbit_kernel` torch extension (g++) in this directory.

Run as `python build_ext.py`; both outputs land beside this file so that `import lowbit_kernel` and
`import bgemm_b200` work once this directory is on sys.path. No JIT cache is involved.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def build_library(verbose: bool = False) -> Path:
    # the library and the native command line (bgemm_cli) that links against it
    subprocess.run(["make", "-C", str(HERE), "-j4", "libbgemm_b200.so", "bgemm_cli"], check=True,
                   stdout=None if verbose else subprocess.DEVNULL)
    return HERE / "libbgemm_b200.so"


def build_extension(verbose: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = HERE / f"lowbit_kernel{suffix}"
    src = HERE / "csrc" / "torch_ext.cpp"
    deps = [src, HERE.parent / "include" / "bgemm_b200.h"]
    if _newer(target, deps):
        return target
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{cuda_home}/include", f"-I{sysconfig.get_paths()['include']}"]
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=lowbit_kernel",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, str(src), "-o", str(target),
           f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python",
           f"-L{HERE}", "-lbgemm_b200", f"-L{cuda_home}/lib64", "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return target


def build_all(verbose: bool = False) -> None:
    build_library(verbose)
    build_extension(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built", HERE / "libbgemm_b200.so", "and lowbit_kernel")
