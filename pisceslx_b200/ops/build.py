"""In-tree build of the sm_100a extension: ``python -m pisceslx_b200.ops.build``.

Each ``.cu`` file is compiled with nvcc for ``sm_100a`` only (no torch headers: seconds per file), the
binding is compiled with g++ against the torch headers, and everything is linked into
``pisceslx_b200/ops/_yv_ops.so``, which ``torch.ops.load_library`` loads.  The build is incremental
(mtime based) and cross-compiles on machines without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
SO = HERE / "_yv_ops.so"

CUDA_SOURCES = ["gemm.cu", "elementwise.cu", "moe.cu", "loss_optim.cu", "attention.cu", "comm.cu", "noalloc.cu", "ssm.cu", "pq_film.cu"]
CPP_SOURCES = ["binding.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-diag-suppress", "550"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _host_cxx() -> str:
    """The distribution's g++.  The library must share the process's libstdc++ with torch: a compiler named by
    ``$CXX`` that links its own static copy gives two sets of locale facets in one process, and the first
    formatted error message (a ``TORCH_CHECK`` that prints a number) then crashes instead of raising.  ``YV_CXX``
    overrides; the link step names ``-lstdc++`` explicitly and the result is checked for that dependency."""
    forced = os.environ.get("YV_CXX")
    if forced:
        return forced
    import shutil
    for cand in ("/usr/bin/g++", shutil.which("g++")):
        if cand and os.path.exists(cand):
            return cand
    return "g++"


def _check_dynamic_libstdcxx(so: Path) -> None:
    r = subprocess.run(["readelf", "-d", str(so)], capture_output=True, text=True)
    if r.returncode == 0 and "libstdc++.so" not in r.stdout:
        raise RuntimeError(f"{so} does not depend on the shared libstdc++ (static C++ runtime linked in): "
                           "set YV_CXX to the system g++")


def _newer(src: Path, dst: Path, extra: List[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src] + extra if p.exists())


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")


def build(verbose: bool = False, force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.inc"))
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    jobs = []
    objs: List[Path] = []
    for name in CUDA_SOURCES:
        src = CSRC / name
        if not src.exists():
            continue
        obj = OBJ / (name + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append([nvcc, "-ccbin", _host_cxx()] + NVCC_FLAGS + ["-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    cxx = _host_cxx()
    for name in CPP_SOURCES:
        src = CSRC / name
        obj = OBJ / (name + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append([cxx, "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_yv_ops",
                         f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
                         "-I", str(CSRC), "-I", os.path.join(_cuda_home(), "include")] + inc +
                        ["-c", str(src), "-o", str(obj)])
    if verbose:
        for j in jobs:
            print(" ".join(j))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    if jobs or not SO.exists() or force:
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cmd = [cxx, "-shared", "-o", str(SO)] + [str(o) for o in objs] + [
            f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            f"-L{os.path.join(_cuda_home(), 'lib64')}", "-lcudart", "-lstdc++", f"-Wl,-rpath,{torch_lib}"]
        _run(cmd)
        _check_dynamic_libstdcxx(SO)
    return SO


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
