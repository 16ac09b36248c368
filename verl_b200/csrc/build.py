"""In-tree build of the sm_100a kernel library.

Kernel sources (``*.cu``) are compiled by nvcc for ``sm_100a`` only and do not include libtorch headers, so each
takes seconds; the thin ``torch.ops`` bindings (``*.cpp``) are compiled by the host compiler. Everything is linked
into ``verl_b200/_C.so`` next to the package so that the built library travels with the source tree.

Usage: ``python -m verl_b200.csrc.build [--force] [--verbose]``
"""

from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
OBJ_DIR = PKG / "_build"
LIB_PATH = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else "nvcc"


def _torch_paths():
    import torch
    from torch.utils import cpp_extension

    inc = cpp_extension.include_paths("cuda") if hasattr(cpp_extension, "include_paths") else []
    try:
        inc = cpp_extension.include_paths(device_type="cuda")
    except TypeError:
        pass
    lib = [str(Path(torch.__file__).parent / "lib")]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = list(inc) + [str(Path(cuda_home) / "include")]
    lib.append(str(Path(cuda_home) / "lib64"))
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, lib, abi


def _needs_build(src: Path, obj: Path, deps: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *deps])


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    cu_files = sorted(CSRC.glob("*.cu"))
    cpp_files = sorted(CSRC.glob("*.cpp"))
    inc, libdirs, abi = _torch_paths()
    jobs = []
    objs = []
    for src in cu_files:
        obj = OBJ_DIR / (src.stem + ".cu.o")
        objs.append(obj)
        if force or _needs_build(src, obj, headers):
            jobs.append(([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], src))
    for src in cpp_files:
        obj = OBJ_DIR / (src.stem + ".cpp.o")
        objs.append(obj)
        if force or _needs_build(src, obj, headers):
            cmd = ["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                   "-I", str(CSRC), "-I", sysconfig.get_paths()["include"]]
            for i in inc:
                cmd += ["-isystem", i]
            cmd += ["-c", str(src), "-o", str(obj)]
            jobs.append((cmd, src))

    def run(job):
        cmd, src = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(run, jobs):
            log = (r.stdout + r.stderr).strip()
            (OBJ_DIR / (src.name + ".log")).write_text(log)
            if r.returncode != 0:
                failed = True
                print(f"[build] FAILED {src.name}\n{log}", file=sys.stderr)
            elif verbose:
                print(f"[build] {src.name}\n{log}")
            else:
                spills = [ln for ln in log.splitlines() if "spill" in ln and "0 bytes spill stores, 0 bytes spill loads" not in ln]
                print(f"[build] {src.name}: ok" + (f" ({len(spills)} kernels spill)" if spills else ""))
    if failed:
        raise RuntimeError("verl_b200 kernel build failed")
    if jobs or not LIB_PATH.exists() or force:
        cmd = ["g++", "-shared", "-o", str(LIB_PATH), *map(str, objs)]
        for d in libdirs:
            cmd += ["-L", d, f"-Wl,-rpath,{d}"]
        cmd += ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            print(r.stdout + r.stderr, file=sys.stderr)
            raise RuntimeError("verl_b200 link failed")
        print(f"[build] linked {LIB_PATH}")
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
