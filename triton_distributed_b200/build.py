"""In-tree build of the native library (``_C*.so``) for sm_100a.

Every ``.cu`` file is compiled by ``nvcc -gencode arch=compute_100a,code=sm_100a`` and every ``.cc``
file by ``g++``; objects land in ``csrc/build/`` and the shared object next to this file, so it travels
with the source tree.  Nothing is compiled at import time: ``python -m triton_distributed_b200.build``
(or ``build()`` below) is the only entry point that runs a compiler.

Stands in for the reference's CMake + setup.py build of its plugin and ``csrc`` library
(CMakeLists.txt:183-227, python/setup.py); here there is no compiler plugin to build, only kernels.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = CSRC / "build"
LIB_NAME = "_C"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def lib_path() -> Path:
    return ROOT / f"{LIB_NAME}.so"


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _sources():
    cu = sorted(CSRC.glob("*.cu")) + sorted((CSRC / "mega").glob("*.cu"))
    cc = sorted(CSRC.glob("*.cc")) + sorted((CSRC / "mega").glob("*.cc"))
    return cu, cc


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths()]
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    libdir = ce.library_paths()[0]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={LIB_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    return inc, libdir, defs


def _stamp(cmd, src: Path) -> str:
    h = hashlib.sha1()
    h.update(" ".join(cmd).encode())
    h.update(src.read_bytes())
    for hdr in sorted((CSRC / "include" / "tdb").glob("*")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(cmd, src: Path, obj: Path, verbose: bool):
    stamp_file = obj.with_suffix(obj.suffix + ".stamp")
    stamp = _stamp(cmd, src)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return f"up to date: {src.name}"
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(stamp)
    out = f"compiled: {src.name}"
    if verbose and (res.stdout or res.stderr):
        out += "\n" + res.stdout + res.stderr
    return out


def build(verbose: bool = False, ptxas_info: bool = False, jobs: int | None = None) -> Path:
    """Compile every source for sm_100a and link ``_C.so`` in-tree.  Returns its path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    cuda = _cuda_home()
    nvcc = f"{cuda}/bin/nvcc"
    inc, torch_lib, defs = _torch_flags()
    common_inc = [f"-I{CSRC / 'include'}", f"-I{cuda}/include"]
    cu, cc = _sources()
    tasks = []
    for src in cu:
        obj = OBJ / (src.stem + ".cu.o")
        cmd = [nvcc, *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
               "--expt-relaxed-constexpr", *common_inc, "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd.insert(1, "-Xptxas=-v")
        tasks.append((cmd, src, obj))
    for src in cc:
        obj = OBJ / (src.stem + ".cc.o")
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", *common_inc]
        if src.name.startswith("bind"):
            cmd += inc + defs + ["-fvisibility=hidden"]
        cmd += ["-c", str(src), "-o", str(obj)]
        tasks.append((cmd, src, obj))
    with ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        for msg in ex.map(lambda t: _compile(*t, verbose or ptxas_info), tasks):
            if verbose or ptxas_info:
                print(msg, flush=True)
    objs = [str(t[2]) for t in tasks]
    out = lib_path()
    newest = max(os.path.getmtime(o) for o in objs)
    if not out.exists() or os.path.getmtime(out) < newest:
        link = ["g++", "-shared", "-o", str(out), *objs, f"-L{torch_lib}", "-ltorch_python", "-ltorch", "-ltorch_cpu",
                "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-L{cuda}/lib64", "-lcudart", f"-Wl,-rpath,{torch_lib}",
                "-Wl,--no-as-needed"]
        res = subprocess.run(link, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(link)}\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"linked: {out}")
    return out


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas" in sys.argv)
