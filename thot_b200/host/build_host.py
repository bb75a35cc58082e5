"""In-tree build of the C++ host layer's Python binding (thot_b200/_nott_b200_host.so).

Compiles host/bindings.cpp (which includes host/nott_b200.hpp) against libtorch and links
libnott_b200.so next to it (rpath $ORIGIN).  Plain g++; no JIT cache is involved, so the
built file travels with the tree.
"""
from __future__ import annotations

import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
OUT = PKG / "_nott_b200_host.so"


def build(force: bool = False) -> Path:
    srcs = [HERE / "bindings.cpp", HERE / "nott_b200.hpp", PKG.parent / "include" / "nott_b200.h"]
    if not force and OUT.exists() and all(OUT.stat().st_mtime >= s.stat().st_mtime for s in srcs):
        return OUT
    import torch
    import pybind11  # noqa: F401

    tdir = Path(torch.__file__).resolve().parent
    cmd = [
        "g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
        "-DTORCH_EXTENSION_NAME=_nott_b200_host", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-I{tdir / 'include'}", f"-I{tdir / 'include' / 'torch' / 'csrc' / 'api' / 'include'}",
        f"-I{sysconfig.get_paths()['include']}", "-I/usr/local/cuda/include",
        str(HERE / "bindings.cpp"), "-o", str(OUT),
        f"-L{tdir / 'lib'}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python",
        f"-L{PKG}", "-l:libnott_b200.so",
        f"-Wl,-rpath,{tdir / 'lib'}", "-Wl,-rpath,$ORIGIN",
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
