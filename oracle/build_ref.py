"""TEST INFRASTRUCTURE: build oracle/_ref/libnott_ref.so, oracle/_ref/libnott_binding.so and
oracle/_ref/liboracle_rowops.so.

libnott_ref.so   = oracle/ref_harness.cpp compiled against the reference's own
                   headers (read in place from the reference checkout, never
                   copied) and the installed libtorch.  Needs the reference tree.
libnott_binding.so = oracle/ref_binding_harness.cpp: the reference's RegisteredLayer / ForwardBinding
                   (src/layer/registry.hpp) driving this library's drop-in modules; needs the
                   reference tree, libtorch with CUDA and the built libnott_b200.so.
liboracle_rowops.so = oracle/oracle_rowops.c, the plain-C restatement; needs only gcc.

The reference checkout is found through NOTT_REFERENCE_ROOT, else in a `reference` folder beside
this repository.

Outputs go to oracle/_ref/ only (git-ignored, shipped with the tree).
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
REF_LIB = OUT / "libnott_ref.so"
BINDING_LIB = OUT / "libnott_binding.so"
C_LIB = OUT / "liboracle_rowops.so"


def reference_root() -> Path | None:
    for cand in (os.environ.get("NOTT_REFERENCE_ROOT"), HERE.parent.parent / "reference"):
        if cand and (Path(cand) / "src" / "activation" / "apply.hpp").exists():
            return Path(cand)
    return None


def _newer(target: Path, *sources: Path) -> bool:
    return target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources)


def build_c_oracle(force: bool = False) -> Path:
    src = HERE / "oracle_rowops.c"
    OUT.mkdir(exist_ok=True)
    if not force and _newer(C_LIB, src):
        return C_LIB
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-std=gnu11", "-ffp-contract=off", "-o", str(C_LIB), str(src), "-lm"]
    subprocess.run(cmd, check=True)
    return C_LIB


def build_reference(force: bool = False) -> Path | None:
    """Returns the library path, or None when the reference tree is not present
    (then a previously built library, if any, is used as is)."""
    root = reference_root()
    src = HERE / "ref_harness.cpp"
    OUT.mkdir(exist_ok=True)
    if root is None:
        return REF_LIB if REF_LIB.exists() else None
    if not force and _newer(REF_LIB, src):
        return REF_LIB
    import torch

    tdir = Path(torch.__file__).resolve().parent
    cmd = [
        "g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-w",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
        f"-I{root}", f"-I{tdir / 'include'}", f"-I{tdir / 'include' / 'torch' / 'csrc' / 'api' / 'include'}",
        "-I/usr/local/cuda/include",
        str(src), "-o", str(REF_LIB),
        f"-L{tdir / 'lib'}", "-ltorch", "-ltorch_cpu", "-lc10",
        f"-Wl,-rpath,{tdir / 'lib'}",
    ]
    subprocess.run(cmd, check=True)
    return REF_LIB


def build_binding(force: bool = False) -> Path | None:
    """The binding harness; None when the reference tree is absent (a prebuilt file is then used as is)."""
    root = reference_root()
    src = HERE / "ref_binding_harness.cpp"
    repo = HERE.parent
    host_hdr = repo / "thot_b200" / "host" / "nott_b200.hpp"
    nb2 = repo / "thot_b200" / "libnott_b200.so"
    OUT.mkdir(exist_ok=True)
    if root is None:
        return BINDING_LIB if BINDING_LIB.exists() else None
    if not nb2.exists():
        raise RuntimeError("build thot_b200/libnott_b200.so first")
    if not force and _newer(BINDING_LIB, src, host_hdr, repo / "include" / "nott_b200.h"):
        return BINDING_LIB
    import torch

    tdir = Path(torch.__file__).resolve().parent
    cmd = [
        "g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-w",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
        f"-I{root}", f"-I{repo}", f"-I{tdir / 'include'}", f"-I{tdir / 'include' / 'torch' / 'csrc' / 'api' / 'include'}",
        "-I/usr/local/cuda/include",
        str(src), "-o", str(BINDING_LIB),
        f"-L{tdir / 'lib'}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
        f"-L{nb2.parent}", "-l:libnott_b200.so",
        f"-Wl,-rpath,{tdir / 'lib'}", "-Wl,-rpath,$ORIGIN/../../thot_b200",
    ]
    subprocess.run(cmd, check=True)
    return BINDING_LIB


if __name__ == "__main__":
    print(build_c_oracle(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
    print(build_binding(force="--force" in sys.argv))
