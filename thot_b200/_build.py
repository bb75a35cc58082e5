"""In-tree build of libnott_b200.so (hand-written sm_100a kernels + the C ABI) and of
libnott_b200_linear.so (the tensor-core linear layer, thot_b200/csrc_linear: the only sources that
instantiate CUTLASS collectives; the core library opens it on first use and works without it).

nvcc cross-compiles for sm_100a without a GPU; each translation unit is compiled in parallel and
the objects are linked into the two libraries next to this file, so they travel with the tree.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libnott_b200.so"
CSRC_LINEAR = PKG_DIR / "csrc_linear"
OBJ_DIR_LINEAR = PKG_DIR / "build_linear"
LINEAR_LIB_PATH = PKG_DIR / "libnott_b200_linear.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: libnott_b200.so cannot be built (there is no CPU fallback)")


def _nccl_include() -> list[str]:
    """The NCCL header (types and enums only; the functions are resolved with dlopen at run time)."""
    try:
        import nvidia.nccl as pkg
        inc = Path(list(pkg.__path__)[0]) / "include"
        if (inc / "nccl.h").exists():
            return ["-I", str(inc)]
    except Exception:
        pass
    return []


def _cutlass_include() -> list[str]:
    """CUTLASS/CuTe headers (header-only) for the tensor-core linear layer; the tree vendored with flashinfer."""
    cands = []
    if os.environ.get("CUTLASS_PATH"):
        cands.append(Path(os.environ["CUTLASS_PATH"]))
    try:
        import importlib.util
        spec = importlib.util.find_spec("flashinfer")
        if spec is not None and spec.submodule_search_locations:
            cands.append(Path(list(spec.submodule_search_locations)[0]) / "data" / "cutlass")
    except Exception:
        pass
    for root in cands:
        if (root / "include" / "cutlass" / "cutlass.h").exists():
            return ["-I", str(root / "include"), "-I", str(root / "tools" / "util" / "include")]
    return []


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
                    + [PKG_DIR.parent / "include" / "nott_b200.h"]):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if sources changed) and return the path of libnott_b200.so."""
    stamp_file = OBJ_DIR / "stamp.txt"
    stamp = _stamp()
    if not force and LIB_PATH.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *_nccl_include(), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH), *map(str, objs), "-ldl"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(stamp)
    return LIB_PATH


def _stamp_linear() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC_LINEAR.glob("*.cu")) + list(CSRC_LINEAR.glob("*.cuh")) + [CSRC / "nb2_common.cuh", PKG_DIR.parent / "include" / "nott_b200.h"]):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_linear(force: bool = False) -> Path | None:
    """Compile thot_b200/csrc_linear into libnott_b200_linear.so.  Returns None (and leaves a previously built
    library as it is) when the sources are not in the tree."""
    srcs = sorted(CSRC_LINEAR.glob("*.cu")) if CSRC_LINEAR.is_dir() else []
    if not srcs:
        return LINEAR_LIB_PATH if LINEAR_LIB_PATH.exists() else None
    stamp_file = OBJ_DIR_LINEAR / "stamp.txt"
    stamp = _stamp_linear()
    if not force and LINEAR_LIB_PATH.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LINEAR_LIB_PATH
    inc = _cutlass_include()
    if not inc:
        raise RuntimeError("CUTLASS headers not found (set CUTLASS_PATH): the tensor-core linear layer cannot be built")
    nvcc = _nvcc()
    OBJ_DIR_LINEAR.mkdir(exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR_LINEAR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *inc, "-diag-suppress", "20012", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(4, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LINEAR_LIB_PATH), *map(str, objs)]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(stamp)
    return LINEAR_LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_linear(force="--force" in sys.argv))
