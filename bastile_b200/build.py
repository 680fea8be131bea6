"""Build ``libbastile_b200.so`` (the sm_100a kernels behind the C ABI) in-tree.

``python -m bastile_b200.build`` compiles every ``csrc/*.cu`` with nvcc for
``sm_100a`` only and links one shared library next to this file.  Objects are
cached under ``csrc/_obj`` and rebuilt when a source or header is newer.  No
torch headers are involved: the library exposes plain ``extern "C"`` entry
points (``include/bastile_b200.h``) that the Python ops reach through ctypes.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = CSRC / "_obj"
LIB_PATH = PKG_DIR / "libbastile_b200.so"
INCLUDE = PKG_DIR.parent / "include"

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set NVCC or add /usr/local/cuda/bin to PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_mtime() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, verbose: bool, ptxas_v: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if ptxas_v:
        cmd[1:1] = ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if ptxas_v:
        print(res.stderr)
    return obj


def build(verbose: bool = False, force: bool = False, ptxas_v: bool = False) -> Path:
    """Compile and link the library; returns its path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, ptxas_v), srcs))
    if LIB_PATH.exists() and all(LIB_PATH.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return LIB_PATH
    cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    p = build(verbose=True, force="--force" in sys.argv, ptxas_v="--ptxas-v" in sys.argv)
    print(f"built {p}")
