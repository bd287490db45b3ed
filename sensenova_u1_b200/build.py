"""Builds the native library of this package for sm_100a, in-tree.

Every ``.cu`` file under ``csrc/`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into
``sensenova_u1_b200/lib/libsnu1_b200.so`` (plain C ABI, loaded with ctypes by
``sensenova_u1_b200.ops._lib``).  nvcc cross-compiles without a GPU.

    python -m sensenova_u1_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "lib"
OBJ_DIR = OUT_DIR / "obj"
LIB_NAME = "libsnu1_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(src: Path, force: bool, verbose: bool) -> tuple[Path, bool]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    dig = _digest(src)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj, False
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr, flush=True)
    stamp.write_text(dig)
    return obj, True


def lib_path() -> Path:
    return OUT_DIR / LIB_NAME


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (when stale) and link the library; returns its path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = _sources()
    if not srcs:
        raise RuntimeError(f"no .cu sources under {CSRC}")
    objs: list[Path] = []
    rebuilt = False
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        for obj, did in pool.map(lambda s: _compile_one(s, force, verbose), srcs):
            objs.append(obj)
            rebuilt = rebuilt or did
    out = lib_path()
    if rebuilt or not out.exists():
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-cudart", "static",
               "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args(argv)
    print(build(force=ns.force, verbose=ns.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
