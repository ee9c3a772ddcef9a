"""Ahead-of-time build of the sm_100a kernel library.

`python -m adana_b200.build` compiles every `csrc/*.cu` with nvcc for sm_100a only
(`-gencode arch=compute_100a,code=sm_100a`) and links `adana_b200/lib/libadana_b200.so`
in-tree.  nvcc cross-compiles, so this works on a machine without a GPU.  Objects are
cached by a hash of (source, headers, flags); an unchanged file is not recompiled.

`--debug` builds the checked variant `libadana_b200_debug.so` (no NDEBUG, `-DADANA_DEBUG`): kernels compare
the indices they compute with the extents they were given and report through the status word instead of
touching memory out of range (csrc/common.cuh).  `ADANA_DEBUG=1` makes `adana_b200.ops._lib` load it.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ_DIR = ROOT / "_build"
LIB_DIR = ROOT / "lib"
LIB_PATH = LIB_DIR / "libadana_b200.so"

_COMMON_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
NVCC_FLAGS = _COMMON_FLAGS + ["-DNDEBUG"]
DEBUG_FLAGS = _COMMON_FLAGS + ["-DADANA_DEBUG"]
DEBUG_LIB_PATH = LIB_DIR / "libadana_b200_debug.so"


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _header_digest(debug: bool = False) -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.read_bytes())
    h.update(" ".join(DEBUG_FLAGS if debug else NVCC_FLAGS).encode())
    return h.hexdigest()


def source_digest(debug: bool = False) -> str:
    """Digest of everything that goes into the library (used to detect a stale .so)."""
    h = hashlib.sha256()
    h.update(_header_digest(debug).encode())
    for p in _sources():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, hdr: str, verbose: bool, debug: bool = False) -> tuple[Path, str]:
    tag = ".debug" if debug else ""
    obj = OBJ_DIR / (src.stem + tag + ".o")
    stamp = OBJ_DIR / (src.stem + tag + ".hash")
    digest = hashlib.sha256(src.read_bytes() + hdr.encode()).hexdigest()
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, ""
    cmd = [_nvcc(), *(DEBUG_FLAGS if debug else NVCC_FLAGS), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(digest)
    (OBJ_DIR / (src.stem + tag + ".ptxas.txt")).write_text(proc.stderr)
    return obj, proc.stderr if verbose else ""


def build(verbose: bool = False, force: bool = False, debug: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    lib_path = DEBUG_LIB_PATH if debug else LIB_PATH
    digest = source_digest(debug)
    stamp = LIB_DIR / (lib_path.stem + ".hash")
    if not force and lib_path.exists() and stamp.exists() and stamp.read_text() == digest:
        return lib_path
    if force:
        for f in OBJ_DIR.glob("*.debug.hash" if debug else "*.hash"):
            if debug or not f.name.endswith(".debug.hash"):
                f.unlink()
    hdr = _header_digest(debug)
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
        results = list(ex.map(lambda s: _compile_one(s, hdr, verbose, debug), srcs))
    for _, log in results:
        if log:
            print(log)
    objs = [str(o) for o, _ in results]
    cmd = [_nvcc(), "-shared", "-o", str(lib_path), *objs, "-lcudart"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(digest)
    return lib_path


def is_stale() -> bool:
    stamp = LIB_DIR / "libadana_b200.hash"
    return not (LIB_PATH.exists() and stamp.exists() and stamp.read_text() == source_digest())


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv, debug="--debug" in sys.argv)
    print(f"built {path}")
