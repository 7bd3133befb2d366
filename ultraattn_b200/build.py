"""Builds the sm_100a kernel library in-tree with nvcc.

Every ``csrc/*.cu`` file is compiled with ``-gencode arch=compute_100a,code=sm_100a`` and linked
into ``ultraattn_b200/lib/libultraattn_sm100.so``. The library exposes a plain C ABI (loaded with
ctypes by :mod:`ultraattn_b200._lib`), so no PyTorch headers are involved and a full rebuild
takes well under a minute. nvcc cross-compiles, so this works on a machine without a GPU.

The reference ships no native code of its own (it builds NCCL and a flash-attention fork through
``scripts/Makefile:47-96``); this is the equivalent build step of this framework.
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
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libultraattn_sm100.so"
OBJ_DIR = LIB_DIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or add /usr/local/cuda/bin to PATH")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    return max((p.stat().st_mtime for p in hdrs), default=0.0)


STAMP_PATH = LIB_DIR / "build_stamp.txt"


def source_digest() -> str:
    """Hash of everything the library is built from (sources, headers, compiler flags). File times
    do not survive every way of copying a tree to another machine; contents do."""
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def needs_build() -> bool:
    """True when the library is missing or was built from other sources than the present ones."""
    if not LIB_PATH.exists() or not STAMP_PATH.exists():
        return True
    return STAMP_PATH.read_text().strip() != source_digest()


def build_all(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    # several ranks may arrive here at once on a machine where the library is missing: one builds,
    # the others wait for the lock and then find the library up to date
    import fcntl
    lock = open(LIB_DIR / ".build.lock", "w")
    fcntl.flock(lock, fcntl.LOCK_EX)
    try:
        if not force and not needs_build():
            return LIB_PATH
        return _build_locked(nvcc, force, verbose)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        lock.close()


def _build_locked(nvcc: str, force: bool, verbose: bool) -> Path:
    hdr = _newest_header_mtime()

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if (not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime
                and obj.stat().st_mtime > hdr):
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose and r.stderr:
            sys.stderr.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs),
           "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB_PATH)          # a reader never sees a half-written library
    STAMP_PATH.write_text(source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
