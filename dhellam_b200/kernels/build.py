"""In-tree build of the sm_100a kernel library.

Compiles every ``csrc/*.cu`` and ``csrc/*.cpp`` with nvcc for ``sm_100a`` and links one
shared object, ``dhellam_b200/lib/libdhellam_b200.so``, which exposes a plain C API
(``csrc/api.h``) that the Python layer calls through ctypes.  nvcc cross-compiles, so
the build runs on a machine without a GPU.

Capability parity: the reference builds one pybind11 extension ``dhellam._Clib`` from
``csrc/`` (setup.py:132-208, 234-244) for whatever GPU is visible at build time
(setup.py:71-87); here the target is fixed to Blackwell and nothing depends on libtorch.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libdhellam_b200.so"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
    "-DNDEBUG",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _digest(path: Path, flags) -> str:
    h = hashlib.sha1()
    h.update(" ".join(flags).encode())
    h.update(path.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, flags, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    stamp = OBJ / (src.stem + ".sha1")
    dig = _digest(src, flags)
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj
    cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJ / (src.stem + ".log")
    log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    stamp.write_text(dig)
    return obj


def sources():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def build(force: bool = False, verbose: bool = False, jobs: int | None = None) -> Path:
    """Compile what changed and (re)link the library.  Returns the library path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    if force:
        for f in OBJ.glob("*.sha1"):
            f.unlink()
    srcs = sources()
    jobs = jobs or min(len(srcs), os.cpu_count() or 4)
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, NVCC_FLAGS, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel from the last compile logs."""
    out = []
    for log in sorted(OBJ.glob("*.log")):
        out.append(f"== {log.stem}")
        out.append(log.read_text())
    return "\n".join(out)


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
