"""In-tree build of the sm_100a kernel library.

All CUDA sources under ``csrc/`` are compiled by ``nvcc`` for
``arch=compute_100a,code=sm_100a`` and linked into one shared object,
``_lib/liblevanter_b200.so``, which :mod:`levanter_b200.ops.lib` loads with
``ctypes``.  The kernels expose plain ``extern "C"`` launchers (raw pointers +
stream), so nothing here depends on the PyTorch C++ headers and a full
rebuild takes seconds.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIBDIR = Path(__file__).resolve().parent / "_lib"
LIBNAME = "liblevanter_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _digest(paths: list[Path]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def lib_path() -> Path:
    return LIBDIR / LIBNAME


def is_current() -> bool:
    stamp = LIBDIR / "build.stamp"
    return lib_path().exists() and stamp.exists() and stamp.read_text().strip() == _digest(_sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link the shared object.  Returns its path."""
    srcs = _sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources in {CSRC}")
    if not force and is_current():
        return lib_path()
    LIBDIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    objs: list[Path] = []
    logs: dict[str, str] = {}

    def compile_one(src: Path) -> Path:
        obj = LIBDIR / (src.stem + ".o")
        flags = NVCC_FLAGS if src.suffix == ".cu" else ["-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        logs[src.name] = r.stderr + r.stdout
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr}\n{r.stdout}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    out = lib_path()
    cmd = [nvcc, "-shared", "-o", str(out), *[str(o) for o in objs], "-gencode", "arch=compute_100a,code=sm_100a", "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr}")
    (LIBDIR / "ptxas.log").write_text("\n".join(f"==== {k}\n{v}" for k, v in sorted(logs.items())))
    (LIBDIR / "build.stamp").write_text(_digest(srcs))
    if verbose:
        print((LIBDIR / "ptxas.log").read_text())
    return out


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
