"""Build the CUDA library in-tree: ``python -m omnikv_b200.build``.

Every ``csrc/*.cu`` is compiled for sm_100a only and linked into
``omnikv_b200/_lib/libomnikv_b200.so`` (a plain C-ABI shared library: it links the CUDA runtime
statically and nothing of PyTorch).  Objects are rebuilt only when a source or header is newer.

``--trace`` builds a second library beside it, ``libomnikv_b200_trace.so``, with ``-DOMNIKV_TRACE``: the
weight-streaming and attention kernels then stamp ``%globaltimer`` at their stages (a profiling aid read by
``profile_cases.py tp_timeline``; select it with ``OMNIKV_B200_LIB=<path>``).  The default library has none of it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "_lib"
LIB = LIBDIR / "libomnikv_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
# --use_fast_math would flush denormals and use approximate division in the softmax weights; the parity
# tolerances are set on fp32-accurate scores, so it is NOT used.
NVCC_FLAGS.remove("--use_fast_math")


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_extension(verbose: bool = False, force: bool = False, trace: bool = False) -> Path:
    LIBDIR.mkdir(exist_ok=True)
    objdir = LIBDIR / "trace" if trace else LIBDIR
    objdir.mkdir(exist_ok=True)
    lib = LIBDIR / "libomnikv_b200_trace.so" if trace else LIB
    extra = ["-DOMNIKV_TRACE"] if trace else []
    headers = list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    nvcc = _nvcc()

    def compile_one(src: Path):
        obj = objdir / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(ROOT / "include"), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            (objdir / (src.stem + ".ptxas.log")).write_text(r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stderr}")
            if verbose:
                print(r.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _stale(lib, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), *map(str, objs),
               "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr}")
    return lib


if __name__ == "__main__":
    print(build_extension(verbose="-v" in sys.argv, force="-f" in sys.argv, trace="--trace" in sys.argv))
