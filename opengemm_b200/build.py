"""Build libopengemm_b200.so in-tree with nvcc, for sm_100a only.

The reference JIT-compiles two libraries into a content-hashed cache
(opengemm/python/build.py:98-125); here one library serves both, sits beside
the package in `opengemm_b200/lib/`, and is rebuilt when any source is newer
than it.  `OPENGEMM_LIB_MM` / `OPENGEMM_LIB_SMM` still override the path, as
in the reference (build.py:100-102).
"""

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
LIB_DIR = PACKAGE / "lib"
LIB_NAME = "libopengemm_b200.so"
UNITS = ("host", "kernels_dense", "kernels_scaled", "no_alloc", "quantize")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC,-fvisibility=hidden"]


def log(message):
    """Same prefix as the reference's log (opengemm/python/log.py:3-4)."""
    print(f"[OpenGEMM] {message}", file=sys.stderr, flush=True)


def nvcc_path():
    home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    candidate = Path(home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else "nvcc"


def sources():
    units = [CSRC / f"{u}.cu" for u in UNITS if (CSRC / f"{u}.cu").exists()]
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [ROOT / "include" / "opengemm_b200.h"]
    return units, headers


def library_file():
    return LIB_DIR / LIB_NAME


def stale():
    lib = library_file()
    if not lib.exists():
        return True
    units, headers = sources()
    built = lib.stat().st_mtime
    return any(p.stat().st_mtime > built for p in units + headers)


def compile_library(verbose=False):
    """Compile every translation unit (in parallel) and link the shared library."""
    units, _ = sources()
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = nvcc_path()

    def one(unit):
        obj = obj_dir / (unit.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-c", str(unit), "-o", str(obj)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        (obj_dir / (unit.stem + ".log")).write_text(done.stdout + done.stderr)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on {unit.name}:\n{done.stderr or done.stdout}")
        return obj

    log(f"compiling {LIB_NAME} for sm_100a ({len(units)} translation units)")
    with ThreadPoolExecutor(max_workers=len(units)) as pool:
        objects = list(pool.map(one, units))
    temporary = LIB_DIR / (LIB_NAME + ".tmp")
    link = [nvcc, *ARCH, "-shared", "-Xcompiler", "-fPIC", *map(str, objects), "-o", str(temporary)]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError("link failed:\n" + (done.stderr or done.stdout))
    temporary.replace(library_file())
    if verbose:
        log(f"built {library_file()}")
    return library_file()


def library_path(impl):
    """The shared library serving `impl` ("mm" or "smm"): an override from the
    environment, else the in-tree build, compiled now if missing or stale and a
    compiler is at hand."""
    override = os.environ.get(f"OPENGEMM_LIB_{impl.upper()}")
    if override:
        return Path(override)
    if stale():
        try:
            compile_library()
        except (OSError, RuntimeError) as exc:
            if not library_file().exists():
                raise RuntimeError(
                    f"{LIB_NAME} is not built and cannot be built here ({exc}); there is no CPU fallback"
                ) from exc
    return library_file()


def prebuild():
    """Compile the library now rather than on the first gemm() (opengemm/python/build.py:128-132)."""
    if stale():
        compile_library(verbose=True)
    return library_file()


if __name__ == "__main__":
    compile_library(verbose=True)
