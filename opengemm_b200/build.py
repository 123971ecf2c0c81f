"""Build libopengemm_b200.so with nvcc, for sm_100a only.

Where the library comes from follows the reference's rules
(opengemm/python/build.py:21-24,70-125) with one library serving both
implementations:

* `OPENGEMM_LIB_MM` / `OPENGEMM_LIB_SMM` name a library to load as is.
* Otherwise the in-tree build, `opengemm_b200/lib/libopengemm_b200.so`, is
  used while the digest recorded beside it (`lib/stamp.json`) still matches
  the sources' content - content, not modification times, which a checkout
  or an installer rewrites.  A stale or missing in-tree library is rebuilt in
  place.
* `OPENGEMM_JIT=1` sets the in-tree library aside: the library is compiled
  into a cache directory (`OPENGEMM_CACHE`, else `$XDG_CACHE_HOME/opengemm_b200`,
  else `~/.cache/opengemm_b200`) under a key that digests the sources, the
  compiler's version and the flags, and is reused from there.  The same cache
  takes over when the package directory cannot be written.
"""

import functools
import hashlib
import json
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
UNITS = ("host", "kernels_dense", "kernels_scaled", "kernels_fixed_dense", "kernels_fixed_scaled",
         "kernels_plain_dense", "kernels_plain_scaled", "no_alloc", "quantize")

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


def source_hash():
    """A digest of every source the library is built from: names and content."""
    digest = hashlib.blake2s(digest_size=8)
    units, headers = sources()
    for path in sorted(units + headers):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


@functools.lru_cache(maxsize=None)
def nvcc_version():
    """The compiler's release line, or None when there is no nvcc to ask."""
    try:
        out = subprocess.run([nvcc_path(), "--version"], capture_output=True, text=True, check=True).stdout
    except (OSError, subprocess.CalledProcessError):
        return None
    return next((line.strip() for line in out.splitlines() if "release" in line), "unknown")


def build_hash():
    """The cache key: the sources, the compiler and the flags that turn them into a library."""
    digest = hashlib.blake2s(digest_size=8)
    digest.update(source_hash().encode())
    digest.update((nvcc_version() or "no nvcc").encode())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def cache_dir():
    root = os.environ.get("OPENGEMM_CACHE")
    if root:
        return Path(root)
    return Path(os.environ.get("XDG_CACHE_HOME", Path.home() / ".cache")) / "opengemm_b200"


def stale():
    """True when the in-tree library is missing or was built from other sources."""
    lib = library_file()
    if not lib.exists():
        return True
    try:
        stamp = json.loads((LIB_DIR / "stamp.json").read_text())
    except (OSError, ValueError):
        return True
    return stamp.get("sources") != source_hash()


def compile_library(verbose=False, out=None):
    """Compile every translation unit (in parallel) and link the shared library
    (`out`, default the in-tree file, whose stamp is written beside it)."""
    units, _ = sources()
    target = Path(out) if out is not None else library_file()
    target.parent.mkdir(parents=True, exist_ok=True)
    obj_dir = target.parent / "obj"
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
    temporary = target.parent / f"{LIB_NAME}.{os.getpid()}.tmp"
    link = [nvcc, *ARCH, "-shared", "-Xcompiler", "-fPIC", *map(str, objects), "-o", str(temporary)]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        temporary.unlink(missing_ok=True)
        raise RuntimeError("link failed:\n" + (done.stderr or done.stdout))
    temporary.replace(target)
    (target.parent / "stamp.json").write_text(json.dumps({"sources": source_hash(), "nvcc": nvcc_version(), "arch": ARCH[1]}))
    if verbose:
        log(f"built {target}")
    return target


def cached_library():
    """The library under the cache directory for this exact build, compiled on first use."""
    out = cache_dir() / build_hash() / LIB_NAME
    if not out.exists():
        log(f"compiles once, then cached at {out.parent}")
        compile_library(out=out)
    return out


def library_path(impl):
    """The shared library serving `impl` ("mm" or "smm"): an override from the
    environment, else the in-tree build, compiled now if missing or stale and a
    compiler is at hand."""
    override = os.environ.get(f"OPENGEMM_LIB_{impl.upper()}")
    if override:
        return Path(override)
    if os.environ.get("OPENGEMM_JIT"):
        return cached_library()
    if stale():
        try:
            compile_library()
        except PermissionError:
            return cached_library()
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
