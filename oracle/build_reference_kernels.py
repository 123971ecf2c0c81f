"""Compile the reference's two sm_100a kernel libraries from its own sources,
where they lie in a reference checkout, into oracle/_ref/ - test and
measurement infrastructure only.

    python oracle/build_reference_kernels.py /path/to/OpenGEMM [--cutlass [CUTLASS_ROOT]]

Writes `oracle/_ref/libopengemm_mm.so`, `oracle/_ref/libopengemm_smm.so`
(one nvcc call each on opengemm/src/{mm,smm}/capi.cu, with the flags the
reference's own build passes, opengemm/python/build.py:26-37,86-95) and
`oracle/_ref/reference_configs.json` (the entries of its two shipped
configs.json files, merged).  With `--cutlass` it also compiles the
reference's CUTLASS stand-in baselines (scripts/utils/cutlass_ref.cu, built
as scripts/utils/cutlass_ref.py:78-99 builds it) into
`oracle/_ref/libcutlass_ref.so` against a CUTLASS 4.x tree: the one named, or
$OPENGEMM_CUTLASS / $CUTLASS_PATH, or a copy vendored with an installed
flashinfer package; that compile takes about six minutes.  Nothing of the
reference's source is copied; the folder is ignored by git.  The product never
loads these files: they let `python -m opengemm_b200.compare`,
`python -m opengemm_b200.benchmark` and bench.py's side measurement time the
reference's kernels and the CUTLASS baselines on the same buffers as this
library's.
"""

import json
import subprocess
import sys
from pathlib import Path

OUT = Path(__file__).resolve().parent / "_ref"
FLAGS = ["-O3", "-gencode=arch=compute_100a,code=sm_100a", "-std=c++20", "--expt-relaxed-constexpr",
         "--split-compile=0", "-diag-suppress", "68,2361", "-shared", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden"]


def build(reference_root, force=False):
    """Returns the output folder, or None when `reference_root` is not a checkout."""
    src = Path(reference_root) / "opengemm" / "src"
    if not (src / "mm" / "capi.cu").exists():
        return None
    OUT.mkdir(parents=True, exist_ok=True)
    stubs = Path("/usr/local/cuda/targets/x86_64-linux/lib/stubs")
    jobs = []
    for impl in ("mm", "smm"):
        out = OUT / f"libopengemm_{impl}.so"
        if out.exists() and not force:
            continue
        command = ["nvcc", *FLAGS, f"-I{src}", f"-I{src / impl}", str(src / impl / "capi.cu"), "-o", str(out), "-lcuda"]
        if stubs.is_dir():
            command.insert(-1, f"-L{stubs}")
        jobs.append((impl, subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for impl, job in jobs:
        text, _ = job.communicate()
        if job.returncode != 0:
            raise RuntimeError(f"nvcc failed on the reference's {impl} library:\n{text}")
    entries = []
    for impl in ("mm", "smm"):
        entries += json.loads((src / impl / "configs.json").read_text())["entries"]
    (OUT / "reference_configs.json").write_text(json.dumps({"arch": "sm_100", "entries": entries}))
    return OUT


def cutlass_root(named=None):
    """A CUTLASS tree with the sm_100 collectives (4.0 or newer), or None."""
    import os
    import re

    candidates = [named, os.environ.get("OPENGEMM_CUTLASS"), os.environ.get("CUTLASS_PATH")]
    try:
        import flashinfer

        candidates.append(Path(flashinfer.__file__).resolve().parent / "data" / "cutlass")
    except Exception:
        pass
    for root in candidates:
        if not root:
            continue
        header = Path(root) / "include" / "cutlass" / "version.h"
        if not header.exists():
            continue
        major = re.search(r"#define CUTLASS_MAJOR (\d+)", header.read_text())
        if major and int(major.group(1)) >= 4:
            return Path(root)
    return None


def build_cutlass(reference_root, root=None, force=False):
    """Compile the reference's CUTLASS baselines; returns the library path or None."""
    source = Path(reference_root) / "scripts" / "utils" / "cutlass_ref.cu"
    tree = cutlass_root(root)
    if not source.exists() or tree is None:
        return None
    OUT.mkdir(parents=True, exist_ok=True)
    out = OUT / "libcutlass_ref.so"
    if out.exists() and not force:
        return out
    command = ["nvcc", *FLAGS, f"-I{tree / 'include'}", f"-I{tree / 'tools' / 'util' / 'include'}", str(source),
               "-o", str(out), "-lcuda"]
    stubs = Path("/usr/local/cuda/targets/x86_64-linux/lib/stubs")
    if stubs.is_dir():
        command.insert(-1, f"-L{stubs}")
    done = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise RuntimeError("nvcc failed on the reference's CUTLASS baselines:\n" + done.stdout[-4000:])
    return out


if __name__ == "__main__":
    args = sys.argv[1:]
    if not args or args[0].startswith("-"):
        raise SystemExit(__doc__)
    where = build(args[0], force=True)
    print(where if where else f"{args[0]} is not an OpenGEMM checkout")
    if "--cutlass" in args:
        at = args.index("--cutlass")
        named = args[at + 1] if at + 1 < len(args) else None
        print(build_cutlass(args[0], named, force=True) or "no CUTLASS 4.x tree found")
