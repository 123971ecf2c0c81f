"""Compile the reference's two sm_100a kernel libraries from its own sources,
where they lie in a reference checkout, into oracle/_ref/ - test and
measurement infrastructure only.

    python oracle/build_reference_kernels.py /path/to/OpenGEMM

Writes `oracle/_ref/libopengemm_mm.so`, `oracle/_ref/libopengemm_smm.so`
(one nvcc call each on opengemm/src/{mm,smm}/capi.cu, with the flags the
reference's own build passes, opengemm/python/build.py:26-37,86-95) and
`oracle/_ref/reference_configs.json` (the entries of its two shipped
configs.json files, merged).  Nothing of the reference's source is copied;
the folder is ignored by git.  The product never loads these files: they let
`python -m opengemm_b200.compare` and bench.py's side measurement time the
reference's kernels on the same buffers as this library's.
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


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    where = build(sys.argv[1], force=True)
    print(where if where else f"{sys.argv[1]} is not an OpenGEMM checkout")
