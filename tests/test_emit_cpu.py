"""The standalone-kernel emitter without a GPU: files, tag lines, and that the
emitted pair compiles with the documented nvcc line and exports its entry point."""

import shutil
import subprocess

import pytest

import opengemm_b200 as og
from opengemm_b200 import emit, run


def test_emit_needs_no_gpu_and_writes_the_tagged_pair(tmp_path):
    stem = tmp_path / "k1024"
    source, header = og.emit_kernel(m=1024, n=1024, k=1024, atype="bf16", file=str(stem))
    cu, cuh = tmp_path / "k1024.cu", tmp_path / "k1024.cuh"
    assert cu.read_text() == source and cuh.read_text() == header
    first, second = source.splitlines()[:2]
    assert first == "// opengemm mm bf16 1024 1024 1024 mm_bf16_1024_1024_1024"
    assert second.startswith("// config: ") and "output_n=" in second and "use_2cta=" in second
    assert emit.parse_tag(source) == ("mm", "bf16", 1024, 1024, 1024, "mm_bf16_1024_1024_1024")
    assert emit.parse_tag(header)[5] == "mm_bf16_1024_1024_1024"
    assert '#include "k1024.cuh"' in source
    assert '#include "' not in header  # self-contained: only toolkit headers
    assert "OG_FIXED_PLAN" in header and "tcgen05.mma" in header
    assert 'extern "C"' in source and "mm_bf16_1024_1024_1024(const void* a, const void* b, void* c, cudaStream_t stream)" in source
    with pytest.raises(ValueError, match="not an opengemm kernel"):
        emit.parse_tag("int main() {}\n")


def test_emit_names_block_scaled_and_mixed_formats(tmp_path):
    source, _ = og.emit_kernel(m=256, n=384, k=512, atype="e2m1", sftype="ue4m3", file=str(tmp_path / "a"))
    assert emit.parse_tag(source)[:2] == ("smm", "nvfp4")
    assert "smm_nvfp4_256_384_512(const void* a, const void* b, const void* sfa, const void* sfb, void* c, cudaStream_t stream)" in source
    source, _ = og.emit_kernel(m=256, n=384, k=512, atype="e4m3", btype="e5m2", file=str(tmp_path / "b"))
    assert emit.parse_tag(source)[1] == "e4m3xe5m2"
    with pytest.raises(ValueError, match="pass m, n and k"):
        og.emit_kernel(atype="bf16")


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc")
def test_emitted_pair_compiles_and_exports_its_entry_point(tmp_path):
    og.emit_kernel(m=300, n=520, k=768, atype="s8", file=str(tmp_path / "ks8"))
    library = run.build(tmp_path / "ks8.cu")
    symbols = subprocess.run(["nm", "-D", str(library)], capture_output=True, text=True).stdout
    assert " T mm_s8_300_520_768" in symbols
    again = run.build(tmp_path / "ks8.cu")  # reused, not rebuilt
    assert again == library
