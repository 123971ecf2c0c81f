"""Standalone kernel emitter: one (dtype, shape, configuration) as a `.cu` /
`.cuh` pair that depends on nothing but the CUDA toolkit.

Same contract as the reference's emitter (opengemm/python/emit.py:808-896):
`emit_kernel` takes operands (only shapes and dtypes are read) or `m, n, k` and
element names, resolves the stored configuration, and writes `<file>.cu` and
`<file>.cuh`; the first line reads `// opengemm <impl> <dtype> <M> <N> <K>
<entry>`, the second `// config: k=v ...`; the entry point is
`extern "C" void mm_<dtype>_<M>_<N>_<K>(a, b, c, stream)` or
`smm_<dtype>_<M>_<N>_<K>(a, b, sfa, sfb, c, stream)`; it builds with

    nvcc -O3 -std=c++20 -gencode=arch=compute_100a,code=sm_100a \
         --expt-relaxed-constexpr -shared -Xcompiler -fPIC k.cu -o k.so -lcuda

It works with no GPU.  Where the reference inlines its templates and folds
every `if constexpr` with a text-level C++ folder (emit.py:20-806,
fold.py:15-844), this emitter leaves the folding to the compiler: the header
is the library's own kernel source, verbatim, preceded by one macro that
overwrites the run-time tile plan with this shape's literals
(`OG_FIXED_PLAN`), and the `.cu` holds a small generated launcher.
"""

from pathlib import Path

from . import capi
from .configs import resolve_config
from .dtypes import DTYPES, dtype_name, k_of
from .log import log

MARK = "// opengemm"
CSRC = Path(__file__).resolve().parent / "csrc"
OUT_TYPES = {0: "CU_TENSOR_MAP_DATA_TYPE_FLOAT32", 1: "CU_TENSOR_MAP_DATA_TYPE_INT32", 2: "CU_TENSOR_MAP_DATA_TYPE_BFLOAT16",
             3: "CU_TENSOR_MAP_DATA_TYPE_FLOAT16"}
KIND_NAMES = ["KIND_F16", "KIND_TF32", "KIND_I8", "KIND_F8F6F4", "KIND_MXF8F6F4", "KIND_MXF4", "KIND_NVF4"]

# Plan fields the kernel reads that are fixed by (dtype, shape, configuration).
FIXED_FIELDS = (
    "rows_m", "rows_n", "k", "tile_n", "block_k", "mma_k", "k_blocks", "stages", "x_bytes", "y_bytes",
    "stage_bytes", "tx_bytes", "tiles_m", "tiles_n", "num_tiles", "group", "idesc", "acc_slots", "acc_stride",
    "sf_col", "sf_slots", "sf_cols", "tmem_cols", "sf_atoms", "sf_yblocks", "k_groups", "walk",
)


def _strip(text):
    """A library header as a fragment: no include guard, no local includes."""
    keep = []
    for line in text.splitlines():
        if line.startswith("#pragma once") or line.startswith('#include "'):
            continue
        keep.append(line)
    return "\n".join(keep).strip() + "\n"


LAUNCHER = r'''
namespace {{

using og::GemmParams;

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encoder() {{
  static EncodeFn fn = [] {{
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &found) != cudaSuccess ||
        found != cudaDriverEntryPointSuccess)
      return EncodeFn(nullptr);
    return reinterpret_cast<EncodeFn>(sym);
  }}();
  return fn;
}}

bool tile_map(CUtensorMap* map, const void* base, CUtensorMapDataType type, cuuint64_t inner, cuuint64_t rows,
              cuuint64_t row_bytes, cuuint32_t box_inner, cuuint32_t box_rows, CUtensorMapSwizzle swizzle) {{
  const cuuint64_t dims[2] = {{inner, rows}};
  const cuuint64_t strides[1] = {{row_bytes}};
  const cuuint32_t box[2] = {{box_inner, box_rows}};
  const cuuint32_t ones[2] = {{1, 1}};
  EncodeFn encode = encoder();
  return encode && encode(map, type, 2, const_cast<void*>(base), dims, strides, box, ones,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}}

// The launch parameters of the last call, reused while the pointers repeat.
struct Cached {{
  const void* a = nullptr;
  const void* b = nullptr;
  const void* sfa = nullptr;
  const void* sfb = nullptr;
  void* c = nullptr;
  GemmParams params;
}};

void launch(const void* a, const void* b, const void* sfa, const void* sfb, void* c, cudaStream_t stream) {{
  cudaPointerAttributes where;
  if (cudaPointerGetAttributes(&where, a) != cudaSuccess) return;
  int current = -1;
  cudaGetDevice(&current);
  if (current != where.device) cudaSetDevice(where.device);

  static int sm_count[64];
  static bool configured[64];
  const int slot = where.device & 63;
  if (!configured[slot]) {{
    cudaDeviceGetAttribute(&sm_count[slot], cudaDevAttrMultiProcessorCount, where.device);
    cudaFuncSetAttribute(og::gemm_kernel<og::{kind}, {cta_group}, {out_bytes}>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, {smem_attr});
    configured[slot] = true;
  }}

  thread_local Cached cache;
  if (cache.a != a || cache.b != b || cache.sfa != sfa || cache.sfb != sfb || cache.c != c) {{
    GemmParams& p = cache.params;
    std::memset(&p, 0, sizeof p);
    const void* x = {swap} ? b : a;   // the operand on the MMA's 128-row side
    const void* y = {swap} ? a : b;
    bool ok = tile_map(&p.map_x, x, CUtensorMapDataType({x_map}), {k}ull, {rows_m}ull, {k}ull * {x_bits} / 8, {block_k}, 128,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    ok = ok && tile_map(&p.map_y, y, CUtensorMapDataType({y_map}), {k}ull, {rows_n}ull, {k}ull * {y_bits} / 8, {block_k},
                        {y_rows}, CU_TENSOR_MAP_SWIZZLE_128B);
    const bool c_aligned = (reinterpret_cast<uintptr_t>(c) & 15) == 0;
    p.epi_staged = ({epi_staged} && c_aligned) ? 1 : 0;
    p.epi_tma = ({epi_tma} && c_aligned) ? 1 : 0;
    if (p.epi_tma)
      ok = ok && tile_map(&p.map_d, c, {out_type}, {n}ull, {m}ull, {n}ull * {out_bytes}, {out_box}, 32,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if ({scaled}) {{
      const void* sfx = {swap} ? sfb : sfa;
      const void* sfy = {swap} ? sfa : sfb;
      ok = ok && tile_map(&p.map_sfx, sfx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 256, 2ull * {atoms_x}, 256, 256,
                          2 * {sf_atoms} > 0 ? 2 * {sf_atoms} : 1, CU_TENSOR_MAP_SWIZZLE_NONE);
      ok = ok && tile_map(&p.map_sfy, sfy, CU_TENSOR_MAP_DATA_TYPE_UINT8, 256, 2ull * {atoms_y}, 256, 256,
                          2 * {sf_atoms} > 0 ? 2 * {sf_atoms} : 1, CU_TENSOR_MAP_SWIZZLE_NONE);
    }}
    if (!ok) return;
    p.d = c;
    p.wait_limit_ns = 2000ull * 1000 * 1000;
    p.ldd = {n};
    p.transpose_out = {swap};
    p.vec_ok = (c_aligned && ({n}ll * {out_bytes}) % 16 == 0) ? 1 : 0;
    p.pdl = 1;
    OG_FIXED_PLAN(p);
    cache.a = a, cache.b = b, cache.sfa = sfa, cache.sfb = sfb, cache.c = c;
  }}

  const int clusters = std::max(1, std::min({num_tiles}, sm_count[slot] / {cta_group}));
  cudaLaunchConfig_t config = {{}};
  config.gridDim = dim3(clusters * {cta_group}, 1, 1);
  config.blockDim = dim3(og::THREADS, 1, 1);
  config.dynamicSmemBytes = {smem_bytes};
  config.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = {cta_group};
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attrs;
  config.numAttrs = 2;
  cudaLaunchKernelEx(&config, og::gemm_kernel<og::{kind}, {cta_group}, {out_bytes}>, cache.params, og::LaunchPad{{}});
}}

}}  // namespace
'''


def emit(name, m, n, k, config, stem):
    """`(source, header)` text of the standalone kernel for one configuration."""
    if name not in DTYPES:
        raise ValueError(f"standalone kernels are emitted for the fourteen formats {list(DTYPES)}, not {name}")
    d = DTYPES[name]
    lib, g = capi.bind(name, m, n, k, config)
    plan = lib.describe(g)
    entry = f"{'smm' if d.impl == 'smm' else 'mm'}_{name}_{m}_{n}_{k}"
    knobs = {key: int(getattr(g, key)) for key in capi.KERNEL_KEYS[d.impl] + capi.LAUNCH_KEYS[d.impl]}
    tag = (f"{MARK} {d.impl} {name} {m} {n} {k} {entry}\n"
           "// config: " + " ".join(f"{key}={value}" for key, value in sorted(knobs.items())) + "\n")

    fixed = " ".join(f"(p).{field} = {plan[field]}{'u' if field == 'idesc' else ''};" for field in FIXED_FIELDS)
    header = (
        tag
        + "// Standalone kernel written by opengemm_b200.emit_kernel: the library's kernel source with this\n"
        + "// shape's tile plan fixed at compile time.  Include it from the .cu beside it.\n"
        + "#pragma once\n#include <algorithm>\n#include <cstdint>\n#include <cstring>\n#include <cuda.h>\n#include <cuda_runtime.h>\n\n"
        + f"#define OG_FIXED_PLAN(p) do {{ {fixed} }} while (0)\n\n"
        + _strip((CSRC / "ptx.cuh").read_text())
        + "\n"
        + _strip((CSRC / "raster.h").read_text())
        + "\n"
        + _strip((CSRC / "quant_math.cuh").read_text())
        + "\n"
        + _strip((CSRC / "kernel.cuh").read_text())
    )
    values = dict(plan)
    values.update(
        kind=KIND_NAMES[plan["kind"]], smem_attr=227 * 1024 - 1024, y_rows=plan["tile_n"] // plan["cta_group"],
        out_type=OUT_TYPES[plan["out"]], out_box=128 // plan["out_bytes"],
        atoms_x=-(-plan["rows_m"] // 128) * plan["k_groups"], atoms_y=-(-plan["rows_n"] // 128) * plan["k_groups"],
    )
    if d.impl == "smm":
        signature = "const void* a, const void* b, const void* sfa, const void* sfb, void* c, cudaStream_t stream"
        call = "launch(a, b, sfa, sfb, c, stream)"
    else:
        signature = "const void* a, const void* b, void* c, cudaStream_t stream"
        call = "launch(a, b, nullptr, nullptr, c, stream)"
    source = (
        tag
        + f"// C[{m}, {n}] = A[{m}, {k}] . B[{n}, {k}]^T for {name} on sm_100a.  Build:\n"
        + "//   nvcc -O3 -std=c++20 -gencode=arch=compute_100a,code=sm_100a --expt-relaxed-constexpr \\\n"
        + f"//        -shared -Xcompiler -fPIC {stem}.cu -o {stem}.so -lcuda\n"
        + f'#include "{stem}.cuh"\n'
        + LAUNCHER.format(**values)
        + f'\nextern "C" __attribute__((visibility("default"))) void {entry}({signature}) {{\n  {call};\n}}\n'
    )
    return source, header


def parse_tag(text):
    """`(impl, dtype, m, n, k, entry)` from an emitted file's first line."""
    first = text.split("\n", 1)[0]
    if not first.startswith(MARK):
        raise ValueError(
            f"not an opengemm kernel: the first line should read '{MARK} <impl> <dtype> <M> <N> <K> <entry>'"
        )
    impl, dtype, m, n, k, entry = first[len(MARK):].split()
    return impl, dtype, int(m), int(n), int(k), entry


def emit_kernel(a=None, b=None, sfa=None, sfb=None, file=None, atype=None, btype=None, m=None, n=None, k=None,
                sftype=None):
    """Emit a standalone CUDA kernel for one dtype and shape.

    Takes operands, or the shape and element names on their own:

        emit_kernel(a, b, file="k")
        emit_kernel(m=1024, n=1024, k=1024, atype="bf16")
        emit_kernel(m=1024, n=1024, k=1024, atype="e4m3", btype="e5m2")
        emit_kernel(m=1024, n=1024, k=1024, atype="e2m1", sftype="ue4m3")

    Only shapes and dtypes are read, so meta tensors work.  The configuration
    is the stored one for the (dtype, shape), else the heuristic's (or a sweep's
    when OPENGEMM_AUTOTUNE=1).  Emitted kernels run the static tile schedule.

    Args:
        a, b: operands `(M, K)` / `(N, K)`, or None to give `m`, `n`, `k` and names.
        sfa, sfb: scales, for a block-scaled kernel; only the dtype is read.
        file: stem to write `<file>.cu` and `<file>.cuh` to; default `<dtype>_<M>_<N>_<K>`.
        atype, btype: element names ("bf16", "e4m3", "e2m1", ...); `btype` defaults to `atype`.
        m, n, k: the shape when no operands are given; `k` in values.
        sftype: "ue4m3" or "ue8m0": with `atype` it names the block-scaled format.

    Returns:
        `(source, header)` text.
    """
    name = dtype_name(a, b, sfa, atype, btype, sftype)
    if a is not None:
        m, n, k = a.size(0), b.size(0), k_of(DTYPES[name], a.size(1))
    elif None in (m, n, k):
        raise ValueError("without operands, pass m, n and k")
    return write_kernel(name, resolve_config(name, m, n, k), m, n, k, file)


def write_kernel(name, config, m, n, k, file=None):
    """Write the .cu and .cuh pair for one configuration; returns `(source, header)` text."""
    file = Path(file) if file else Path(f"{name}_{m}_{n}_{k}")
    if file.suffix in (".cu", ".cuh"):
        file = file.with_suffix("")
    source, header = emit(name, m, n, k, config, file.name)
    file.parent.mkdir(parents=True, exist_ok=True)
    Path(str(file) + ".cuh").write_text(header)
    Path(str(file) + ".cu").write_text(source)
    log(f"wrote {file}.cu and {file}.cuh")
    return source, header
