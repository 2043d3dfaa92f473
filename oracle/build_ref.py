#!/usr/bin/env python
"""Side-build of the REFERENCE's own CUDA extensions for sm_100a, as checker binaries (test infrastructure only).

    python oracle/build_ref.py /path/to/reference [names ...]

Compiles, from the sources where they lie in the reference checkout (nothing is copied), the extensions that depend
only on torch and the CUDA toolkit:

    quant_sscan_cuda           csrc/selective_scan/quant_sscan.cpp, quant_sscan_fwd.cu
    quant_causal_conv1d_cuda   csrc/causal_conv1d/quant_causal_conv1d{.cpp,_fwd.cu,_update.cu}
    quamba2_conv1d_cuda        csrc/causal_conv1d/quamba2_conv1d{.cpp,_fwd.cu,_update.cu}
    quant_hadamard             csrc/hadamard/quant_hadamard.cpp, quant_hadamard_fwd.cu
    quant_embedding_cuda       csrc/embedding/quant_embedding.cpp, quant_embedding_fwd.cu

with the reference's own compiler flags (setup.py:87-347) and ``-gencode arch=compute_100a,code=sm_100a``.  Outputs go to
oracle/_ref/<name>/ (git-ignored).  ``quant_linear_cuda`` needs the CUTLASS sources of an empty submodule and is not
built.  The GPU tests import these modules when present and compare this package's kernels with them; nothing in the
product path does.
"""
import sys
from pathlib import Path

OUT = Path(__file__).resolve().parent / "_ref"

EXTENSIONS = {
    "quant_sscan_cuda": ("selective_scan", ["quant_sscan.cpp", "quant_sscan_fwd.cu"]),
    "quant_causal_conv1d_cuda": ("causal_conv1d", ["quant_causal_conv1d.cpp", "quant_causal_conv1d_fwd.cu",
                                                   "quant_causal_conv1d_update.cu"]),
    "quamba2_conv1d_cuda": ("causal_conv1d", ["quamba2_conv1d.cpp", "quamba2_conv1d_fwd.cu", "quamba2_conv1d_update.cu"]),
    "quant_hadamard": ("hadamard", ["quant_hadamard.cpp", "quant_hadamard_fwd.cu"]),
    "quant_embedding_cuda": ("embedding", ["quant_embedding.cpp", "quant_embedding_fwd.cu"]),
}

NVCC_FLAGS = ["-O3", "-std=c++17", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
              "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_HALF2_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_OPERATORS__",
              "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
              "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math", "-lineinfo", "-DCUDA_ARCH=100",
              "-gencode", "arch=compute_100a,code=sm_100a", "--threads", "4"]


def build(ref: Path, names):
    import os
    from torch.utils import cpp_extension
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    results = {}
    for name in names:
        sub, files = EXTENSIONS[name]
        src_dir = ref / "csrc" / sub
        bdir = OUT / name
        bdir.mkdir(parents=True, exist_ok=True)
        try:
            cpp_extension.load(name=name, sources=[str(src_dir / f) for f in files], extra_cflags=["-O3", "-std=c++17"],
                               extra_cuda_cflags=NVCC_FLAGS, extra_include_paths=[str(ref / "csrc"), str(src_dir)],
                               build_directory=str(bdir), verbose=False, is_python_module=False)
            results[name] = "built"
        except Exception as e:        # record and go on: a kernel that does not build is "reference kernel unavailable"
            results[name] = f"FAILED: {str(e).splitlines()[-1][:200] if str(e) else type(e).__name__}"
        print(name, "->", results[name], flush=True)
    return results


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    build(Path(sys.argv[1]), sys.argv[2:] or list(EXTENSIONS))
