"""Build the CUDA library in-tree with nvcc for sm_100a (no JIT cache, no torch extension).

    python -m quamba_b200.build            # builds quamba_b200/libquamba_b200.so if out of date
"""
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libquamba_b200.so"
SOURCES = ["lib.cu", "conv1d.cu", "hadamard.cu", "hadamard_tc.cu", "sscan.cu", "ssd.cu", "ssd_tc.cu", "linear.cu", "gemm_tc.cu", "norm.cu",
           "embedding.cu", "decode.cu", "peer.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _stale(obj: Path, src: Path) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    deps = [src] + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc")) + [PKG.parent / "include" / "quamba_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    objs, procs = [], []
    for name in SOURCES:
        src, obj = CSRC / name, objdir / (name + ".o")
        objs.append(obj)
        if force or _stale(obj, src):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for name, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(f"--- nvcc {name} ---\n{out}\n")
        (objdir / (name + ".log")).write_text(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the log above")
    if procs or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
