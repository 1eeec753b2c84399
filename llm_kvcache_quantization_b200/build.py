"""Builds libkvq.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m llm_kvcache_quantization_b200.build [--force] [--verbose] [-DNAME=VALUE ...] [--out PATH]

The library is written next to this file so that it travels with a source
snapshot; nothing is installed into site-packages and no JIT cache is used.
`-D` and `--out` build a second, differently configured copy (the profiling variants: phase
ablations of the decode kernel, occupancy settings); `KVQ_LIBRARY=PATH` makes the package load it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libkvq.so")

SOURCES = ("kvq_api.cu", "kvq_quantize.cu", "kvq_decode.cu", "kvq_dequantize.cu", "kvq_calibrate.cu", "kvq_kivi.cu")

# No --use_fast_math / -ftz / -prec-div=false: the quantizer needs IEEE fp32
# division, RN fp16 conversions and fp16 subnormals to stay bit-exact.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "kvq.h"), __file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), out: str | None = None) -> str:
    """Compile the library if it is missing or older than its sources.  `defines` ("NAME=VALUE") and `out`
    produce a variant next to (never instead of) the default library."""
    if out is None and defines:
        raise ValueError("a build with extra defines needs its own output path")
    target = out or LIB_PATH
    if out is None and not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), "-shared", "-o", target, "-I", INCLUDE, "-I", CSRC, *NVCC_FLAGS]
    cmd += [f"-D{d}" for d in defines]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-lcudart"]          # the driver API entry point for tensor maps is resolved at run time
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libkvq.so")
    return target


if __name__ == "__main__":
    argv = sys.argv[1:]
    out_path = argv[argv.index("--out") + 1] if "--out" in argv else None
    print(build(force="--force" in argv, verbose="--verbose" in argv,
                defines=[a[2:] for a in argv if a.startswith("-D")], out=out_path))
