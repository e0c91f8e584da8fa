"""Builds the sm_100a shared libraries of the NVFP4 hot path with nvcc, in-tree.

    python tirx-kernels_b200/build.py [--force] [--verbose]

Outputs (git-ignored, next to this file):
    lib/libb200nvfp4.so           quantizers, GEMM, probe  (the product; no cuBLAS dependency)
    lib/libb200nvfp4_cublaslt.so  cuBLASLt NVFP4 baseline   (library peer used only by benches)

nvcc cross-compiles without a GPU, so this runs on a CPU-only machine.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build"
INCLUDE = ROOT.parent / "include"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    f"-I{INCLUDE}",
]

MAIN_SOURCES = ["capi.cu", "quantize.cu", "rmsnorm_fp4quant.cu", "add_rmsnorm_fp4quant.cu", "nvfp4_gemm.cu"]
CUBLASLT_SOURCES = ["cublaslt_baseline.cu"]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else "nvcc"


def _headers_mtime() -> float:
    stamps = [p.stat().st_mtime for p in CSRC.glob("*.cuh")]
    stamps += [p.stat().st_mtime for p in INCLUDE.glob("*.h")]
    stamps.append(Path(__file__).stat().st_mtime)
    return max(stamps)


def _run(cmd: list[str], verbose: bool, log_name: str) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    OBJ.mkdir(exist_ok=True)
    (OBJ / f"{log_name}.log").write_text(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({proc.returncode}): {' '.join(cmd)}")


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    OBJ.mkdir(exist_ok=True)
    obj = OBJ / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if not force and obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    _run([_nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, "-c", str(src), "-o", str(obj)], verbose, src.stem)
    return obj


def _link(objs: list[Path], out: Path, extra: list[str], force: bool, verbose: bool) -> None:
    LIB.mkdir(exist_ok=True)
    if not force and out.exists() and all(out.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return
    cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(out), *map(str, objs), *extra]
    _run(cmd, verbose, out.stem)


def build(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    """Compile every CUDA source for sm_100a and link both shared libraries."""
    built: dict[str, Path] = {}
    main_objs = [_compile(CSRC / s, force, verbose) for s in MAIN_SOURCES if (CSRC / s).exists()]
    main = LIB / "libb200nvfp4.so"
    _link(main_objs, main, ["-cudart", "static"], force, verbose)
    built["main"] = main
    lt_sources = [CSRC / s for s in CUBLASLT_SOURCES if (CSRC / s).exists()]
    if lt_sources:
        lt_objs = [_compile(s, force, verbose) for s in lt_sources]
        lt = LIB / "libb200nvfp4_cublaslt.so"
        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        _link(lt_objs, lt, ["-cudart", "static", f"-L{cuda_home}/lib64", "-lcublasLt"], force, verbose)
        built["cublaslt"] = lt
    return built


if __name__ == "__main__":
    paths = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    for name, path in paths.items():
        print(f"{name}: {path}")
