"""Builds the in-tree native libraries with nvcc for sm_100a.

    python tensorrt_b200/csrc/build.py            # build what is out of date
    python tensorrt_b200/csrc/build.py --force

(run as a file, not through the package: importing tensorrt_b200 needs the library this script builds)

Outputs (git-ignored, kept next to the sources so they travel with the tree):
    tensorrt_b200/libbert_b200.so          kernels + C ABI (include/bert_b200.h)
    tensorrt_b200/libbert_b200_plugin.so   IPluginV3 adapters (needs the TensorRT public headers)
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
ROOT = PKG.parent
OBJ = PKG / "build"
LIB = PKG / "libbert_b200.so"
PLUGIN_LIB = PKG / "libbert_b200_plugin.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", f"-I{ROOT / 'include'}", f"-I{CSRC}",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return nvcc


def _trt_include() -> Path | None:
    """Directory holding NvInferRuntime.h (TensorRT public headers), if any."""
    # TENSORRT_INCLUDE_DIR, a TensorRT-OSS checkout named by REFERENCE_ROOT or lying next to this repository, system paths
    ref = os.environ.get("REFERENCE_ROOT") or ROOT.parent / "reference"
    cands = [os.environ.get("TENSORRT_INCLUDE_DIR"), Path(ref) / "include", "/usr/include/x86_64-linux-gnu", "/usr/local/tensorrt/include"]
    for c in cands:
        if c and (Path(c) / "NvInferRuntime.h").exists():
            return Path(c)
    return None


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


def _compile(src: Path, extra: list[str]) -> Path:
    obj = OBJ / (src.stem + ".o")
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((ROOT / "include").glob("*.h")) + list((CSRC / "plugin").glob("*.h"))
    if _newer(obj, [src] + headers):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    if force:
        for f in OBJ.glob("*.o"):
            f.unlink()
    srcs = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, []), srcs))
    if force or not _newer(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(f"built {LIB}")
    trt = _trt_include()
    psrcs = sorted((CSRC / "plugin").glob("*.cpp"))
    if trt is not None and psrcs:
        extra = [f"-I{trt}", f"-I{CSRC / 'plugin'}"]
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            pobjs = list(ex.map(lambda s: _compile(s, extra), psrcs))
        if force or not _newer(PLUGIN_LIB, pobjs + [LIB]):
            cmd = [_nvcc(), "-shared", "-o", str(PLUGIN_LIB), *map(str, pobjs), f"-L{PKG}", "-l:libbert_b200.so",
                   "-Xlinker", "-rpath,$ORIGIN", "-lcudart"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"plugin link failed:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"built {PLUGIN_LIB}")
    elif verbose and psrcs:
        print("TensorRT headers not found: keeping the existing plugin library" if PLUGIN_LIB.exists() else "TensorRT headers not found: plugin library not built")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
