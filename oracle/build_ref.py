"""Builds oracle/_ref/libref_bert.so: the REFERENCE's own BERT plugin kernels, compiled from the sources where they
lie in the TensorRT-OSS tree (never copied), plus oracle/ref_shim.cu. Test infrastructure only.

    python oracle/build_ref.py [--force]

Needs a checkout of the reference tree (environment variable REFERENCE_ROOT, else the build machine's default
location below) and nvcc; without the tree an existing library is kept and nothing is built. The reference's build system is not run: each source is compiled directly.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
LIB = OUT / "libref_bert.so"
# the TensorRT-OSS checkout: REFERENCE_ROOT, else a directory "reference" next to this repository
REF = Path(os.environ.get("REFERENCE_ROOT") or HERE.parent.parent / "reference")

PLUGIN_SOURCES = [
    "plugin/skipLayerNormPlugin/skipLayerNormKernel.cu",
    "plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernelHFace.cu",
    "plugin/skipLayerNormPlugin/skipLayerNormInt8InterleavedKernelMTron.cu",
    "plugin/embLayerNormPlugin/embLayerNormKernel.cu",
    "plugin/embLayerNormPlugin/embLayerNormVarSeqlenKernelHFace.cu",
    "plugin/embLayerNormPlugin/embLayerNormVarSeqlenKernelMTron.cu",
    "plugin/common/cudaDriverWrapper.cpp",
    "plugin/vc/checkMacrosPlugin.cpp",
]


def _sources():
    srcs = [REF / s for s in PLUGIN_SOURCES]
    # the precompiled sm100 attention kernels the reference ships as byte arrays (executed, never inspected)
    srcs += sorted((REF / "plugin/bertQKVToContextPlugin/fused_multihead_attention_v2").glob("*kernel.sm100.cpp"))
    # and the fixed-length kernels of plugin versions 1-3
    srcs += sorted((REF / "plugin/bertQKVToContextPlugin/fused_multihead_attention").glob("*kernel.sm100.cpp"))
    return srcs


def build(force: bool = False, verbose: bool = False) -> Path | None:
    if not (REF / "plugin").is_dir():
        if verbose:
            print(f"reference tree not found at {REF}: keeping {LIB}" if LIB.exists() else f"reference tree not found at {REF}")
        return LIB if LIB.exists() else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OUT.mkdir(exist_ok=True)
    flags = ["-std=c++17", "-gencode", "arch=compute_100,code=sm_100", "--expt-relaxed-constexpr", "-O2", "-DENABLE_SM100",
             "-Xcompiler", "-fPIC,-fvisibility=hidden,-w", "-w", f"-I{REF / 'include'}", f"-I{REF / 'plugin'}",
             f"-I{REF / 'plugin' / 'common'}", f"-I{REF}"]
    srcs = _sources() + [HERE / "ref_shim.cu"]

    def compile_one(src: Path) -> Path:
        obj = OUT / (src.name.replace(".", "_") + ".o")
        if not force and obj.exists() and obj.stat().st_mtime >= src.stat().st_mtime:
            return obj
        r = subprocess.run([nvcc, *flags, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        r = subprocess.run([nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart", "-ldl"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(f"built {LIB}")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
