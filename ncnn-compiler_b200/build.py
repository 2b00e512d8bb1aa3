"""Builds libncnn_b200.so in-tree: nvcc for sm_100a only, static CUDA runtime."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libncnn_b200.so")
SOURCES = ["engine.cu", "engine_import.cu", "engine_plan.cu", "engine_emit.cu", "tc_gemm.cu", "c_api.cu", "no_alloc.cu", "loader.cpp", "dynamic.cpp", "multi.cpp"]
HEADERS = ["exports.map", "engine.h", "engine_impl.h", "tc_gemm.h", "tc_gemm.cuh", "tc_gemm2.cuh", "tc_stem.cuh", "tc_stem_pool.cuh", "tc_conv_halo.cuh", "tc_dw_project.cuh", "ptx_sm100.cuh", "kernels.cuh", "ip_rows.cuh", "loader.h",
           os.path.join("..", "..", "include", "ncnn_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > built for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        build_compile_tool()
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objects = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
        objects.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(out)
    # only the C ABI is exported, as the reference restricts its library to the entry symbols
    subprocess.check_call([nvcc, "-shared", "-o", LIB, *objects, "-Xlinker", "--no-undefined", "-Xlinker",
                           "--version-script=" + os.path.join(CSRC, "exports.map")])
    build_compile_tool()
    return LIB


def build_compile_tool() -> str:
    """ncnn-b200-compile: the sm_100a target of the reference's ncnn-compile (host tool, g++)."""
    tool = os.path.join(HERE, "ncnn-b200-compile")
    src = os.path.join(CSRC, "ncnn_b200_compile.cpp")
    if not os.path.exists(tool) or os.path.getmtime(tool) < max(os.path.getmtime(src), os.path.getmtime(LIB)):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-o", tool, src, "-L" + HERE, "-lncnn_b200",
                               "-Wl,-rpath," + HERE])
    return tool


if __name__ == "__main__":
    print(build(force=True, verbose=True))
