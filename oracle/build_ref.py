"""Compile the reference's own CUDA kernels for this path into ``oracle/_ref/libinferencequant_ref.so``.

Test infrastructure and second baseline, never the product. The reference's host side is Rust and cannot be built
here, but its GGUF kernel sources are plain CUDA C++ that include only in-tree headers
(crates/inference-quant/kernels/cuda/mmq_gguf/mmq_common.cuh:1-2 calls itself self-contained), so the instances
for Q8_0 / Q4_K / Q6_K and the activation quantizers compile with nvcc alone. They are compiled where they lie in the
reference checkout, with the flags of the reference's build script (crates/inference-quant/build.rs:73-84) and
``sm_100a`` as the architecture; nothing is copied. The result exports the reference's ``extern "C"`` launchers
(crates/inference-quant/src/gguf/ffi.rs:602-700,835-1125): the generic dp4a / mma.sync kernels the reference would run
on a B200. The checkout is only present on the build machine; elsewhere the prebuilt library is used as it is.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libinferencequant_ref.so")

KERNEL_DIR = "crates/inference-quant/kernels/cuda"
SOURCES = [
    "mmvq_gguf/mmvq_quantize.cu",            # Q8_1 and tensor-core-tier activation quantizers
    "mmvq_gguf/mmvq_instance_q4_k.cu",       # decode matvec: plain, fused_glu, fused_qkv, tensor-core tier
    "mmvq_gguf/mmvq_instance_q6_k.cu",
    "mmvq_gguf/mmvq_instance_q8_0.cu",       # + the matvec against unquantized activations
    "mmq_gguf/mmq_quantize.cu",              # prefill activation quantizers
    "mmq_gguf/mmq_instance_q4_k.cu",         # prefill tile GEMM
    "mmq_gguf/mmq_instance_q6_k.cu",
    "mmq_gguf/mmq_instance_q8_0.cu",
    "gguf_quantize/k_quantize_instance_ggufq.cu",  # device Q6_K / Q8_0 weight quantizers
]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math",
    "-Xcompiler", "-fPIC",
]


def reference_root() -> str | None:
    for cand in (os.environ.get("INFERENCE_RS_REFERENCE"), "/root/reference"):
        if cand and os.path.isdir(os.path.join(cand, KERNEL_DIR)):
            return cand
    return None


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def build(force: bool = False) -> str | None:
    """Build the library when the reference checkout is present and the library is missing (or ``force``); return its
    path, or None when there is neither a checkout nor a prebuilt library."""
    root = reference_root()
    if root is None:
        return LIB if os.path.exists(LIB) else None
    srcs = [os.path.join(root, KERNEL_DIR, s) for s in SOURCES]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    nvcc = _nvcc()
    os.makedirs(OUT_DIR, exist_ok=True)

    def compile_one(src: str) -> str:
        obj = os.path.join(OUT_DIR, os.path.splitext(os.path.basename(src))[0] + ".o")
        res = subprocess.run([nvcc, *FLAGS, "-c", src, "-o", obj], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        objs = list(pool.map(compile_one, srcs))
    res = subprocess.run([nvcc, "-shared", "-o", LIB + ".tmp", *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                         capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(LIB + ".tmp", LIB)
    for o in objs:
        os.remove(o)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
