"""Compiles the CUDA sources under ``csrc/`` for sm_100a into ``lib/sm100a/libinferencequant_b200.so``.

The directory name follows the reference's kernel-library convention: one directory per architecture,
``sm100a`` for compute capability 10.0 (crates/inference-tensor/src/kernel_library.rs:152-172), so the
folder can be given to a host as its ``INFERENCE_KERNEL_DIR``.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib", "sm100a")
LIB = os.path.join(OUT_DIR, "libinferencequant_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


# diagnostics builds: B200Q_BUILD_DEFINES="-DB200Q_GEMV_TRACE=1" adds the decode GEMV's timestamp sites (part of the digest)
NVCC_FLAGS += os.environ.get("B200Q_BUILD_DEFINES", "").split()

# per-file additions: the weight quantizers repeat the reference's scale searches operation for operation, which rules out
# contracting a multiply and an add into one fused operation
EXTRA_FLAGS = {"quantize_weights.cu": ["-fmad=false"]}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(repr(sorted(EXTRA_FLAGS.items())).encode())
    return h.hexdigest()


def _stamp(src: str, hdr: str) -> str:
    with open(src, "rb") as fh:
        return hashlib.sha256(fh.read() + hdr.encode()).hexdigest()


def _compile(nvcc: str, src: str, obj: str, extra: list[str]) -> tuple[str, str]:
    cmd = [nvcc, *NVCC_FLAGS, *EXTRA_FLAGS.get(os.path.basename(src), []), *extra, "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return src, res.stdout + res.stderr


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Build the shared library if any source changed; return its path."""
    hdr = _headers_digest()
    # one digest over every source: a library built from these exact sources is reused even where the object
    # directory did not travel with it
    total = hashlib.sha256(hdr.encode())
    for src in _sources():
        total.update(_stamp(src, hdr).encode())
    digest_file = LIB + ".digest"
    if (not force and not ptxas_info and os.path.exists(LIB) and os.path.exists(digest_file)
            and open(digest_file).read() == total.hexdigest()):
        return LIB
    nvcc = _nvcc()
    os.makedirs(OUT_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    jobs, objs = [], []
    for src in _sources():
        base = os.path.splitext(os.path.basename(src))[0]
        obj = os.path.join(OBJ_DIR, base + ".o")
        stamp_file = obj + ".stamp"
        stamp = _stamp(src, hdr)
        objs.append(obj)
        fresh = (not force and not ptxas_info and os.path.exists(obj) and os.path.exists(stamp_file)
                 and open(stamp_file).read() == stamp)
        if not fresh:
            jobs.append((src, obj, stamp_file, stamp))
    logs = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as pool:
            futs = {pool.submit(_compile, nvcc, src, obj, extra): (obj, sf, st) for src, obj, sf, st in jobs}
            for fut in cf.as_completed(futs):
                src, log = fut.result()
                obj, sf, st = futs[fut]
                with open(sf, "w") as fh:
                    fh.write(st)
                logs.append((src, log))
                if verbose:
                    print(f"compiled {os.path.basename(src)}", file=sys.stderr)
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB + ".tmp", *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        os.replace(LIB + ".tmp", LIB)
    with open(digest_file, "w") as fh:
        fh.write(total.hexdigest())
    if ptxas_info:
        with open(os.path.join(OBJ_DIR, "ptxas_info.log"), "w") as fh:
            for src, log in sorted(logs):
                fh.write(f"==== {os.path.basename(src)}\n{log}\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas-info" in sys.argv))
