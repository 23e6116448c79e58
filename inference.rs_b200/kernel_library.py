"""Finds and loads ``libinferencequant_b200.so`` and declares its C ABI for ctypes.

Mirrors how the reference resolves its kernel libraries (crates/inference-tensor/src/kernel_library.rs:176-193):
``$INFERENCE_KERNEL_DIR/sm100a/`` first, then the package's own ``lib/sm100a/``. A missing library or symbol is an
error, never a fallback.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libinferencequant_b200.so"
ARCH_DIR = "sm100a"


class KernelLibraryError(RuntimeError):
    """`status` carries the library's return code where one caused the error (< 0: a B200Q_ERR_* code, > 0: a cudaError_t)."""

    status: int | None = None


_vp, _i32, _i64 = C.c_void_p, C.c_int, C.c_int64

_PLAIN_ARGS = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp]
_QUANT_ARGS = [_vp, _vp, _i32, _i32, _i32, _vp]
_MMQ_QUANT_ARGS = [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp]

# symbol -> (argtypes, restype); every name include/inferencequant_b200.h declares
SYMBOLS: dict[str, tuple[list, object]] = {}
for _e in ("bf16", "f16", "f32"):
    SYMBOLS[f"launch_mmvq_gguf_quantize_q8_1_{_e}"] = (_QUANT_ARGS, None)
    for _t in ("q8_0", "q4_k", "q6_k"):
        SYMBOLS[f"launch_mmvq_gguf_{_t}_{_e}_plain"] = (_PLAIN_ARGS, None)
for _e in ("bf16", "f16", "f32"):
    SYMBOLS[f"launch_mmvq_tc_quantize_{_e}"] = ([_vp, _vp, _i32, _i32, _vp], None)
    for _t in ("q4_k", "q6_k"):
        SYMBOLS[f"launch_mmvq_tc_gguf_{_t}_{_e}_plain"] = ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp], None)
for _e in ("bf16", "f32"):
    SYMBOLS[f"launch_mmvq_gguf_q8_0_{_e}_exact"] = ([_vp, _vp, _vp, _i32, _i32, _i32, _vp], None)
for _e in ("bf16", "f16", "f32"):
    for _t in ("q8_0", "q4_k", "q6_k"):
        SYMBOLS[f"launch_mmvq_gguf_{_t}_{_e}_fused_glu"] = ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp], None)
        SYMBOLS[f"launch_mmvq_gguf_{_t}_{_e}_fused_qkv"] = ([_vp] * 7 + [_i32] * 6 + [_vp], None)
for _l in ("D4", "DS4"):
    SYMBOLS[f"launch_mmq_quantize_q8_1_{_l}"] = (_MMQ_QUANT_ARGS, None)
for _l in ("D4", "DS4"):
    SYMBOLS[f"launch_mmq_quantize_glu_q8_1_{_l}"] = ([_vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _i32, _vp], None)
    SYMBOLS[f"launch_mmq_quantize_glu_q8_1_{_l}_f32"] = ([_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp], None)
for _t in ("q8_0", "q4_k", "q6_k"):
    SYMBOLS[f"launch_mmq_gguf_{_t}"] = ([_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _i32, _i32, _vp], None)
SYMBOLS.update({
    "b200q_version": ([], C.c_char_p),
    "b200q_last_error": ([], C.c_char_p),
    "b200q_set_option": ([C.c_char_p, _i32], _i32),
    "b200q_get_option": ([C.c_char_p, C.POINTER(_i32)], _i32),
    "b200q_device_status": ([C.POINTER(C.c_uint * 4)], _i32),
    "b200q_reset_device_status": ([], _i32),
    "b200q_take_launch_status": ([], _i32),
    "b200q_set_trace_buffer": ([_vp, _i32], _i32),
    "b200q_gemv": ([_i32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp], _i32),
    "b200q_gemm": ([_i32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp], _i32),
    "b200q_gemv_tc": ([_i32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _vp], _i32),
    "b200q_gemv_tc_workspace_bytes": ([_i32, _i32], _i64),
    "b200q_peer_allreduce_buffer_bytes": ([_i64], _i64),
    "b200q_peer_allreduce": ([_vp, _i32, _i32, _i64, _i32, _vp, _vp, _i64, _vp], _i32),
    "b200q_gemv_allreduce": ([_i32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _i32, _i32, _i64, _vp], _i32),
    "b200q_gemv_group": ([_i32, C.POINTER(_i32), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i32), _i32, _i32, _vp, _vp], _i32),
    "b200q_gemv_group_act": ([_i32, C.POINTER(_i32), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i32), _i32, _i32, _vp, _i32, _vp], _i32),
    "b200q_gemv_static_scratch": ([_i32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp], _i32),
    "b200q_gemv_plan": ([_i32, _i32, _i32, _i32, C.POINTER(_i32 * 10)], _i32),
    "b200q_set_weight_successor": ([_vp, _vp, _i32, _i32, _i32], _i32),
    "b200q_quantize": ([_i32, _vp, _vp, _i64, _vp], _i32),
    "b200q_dequantize": ([_i32, _i32, _vp, _vp, _i64, _i32, _vp], _i32),
    "b200q_get_rows": ([_i32, _i32, _vp, _vp, _vp, _i64, _i32, _i64, _vp], _i32),
    "b200q_clear_weight_successors": ([], _i32),
})
DATA_SYMBOLS = ["inference_kernel_build_id"]

_lib = None


def search_paths() -> list[str]:
    out = []
    env = os.environ.get("INFERENCE_KERNEL_DIR")
    if env:
        out.append(os.path.join(env, ARCH_DIR, LIB_NAME))
    out.append(os.path.join(HERE, "lib", ARCH_DIR, LIB_NAME))
    return out


def library_path() -> str:
    for p in search_paths():
        if os.path.exists(p):
            return p
    raise KernelLibraryError(
        f"{LIB_NAME} not found (looked in {search_paths()}); build it with `python inference.rs_b200/build.py`. "
        "There is no CPU fallback.")


def library() -> C.CDLL:
    """The loaded library with argtypes set; raises KernelLibraryError if it or any declared symbol is missing."""
    global _lib
    if _lib is None:
        lib = C.CDLL(library_path())
        missing = []
        for name, (argtypes, restype) in SYMBOLS.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                missing.append(name)
                continue
            fn.argtypes = argtypes
            fn.restype = restype
        for name in DATA_SYMBOLS:
            try:
                C.c_char.in_dll(lib, name)
            except ValueError:
                missing.append(name)
        if missing:
            raise KernelLibraryError(f"{library_path()} lacks symbols: {missing}")
        _lib = lib
    return _lib


def build_id() -> str:
    lib = library()
    return C.string_at(C.addressof(C.c_char.in_dll(lib, "inference_kernel_build_id"))).decode()


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = library().b200q_last_error().decode()
        err = KernelLibraryError(f"{what or 'b200q call'} failed with status {rc}: {msg}")
        err.status = rc
        raise err


def device_status() -> tuple[int, int, int, int]:
    buf = (C.c_uint * 4)()
    check(library().b200q_device_status(C.byref(buf)), "b200q_device_status")
    return tuple(int(v) for v in buf)
