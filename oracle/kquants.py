"""numpy front end of the CPU oracle (``kquants_oracle.c``): test infrastructure only.

Every function here wraps one C function of the oracle; the C source names the reference file and
lines each one restates. Arrays are numpy; packed blocks are ``uint8`` arrays in the GGUF layout.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

Q8_0, Q4_K, Q6_K = 8, 12, 14  # GGUF type ids
LLAMACPP, IKLLAMA = 0, 1
TYPE_NAMES = {Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k"}
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        L = C.CDLL(_build.build())
        i64, i32, vp = C.c_int64, C.c_int, C.c_void_p
        L.orc_quantize.argtypes = [i32, vp, vp, i64, i64, i32]
        L.orc_quantize.restype = i32
        L.orc_dequantize.argtypes = [i32, vp, vp, i64]
        L.orc_dequantize.restype = i32
        L.orc_quantize_q6_k.argtypes = [vp, vp, i64, vp, i64, i32]
        L.orc_quantize_q6_k.restype = None
        L.orc_quantize_q8_1_cpu.argtypes = [vp, vp, i64]
        L.orc_quantize_q8_1_mmvq.argtypes = [vp, vp, i64, i64, i64]
        L.orc_quantize_q8_1_mmq.argtypes = [vp, vp, i64, i64, i64, i32]
        L.orc_quantize_mmvq_tc.argtypes = [vp, vp, i64, i64]
        L.orc_quantize_q8_k.argtypes = [vp, vp, i64]
        L.orc_matmul.argtypes = [i32, i64, i64, i64, vp, vp, vp, i32]
        L.orc_matmul.restype = i32
        L.orc_matmul_q8_1.argtypes = [i32, i64, i64, i64, i64, vp, vp, vp, i32]
        L.orc_matmul_q8_1.restype = i32
        L.orc_matmul_dense.argtypes = [i32, i64, i64, i64, vp, vp, vp, i32]
        L.orc_matmul_dense.restype = i32
        L.orc_fnv1a64.argtypes = [vp, i64]
        L.orc_fnv1a64.restype = C.c_uint64
        L.orc_max_threads.restype = i32
        for name in ("orc_widen_bf16", "orc_narrow_bf16", "orc_widen_f16", "orc_narrow_f16"):
            getattr(L, name).argtypes = [vp, vp, i64]
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f16_to_f32.restype = C.c_float
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def weight_bytes(type_id: int, rows: int, k: int) -> int:
    return rows * (k // BLOCK_ELEMS[type_id]) * BLOCK_BYTES[type_id]


def quantize(type_id: int, w, mode: int = LLAMACPP) -> np.ndarray:
    """Pack f32 ``w[rows, k]`` to ``type_id`` blocks: uint8 ``[rows, k/block*block_bytes]``."""
    w = _f32(w)
    rows, k = w.shape
    if k % BLOCK_ELEMS[type_id]:
        raise ValueError(f"k={k} is not a multiple of the {TYPE_NAMES[type_id]} block")
    out = np.zeros((rows, weight_bytes(type_id, 1, k)), dtype=np.uint8)
    rc = lib().orc_quantize(type_id, _p(w), _p(out), rows, k, mode)
    if rc:
        raise ValueError(f"orc_quantize failed: {rc}")
    return out


def quantize_q6_k_imatrix(w, imatrix, mode: int = LLAMACPP) -> np.ndarray:
    w = _f32(w)
    rows, k = w.shape
    im = _f32(imatrix)
    assert im.size == k
    out = np.zeros((rows, weight_bytes(Q6_K, 1, k)), dtype=np.uint8)
    lib().orc_quantize_q6_k(_p(w), _p(out), rows * k, _p(im), k, mode)
    return out


def dequantize(type_id: int, packed: np.ndarray, k: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    rows = packed.size // weight_bytes(type_id, 1, k)
    out = np.empty((rows, k), dtype=np.float32)
    rc = lib().orc_dequantize(type_id, _p(packed), _p(out), rows * k)
    if rc:
        raise ValueError("orc_dequantize failed")
    return out


def quantize_q8_1_cpu(x) -> np.ndarray:
    x = _f32(x)
    out = np.zeros(x.size // 32 * 36, dtype=np.uint8)
    lib().orc_quantize_q8_1_cpu(_p(x), _p(out), x.size)
    return out


def quantize_q8_1_mmvq(x, k_padded: int | None = None) -> np.ndarray:
    """The decode path's Q8_1 activations: uint8 ``[rows, k_padded/32*36]``."""
    x = _f32(x)
    rows, k = x.shape
    if k_padded is None:
        k_padded = (k + 511) // 512 * 512
    out = np.zeros((rows, k_padded // 32 * 36), dtype=np.uint8)
    lib().orc_quantize_q8_1_mmvq(_p(x), _p(out), k, k_padded, rows)
    return out


def quantize_mmvq_tc(x) -> np.ndarray:
    """The tensor-core matvec tier's activation layout: uint8 ``[ceil(rows / 8) * ceil(k / 32) * 288]``."""
    x = _f32(x)
    rows, k = x.shape
    out = np.zeros(((rows + 7) // 8) * ((k + 31) // 32) * 288, dtype=np.uint8)
    lib().orc_quantize_mmvq_tc(_p(x), _p(out), k, rows)
    return out


def quantize_q8_1_mmq(x, k_padded: int, layout: int) -> np.ndarray:
    """The prefill path's activations: uint8 ``[k_padded/128, rows, 144]``; layout 0 = D4, 1 = DS4."""
    x = _f32(x)
    rows, k = x.shape
    out = np.zeros((k_padded // 128, rows, 144), dtype=np.uint8)
    lib().orc_quantize_q8_1_mmq(_p(x), _p(out), k, k_padded, rows, layout)
    return out


def quantize_q8_k(x) -> np.ndarray:
    x = _f32(x)
    out = np.zeros(x.size // 256 * 292, dtype=np.uint8)
    lib().orc_quantize_q8_k(_p(x), _p(out), x.size)
    return out


def matmul(type_id: int, x, packed: np.ndarray, n: int, threads: int = 0) -> np.ndarray:
    """The reference CPU path: ``x[m,k] . W[n,k]^T`` with Q8_K / Q8_0 activations; f32 ``[m, n]``."""
    x = _f32(x)
    m, k = x.shape
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    assert packed.size == weight_bytes(type_id, n, k), (packed.size, weight_bytes(type_id, n, k))
    out = np.empty((m, n), dtype=np.float32)
    rc = lib().orc_matmul(type_id, m, k, n, _p(x), _p(packed), _p(out), threads)
    if rc:
        raise ValueError(f"orc_matmul failed: {rc}")
    return out


def matmul_q8_1(type_id: int, acts: np.ndarray, m: int, k: int, k_padded: int, packed: np.ndarray, n: int,
                threads: int = 0) -> np.ndarray:
    """The decode kernels' arithmetic on given Q8_1 blocks, accumulated in double; f64 ``[m, n]``."""
    acts = np.ascontiguousarray(acts, dtype=np.uint8)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    assert acts.size == m * (k_padded // 32) * 36
    out = np.empty((m, n), dtype=np.float64)
    rc = lib().orc_matmul_q8_1(type_id, m, k, k_padded, n, _p(acts), _p(packed), _p(out), threads)
    if rc:
        raise ValueError(f"orc_matmul_q8_1 failed: {rc}")
    return out


def matmul_dense(type_id: int, x, packed: np.ndarray, n: int, threads: int = 0) -> np.ndarray:
    """``x . dequant(W)^T`` in double; f64 ``[m, n]``."""
    x = _f32(x)
    m, k = x.shape
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty((m, n), dtype=np.float64)
    rc = lib().orc_matmul_dense(type_id, m, k, n, _p(x), _p(packed), _p(out), threads)
    if rc:
        raise ValueError(f"orc_matmul_dense failed: {rc}")
    return out


def fnv1a64(data: np.ndarray) -> int:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    return int(lib().orc_fnv1a64(_p(data), data.size))


def widen_bf16(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().orc_widen_bf16(_p(bits), _p(out), bits.size)
    return out


def narrow_bf16(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_narrow_bf16(_p(x), _p(out), x.size)
    return out


def widen_f16(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().orc_widen_f16(_p(bits), _p(out), bits.size)
    return out


def narrow_f16(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_narrow_f16(_p(x), _p(out), x.size)
    return out


def pinned_layer(rows: int = 8, cols: int = 512):
    """The reference's known-answer layer (crates/inference-quant/src/gguf/requantize.rs:1076-1093):
    an LCG (seed 12345) giving small values with sparse outliers, then a skewed importance matrix."""
    state = 12345
    vals = np.empty(rows * cols, dtype=np.float32)
    two24 = np.float32(1 << 24)

    def nxt():
        nonlocal state
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        return np.float32(np.float32(state >> 8) / two24), state

    for i in range(rows * cols):
        u, s = nxt()
        scale = np.float32(0.4) if ((s >> 4) & 31) == 0 else np.float32(0.04)
        vals[i] = np.float32(np.float32(u - np.float32(0.5)) * scale)
    imat = np.empty(cols, dtype=np.float32)
    for i in range(cols):
        u, _ = nxt()
        u3 = np.float32(np.float32(u * u) * u)  # f32::powi(3)
        imat[i] = np.float32(np.float32(0.05) + np.float32(np.float32(4.0) * u3))
    return vals.reshape(rows, cols), imat
