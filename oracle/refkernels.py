"""ctypes front end of ``oracle/_ref/libinferencequant_ref.so``: the reference's own CUDA kernels for this path,
compiled from the reference checkout by ``oracle/build_ref.py``. Test infrastructure and second baseline only.

Every wrapper calls one ``extern "C"`` launcher of the reference exactly as its Rust host does
(crates/inference-quant/src/gguf/fast_mmvq.rs:477-665,2049-2126 and fast_mmq.rs:420-520), on torch CUDA tensors and the
current torch stream, with the scratch sizes the host allocates. ``available()`` is False where the library was not
built (no reference checkout and no prebuilt file).
"""
from __future__ import annotations

import ctypes as C
import os

from . import build_ref as _build_ref

Q8_0, Q4_K, Q6_K = 8, 12, 14
NAMES = {Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k"}
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}
# scale layout of the 144-byte prefill activation blocks per weight type (fast_mmq.rs:167-190)
MMQ_LAYOUT = {Q8_0: "D4", Q4_K: "DS4", Q6_K: "D4"}
GLU_ACTIVATIONS = {"silu": 0, "gelu": 1, "relu": 2, "gelu_erf": 3, "sigmoid": 4}  # kernels/cuda/glu_activation.cuh:4-10

_lib = None
_tried = False

_vp, _i32, _i64 = C.c_void_p, C.c_int, C.c_int64


def available() -> bool:
    return lib() is not None


def lib():
    global _lib, _tried
    if not _tried:
        _tried = True
        path = _build_ref.LIB if os.path.exists(_build_ref.LIB) else None
        if path is None and _build_ref.reference_root() is not None:
            path = _build_ref.build()
        if path is not None:
            L = C.CDLL(path)
            for e in ("bf16", "f16", "f32"):
                getattr(L, f"launch_mmvq_gguf_quantize_q8_1_{e}").argtypes = [_vp, _vp, _i32, _i32, _i32, _vp]
                getattr(L, f"launch_mmvq_tc_quantize_{e}").argtypes = [_vp, _vp, _i32, _i32, _vp]
                for t in NAMES.values():
                    getattr(L, f"launch_mmvq_gguf_{t}_{e}_plain").argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp]
                    getattr(L, f"launch_mmvq_gguf_{t}_{e}_fused_glu").argtypes = [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]
                    getattr(L, f"launch_mmvq_gguf_{t}_{e}_fused_qkv").argtypes = [_vp] * 7 + [_i32] * 6 + [_vp]
                for t in ("q4_k", "q6_k"):
                    getattr(L, f"launch_mmvq_tc_gguf_{t}_{e}_plain").argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp]
            for e in ("bf16", "f32"):
                getattr(L, f"launch_mmvq_gguf_q8_0_{e}_exact").argtypes = [_vp, _vp, _vp, _i32, _i32, _i32, _vp]
            for lay in ("D4", "DS4"):
                getattr(L, f"launch_mmq_quantize_q8_1_{lay}").argtypes = [_vp, _vp, _vp, _i32] + [_i64] * 8 + [_vp]
            for t in NAMES.values():
                getattr(L, f"launch_mmq_gguf_{t}").argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _i32, _i32, _vp]
            L.launch_q6_k_encode.argtypes = [_vp, _vp, _i64, _i64, _i32, _vp, _vp, _vp, _vp, _vp]
            L.launch_q6_k_encode.restype = _i32
            L.launch_q8_0_encode.argtypes = [_vp, _i64, _i32, _vp, _vp, _vp]
            L.launch_q8_0_encode.restype = _i32
            _lib = L
    return _lib


def _elem(dtype) -> str:
    import torch
    return {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dtype]


def _type_x(dtype) -> int:
    import torch
    return {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}[dtype]


def _stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def pad(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def quantize_q8_1(x, k_padded: int | None = None):
    """x [b, k] -> Q8_1 blocks [b, k_padded / 32, 36] (launch_mmvq_gguf_quantize_q8_1_*; k padded to 512 as
    fast_mmvq.rs:535-538 does)."""
    import torch
    b, k = x.shape
    kp = k_padded or pad(k, 512)
    vy = torch.empty(b, kp // 32, 36, dtype=torch.uint8, device=x.device)
    getattr(lib(), f"launch_mmvq_gguf_quantize_q8_1_{_elem(x.dtype)}")(x.data_ptr(), vy.data_ptr(), k, kp, b, _stream())
    return vy


def mmvq_plain(type_id: int, w, vy, n: int, k: int, b: int, dtype):
    """The dp4a decode matvec on Q8_1 blocks, b = 1..8 (launch_mmvq_gguf_<type>_<elem>_plain)."""
    import torch
    out = torch.empty(b, n, dtype=dtype, device=w.device)
    stride_blocks = vy.numel() // 36 // vy.shape[0]  # Q8_1 blocks per activation row, whatever the tensor's shape
    getattr(lib(), f"launch_mmvq_gguf_{NAMES[type_id]}_{_elem(dtype)}_plain")(
        w.data_ptr(), vy.data_ptr(), out.data_ptr(), k, n, stride_blocks, n, b, _stream())
    return out


def mmvq(type_id: int, w, x, n: int):
    """quantize + plain matvec, as fast_mmvq::plain runs them."""
    return mmvq_plain(type_id, w, quantize_q8_1(x), n, x.shape[1], x.shape[0], x.dtype)


def fused_glu(type_id: int, w_gate, w_up, x, n: int, activation: str = "silu", vy=None):
    """act(x . gate^T) * (x . up^T) in one launch (launch_mmvq_gguf_<type>_<elem>_fused_glu), b = 1..8; on the Q8_1
    blocks `vy` of x where given, else on the reference quantizer's."""
    import torch
    b, k = x.shape
    vy = quantize_q8_1(x) if vy is None else vy
    out = torch.empty(b, n, dtype=x.dtype, device=x.device)
    getattr(lib(), f"launch_mmvq_gguf_{NAMES[type_id]}_{_elem(x.dtype)}_fused_glu")(
        w_gate.data_ptr(), w_up.data_ptr(), vy.data_ptr(), out.data_ptr(), k, n, vy.numel() // 36 // b, n, b,
        GLU_ACTIVATIONS[activation], _stream())
    return out


def fused_qkv(type_id: int, wq, wk, wv, x, nq: int, nk: int, nv: int, vy=None):
    """q, k, v projections of one input in one launch (launch_mmvq_gguf_<type>_<elem>_fused_qkv), b = 1..8; on the Q8_1
    blocks `vy` of x where given, else on the reference quantizer's."""
    import torch
    b, k = x.shape
    vy = quantize_q8_1(x) if vy is None else vy
    outs = [torch.empty(b, n, dtype=x.dtype, device=x.device) for n in (nq, nk, nv)]
    getattr(lib(), f"launch_mmvq_gguf_{NAMES[type_id]}_{_elem(x.dtype)}_fused_qkv")(
        wq.data_ptr(), wk.data_ptr(), wv.data_ptr(), vy.data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(),
        k, nq, nk, nv, vy.numel() // 36 // b, b, _stream())
    return outs


def tc_scratch_bytes(k: int, b: int) -> int:
    """fast_mmvq.rs:1898-1902: 288 bytes per 32-value block and 8-row half."""
    return (k // 32) * 288 * ((b + 7) // 8)


def tc_quantize(x):
    import torch
    b, k = x.shape
    vy = torch.empty(tc_scratch_bytes(k, b), dtype=torch.uint8, device=x.device)
    getattr(lib(), f"launch_mmvq_tc_quantize_{_elem(x.dtype)}")(x.data_ptr(), vy.data_ptr(), k, b, _stream())
    return vy


def tc_plain(type_id: int, w, vy, n: int, k: int, b: int, dtype, cfg: int = 1):
    """The int8 mma.sync matvec for 1..16 rows (launch_mmvq_tc_gguf_{q4_k,q6_k}_<elem>_plain)."""
    import torch
    out = torch.empty(b, n, dtype=dtype, device=w.device)
    getattr(lib(), f"launch_mmvq_tc_gguf_{NAMES[type_id]}_{_elem(dtype)}_plain")(
        w.data_ptr(), vy.data_ptr(), out.data_ptr(), k, n, n, b, cfg, _stream())
    return out


def exact_q8_0(w, x, n: int):
    """Q8_0 weights against unquantized activations, f32 accumulation (launch_mmvq_gguf_q8_0_{bf16,f32}_exact)."""
    import torch
    b, k = x.shape
    out = torch.empty(b, n, dtype=x.dtype, device=x.device)
    getattr(lib(), f"launch_mmvq_gguf_q8_0_{_elem(x.dtype)}_exact")(w.data_ptr(), x.data_ptr(), out.data_ptr(), k, n, b, _stream())
    return out


def mmq_k_padded(k: int) -> int:
    return pad(pad(k, 512), 128)


def mmq_quantize(x, layout: str):
    """x [m, k] -> 144-byte blocks, block index (k / 128) * m + row, plus the host's 128 spare blocks
    (fast_mmq.rs:686-692)."""
    import torch
    m, k = x.shape
    kp = mmq_k_padded(k)
    vy = torch.zeros(m * (kp // 128) * 144 + 128 * 144, dtype=torch.uint8, device=x.device)
    getattr(lib(), f"launch_mmq_quantize_q8_1_{layout}")(x.data_ptr(), None, vy.data_ptr(), _type_x(x.dtype), k, k, 0, 0, kp, m, 1, 1,
                                                         _stream())
    return vy


_fixup = {}


def mmq(type_id: int, w, vy, m: int, n: int, k: int, dtype):
    """The prefill tile GEMM on quantized activations (launch_mmq_gguf_<type>), called as fast_mmq.rs:489-512 calls it."""
    import torch
    dev = w.device
    props = torch.cuda.get_device_properties(dev)
    nsm = props.multi_processor_count
    key = (dev.index, nsm)
    if key not in _fixup:
        _fixup[key] = torch.empty(nsm * 128 * 128 * 4, dtype=torch.uint8, device=dev)
    out = torch.empty(m, n, dtype=dtype, device=dev)
    smpbo = getattr(props, "shared_memory_per_block_optin", 232448)
    cc = (props.major * 10 + props.minor) * 10
    getattr(lib(), f"launch_mmq_gguf_{NAMES[type_id]}")(
        _fixup[key].data_ptr(), w.data_ptr(), vy.data_ptr(), out.data_ptr(), k, n, m, k // BLOCK_ELEMS[type_id], n, cc, nsm, smpbo, 32,
        _type_x(dtype), _stream())
    return out


def mmq_forward(type_id: int, w, x, n: int):
    """quantize + tile GEMM, as fast_mmq::plain runs them."""
    return mmq(type_id, w, mmq_quantize(x, MMQ_LAYOUT[type_id]), x.shape[0], n, x.shape[1], x.dtype)


def encode_q6_k(x):
    """f32 [rows, cols] on the device -> Q6_K bytes [rows, cols / 256 * 210] by the reference's device quantizer
    (launch_q6_k_encode; byte-exact with its CPU quantizer by its own tests)."""
    import torch
    rows, cols = x.shape
    ls = torch.empty(rows * cols, dtype=torch.int8, device=x.device)
    scales = torch.empty(rows * cols // 16, dtype=torch.float32, device=x.device)
    out = torch.empty(rows, cols // 256 * 210, dtype=torch.uint8, device=x.device)
    dec = torch.empty(rows, cols, dtype=torch.float32, device=x.device)
    rc = lib().launch_q6_k_encode(x.data_ptr(), None, rows, 1, cols, ls.data_ptr(), scales.data_ptr(), out.data_ptr(), dec.data_ptr(),
                                  _stream())
    if rc != 0:
        raise RuntimeError(f"launch_q6_k_encode: CUDA error {rc}")
    return out, dec


def encode_q8_0(x):
    import torch
    rows, cols = x.shape
    out = torch.empty(rows, cols // 32 * 34, dtype=torch.uint8, device=x.device)
    dec = torch.empty(rows, cols, dtype=torch.float32, device=x.device)
    rc = lib().launch_q8_0_encode(x.data_ptr(), rows, cols, out.data_ptr(), dec.data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"launch_q8_0_encode: CUDA error {rc}")
    return out, dec
