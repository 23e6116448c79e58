"""torch-tensor front end of the C ABI: device memory and streams come from torch, the arithmetic from the library.

Every function launches on torch's current CUDA stream and raises if the kernel library is unavailable.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import kernel_library as kl
from .dtypes import (ELEM_BF16, ELEM_F16, ELEM_F32, ELEM_TAG, MATRIX_ROW_PADDING, MMQ_TYPE_X, GgmlDType, pad)

_ELEM_OF = {torch.float32: ELEM_F32, torch.float16: ELEM_F16, torch.bfloat16: ELEM_BF16}


def elem_of(dtype: torch.dtype) -> int:
    try:
        return _ELEM_OF[dtype]
    except KeyError:
        raise TypeError(f"activations must be f32, f16 or bf16, not {dtype}") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("expected a CUDA tensor")
        if not t.is_contiguous():
            raise ValueError("expected a contiguous tensor")


def upload_weights(packed: np.ndarray | torch.Tensor, dtype: GgmlDType, device="cuda") -> torch.Tensor:
    """Packed GGUF blocks -> device buffer followed by 512 elements' worth of zero bytes, as the reference's
    `load_quantized` does (crates/inference-tensor/src/quantized/cuda.rs:511-530)."""
    if isinstance(packed, np.ndarray):
        arr = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    if not arr.flags.writeable:
        arr = arr.copy()  # torch tensors alias their numpy source and want it writable
    packed = torch.from_numpy(arr)
    packed = packed.reshape(-1)
    padding = MATRIX_ROW_PADDING * dtype.type_size // dtype.block_size
    buf = torch.zeros(packed.numel() + padding, dtype=torch.uint8, device=device)
    buf[: packed.numel()].copy_(packed)
    return buf


def quantize_weights(x: torch.Tensor, dtype: GgmlDType) -> torch.Tensor:
    """`b200q_quantize`: f32 [n, k] on the device -> packed blocks followed by the reference's padding (a buffer
    `upload_weights` would have produced), byte for byte the reference CPU quantizer's."""
    _require_cuda(x)
    if x.dtype != torch.float32:
        raise TypeError("weights are quantized from f32")
    n, k = x.shape
    nbytes = n * dtype.row_bytes(k)
    padding = MATRIX_ROW_PADDING * dtype.type_size // dtype.block_size
    buf = torch.zeros(nbytes + padding, dtype=torch.uint8, device=x.device)
    kl.check(kl.library().b200q_quantize(int(dtype), x.data_ptr(), buf.data_ptr(), n * k, _stream()), "b200q_quantize")
    return buf


def dequantize(dtype: GgmlDType, w: torch.Tensor, n: int, k: int, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """`b200q_dequantize`: packed [n, k] -> values [n, k] of `out_dtype`."""
    _require_cuda(w)
    out = torch.empty((n, k), dtype=out_dtype, device=w.device)
    kl.check(kl.library().b200q_dequantize(int(dtype), elem_of(out_dtype), w.data_ptr(), out.data_ptr(), n, k, _stream()), "b200q_dequantize")
    return out


def get_rows(dtype: GgmlDType, w: torch.Tensor, ids: torch.Tensor, n: int, k: int, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """`b200q_get_rows`: rows `ids` (int32, any shape) of a packed [n, k] table -> [*ids.shape, k] of `out_dtype`."""
    _require_cuda(w)
    flat = ids.reshape(-1).to(device=w.device, dtype=torch.int32).contiguous()
    out = torch.empty((flat.numel(), k), dtype=out_dtype, device=w.device)
    kl.check(kl.library().b200q_get_rows(int(dtype), elem_of(out_dtype), w.data_ptr(), flat.data_ptr(), out.data_ptr(), flat.numel(), k, n,
                                         _stream()), "b200q_get_rows")
    return out.reshape(*ids.shape, k)


def quantize_q8_1(x: torch.Tensor, k_padded: int | None = None) -> torch.Tensor:
    """`launch_mmvq_gguf_quantize_q8_1_<dtype>`: x [rows, k] -> uint8 [rows, k_padded / 32 * 36]."""
    _require_cuda(x)
    rows, k = x.shape
    k_padded = pad(k, MATRIX_ROW_PADDING) if k_padded is None else k_padded
    out = torch.empty((rows, k_padded // 32 * 36), dtype=torch.uint8, device=x.device)
    fn = getattr(kl.library(), f"launch_mmvq_gguf_quantize_q8_1_{ELEM_TAG[elem_of(x.dtype)]}")
    fn(x.data_ptr(), out.data_ptr(), k, k_padded, rows, _stream())
    return out


def quantize_mmq_q8_1(x: torch.Tensor, layout: str, k_padded: int | None = None) -> torch.Tensor:
    """`launch_mmq_quantize_q8_1_{D4,DS4}`: x [rows, k] -> uint8 [k_padded / 128, rows, 144]."""
    _require_cuda(x)
    rows, k = x.shape
    k_padded = pad(pad(k, MATRIX_ROW_PADDING), 128) if k_padded is None else k_padded
    out = torch.empty((k_padded // 128, rows, 144), dtype=torch.uint8, device=x.device)
    fn = getattr(kl.library(), f"launch_mmq_quantize_q8_1_{layout}")
    fn(x.data_ptr(), None, out.data_ptr(), MMQ_TYPE_X[elem_of(x.dtype)], k, k, 0, 0, k_padded, rows, 1, 1, _stream())
    return out


def quantize_mmq_q8_1_glu(gate: torch.Tensor, up: torch.Tensor, layout: str, activation: str = "silu", k_padded: int | None = None,
                          typed: bool = True) -> torch.Tensor:
    """`launch_mmq_quantize_glu_q8_1_{D4,DS4}` (or its `_f32` form when `typed` is false): act(gate) * up, [rows, k] each,
    quantized to the prefill blocks; uint8 [k_padded / 128, rows, 144]."""
    _require_cuda(gate, up)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up have the same shape and type")
    rows, k = gate.shape
    k_padded = pad(pad(k, MATRIX_ROW_PADDING), 128) if k_padded is None else k_padded
    out = torch.empty((k_padded // 128, rows, 144), dtype=torch.uint8, device=gate.device)
    act = GLU_ACTIVATIONS[activation]
    if typed:
        getattr(kl.library(), f"launch_mmq_quantize_glu_q8_1_{layout}")(gate.data_ptr(), up.data_ptr(), None, out.data_ptr(),
                                                                       MMQ_TYPE_X[elem_of(gate.dtype)], k, k, k_padded, rows, act, _stream())
    else:
        if gate.dtype != torch.float32:
            raise TypeError("the _f32 launcher takes f32 inputs")
        getattr(kl.library(), f"launch_mmq_quantize_glu_q8_1_{layout}_f32")(gate.data_ptr(), up.data_ptr(), None, out.data_ptr(), k, k,
                                                                           k_padded, rows, act, _stream())
    return out


def mmvq_plain(dtype: GgmlDType, w: torch.Tensor, vy: torch.Tensor, n: int, k: int, b: int,
               out_dtype: torch.dtype, k_padded: int | None = None) -> torch.Tensor:
    """`launch_mmvq_gguf_<type>_<out>_plain` on Q8_1 blocks `vy`; returns [b, n]."""
    _require_cuda(w, vy)
    k_padded = pad(k, MATRIX_ROW_PADDING) if k_padded is None else k_padded
    dst = torch.empty((b, n), dtype=out_dtype, device=w.device)
    fn = getattr(kl.library(), f"launch_mmvq_gguf_{dtype.tag}_{ELEM_TAG[elem_of(out_dtype)]}_plain")
    fn(w.data_ptr(), vy.data_ptr(), dst.data_ptr(), k, n, k_padded // 32, n, b, _stream())
    rc = kl.library().b200q_take_launch_status()
    if rc:
        raise kl.KernelLibraryError(f"launch_mmvq_gguf_{dtype.tag}_*_plain failed with status {rc}")
    return dst


GLU_ACTIVATIONS = {"silu": 0, "gelu": 1, "relu": 2, "gelu_erf": 3, "sigmoid": 4}  # kernels/cuda/glu_activation.cuh:4-10


def mmvq_fused_glu(dtype: GgmlDType, w_gate: torch.Tensor, w_up: torch.Tensor, vy: torch.Tensor, n: int, k: int, b: int,
                   out_dtype: torch.dtype, activation: str = "silu", k_padded: int | None = None) -> torch.Tensor:
    """`launch_mmvq_gguf_<type>_<out>_fused_glu` on Q8_1 blocks `vy`: act(y . gate^T) * (y . up^T), [b, n]
    (fast_mmvq::fused_glu, crates/inference-quant/src/gguf/fast_mmvq.rs)."""
    _require_cuda(w_gate, w_up, vy)
    k_padded = pad(k, MATRIX_ROW_PADDING) if k_padded is None else k_padded
    dst = torch.empty((b, n), dtype=out_dtype, device=vy.device)
    name = f"launch_mmvq_gguf_{dtype.tag}_{ELEM_TAG[elem_of(out_dtype)]}_fused_glu"
    getattr(kl.library(), name)(w_gate.data_ptr(), w_up.data_ptr(), vy.data_ptr(), dst.data_ptr(), k, n, k_padded // 32, n, b,
                                GLU_ACTIVATIONS[activation], _stream())
    rc = kl.library().b200q_take_launch_status()
    if rc:
        raise kl.KernelLibraryError(f"{name} failed with status {rc}")
    return dst


def mmvq_fused_qkv(dtype: GgmlDType, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, vy: torch.Tensor, nq: int, nk: int,
                   nv: int, k: int, b: int, out_dtype: torch.dtype, k_padded: int | None = None) -> list[torch.Tensor]:
    """`launch_mmvq_gguf_<type>_<out>_fused_qkv` on Q8_1 blocks `vy`: the three projections [b, nq], [b, nk], [b, nv]."""
    _require_cuda(wq, wk, wv, vy)
    k_padded = pad(k, MATRIX_ROW_PADDING) if k_padded is None else k_padded
    outs = [torch.empty((b, n), dtype=out_dtype, device=vy.device) for n in (nq, nk, nv)]
    name = f"launch_mmvq_gguf_{dtype.tag}_{ELEM_TAG[elem_of(out_dtype)]}_fused_qkv"
    getattr(kl.library(), name)(wq.data_ptr(), wk.data_ptr(), wv.data_ptr(), vy.data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(),
                                outs[2].data_ptr(), k, nq, nk, nv, k_padded // 32, b, _stream())
    rc = kl.library().b200q_take_launch_status()
    if rc:
        raise kl.KernelLibraryError(f"{name} failed with status {rc}")
    return outs


MMQ_LAYOUT = {GgmlDType.Q8_0: "D4", GgmlDType.Q4K: "DS4", GgmlDType.Q6K: "D4"}  # fast_mmq.rs:167-190


def mmq(dtype: GgmlDType, w: torch.Tensor, vy: torch.Tensor, m: int, n: int, k: int, out_dtype: torch.dtype) -> torch.Tensor:
    """`launch_mmq_gguf_<type>` on activation blocks `vy` from `quantize_mmq_q8_1(x, MMQ_LAYOUT[dtype])`; returns
    [m, n] of `out_dtype`, called as the reference's host calls it (crates/inference-quant/src/gguf/fast_mmq.rs:489-512)."""
    _require_cuda(w, vy)
    dst = torch.empty((m, n), dtype=out_dtype, device=w.device)
    props = torch.cuda.get_device_properties(w.device)
    fn = getattr(kl.library(), f"launch_mmq_gguf_{dtype.tag}")
    fn(None, w.data_ptr(), vy.data_ptr(), dst.data_ptr(), k, n, m, k // dtype.block_size, n, (props.major * 10 + props.minor) * 10,
       props.multi_processor_count, 232448, 32, MMQ_TYPE_X[elem_of(out_dtype)], _stream())
    rc = kl.library().b200q_take_launch_status()
    if rc:
        raise kl.KernelLibraryError(f"launch_mmq_gguf_{dtype.tag} failed with status {rc}")
    return dst


TC_ACT_BLOCK_BYTES = 288  # per 32-value block and 8-row half (crates/inference-quant/src/gguf/fast_mmvq.rs:94)


def mmvq_tc_quantize(x: torch.Tensor) -> torch.Tensor:
    """`launch_mmvq_tc_quantize_<dtype>`: x [rows <= 16, k] contiguous -> the tensor-core tier's activation scratch,
    uint8 [ceil(rows / 8) * ceil(k / 32) * 288] (the size the reference's host allocates, fast_mmvq.rs:1898-1902)."""
    _require_cuda(x)
    rows, k = x.shape
    out = torch.empty(((rows + 7) // 8) * ((k + 31) // 32) * TC_ACT_BLOCK_BYTES, dtype=torch.uint8, device=x.device)
    fn = getattr(kl.library(), f"launch_mmvq_tc_quantize_{ELEM_TAG[elem_of(x.dtype)]}")
    fn(x.data_ptr(), out.data_ptr(), k, rows, _stream())
    rc = kl.library().b200q_take_launch_status()
    if rc:
        raise kl.KernelLibraryError(f"launch_mmvq_tc_quantize_* failed with status {rc}")
    return out


def mmvq_tc_plain(dtype: GgmlDType, w: torch.Tensor, vy: torch.Tensor, n: int, k: int, b: int, out_dtype: torch.dtype,
                  cfg: int = 1) -> torch.Tensor:
    """`launch_mmvq_tc_gguf_{q4_k,q6_k}_<out>_plain` on the scratch `mmvq_tc_quantize` wrote; returns [b, n]."""
    _require_cuda(w, vy)
    if dtype not in (GgmlDType.Q4K, GgmlDType.Q6K):
        raise ValueError("the reference's tensor-core matvec launchers exist for Q4_K and Q6_K")
    dst = torch.empty((b, n), dtype=out_dtype, device=w.device)
    fn = getattr(kl.library(), f"launch_mmvq_tc_gguf_{dtype.tag}_{ELEM_TAG[elem_of(out_dtype)]}_plain")
    fn(w.data_ptr(), vy.data_ptr(), dst.data_ptr(), k, n, n, b, cfg, _stream())
    rc = kl.library().b200q_take_launch_status()
    if rc:
        raise kl.KernelLibraryError(f"launch_mmvq_tc_gguf_{dtype.tag}_*_plain failed with status {rc}")
    return dst


def mmvq_exact_q8_0(w: torch.Tensor, x: torch.Tensor, n: int) -> torch.Tensor:
    """`launch_mmvq_gguf_q8_0_{bf16,f32}_exact`: Q8_0 weights against unquantized activations x [b <= 8, k] (bf16 or
    f32), f32 accumulation; returns [b, n] in x's type."""
    _require_cuda(w, x)
    b, k = x.shape
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"the exact Q8_0 matvec takes bf16 or f32 activations, not {x.dtype}")
    if b > 8:
        raise ValueError("the exact Q8_0 matvec takes at most 8 activation rows")
    dst = torch.empty((b, n), dtype=x.dtype, device=x.device)
    fn = getattr(kl.library(), f"launch_mmvq_gguf_q8_0_{ELEM_TAG[elem_of(x.dtype)]}_exact")
    fn(w.data_ptr(), x.data_ptr(), dst.data_ptr(), k, n, b, _stream())
    rc = kl.library().b200q_take_launch_status()
    if rc:
        raise kl.KernelLibraryError(f"launch_mmvq_gguf_q8_0_*_exact failed with status {rc}")
    return dst


ACT_QUANT_Q8_1, ACT_QUANT_CPU = 0, 1


def gemv(dtype: GgmlDType, w: torch.Tensor, x: torch.Tensor, n: int, out: torch.Tensor | None = None,
         act_quant: int = ACT_QUANT_Q8_1) -> torch.Tensor:
    """`b200q_gemv`: one launch, activations quantized in the kernel's prologue (to Q8_1, or with
    ``ACT_QUANT_CPU`` to the reference CPU path's Q8_K / Q8_0). x [b, k] -> [b, n] of x's dtype."""
    _require_cuda(w, x)
    b, k = x.shape
    dst = torch.empty((b, n), dtype=x.dtype, device=x.device) if out is None else out
    kl.check(kl.library().b200q_gemv(int(dtype), elem_of(x.dtype), w.data_ptr(), x.data_ptr(), dst.data_ptr(), k, n,
                                     x.stride(0), dst.stride(0), b, act_quant, _stream()), "b200q_gemv")
    return dst


def gemv_group(dtypes, ws, x: torch.Tensor, ns, outs=None, act_quant: int = 0):
    """`b200q_gemv_group` / `b200q_gemv_group_act`: several weight matrices (same K) on one activation row x [1, k] in one
    launch; `act_quant` as for `gemv`."""
    _require_cuda(x, *ws)
    if x.dim() != 2 or x.shape[0] != 1:
        raise ValueError("gemv_group takes a single activation row [1, k]")
    k = x.shape[1]
    n = len(ws)
    if outs is None:
        outs = [torch.empty((1, ni), dtype=x.dtype, device=x.device) for ni in ns]
    types = (C.c_int * n)(*[int(d) for d in dtypes])
    wp = (C.c_void_p * n)(*[w.data_ptr() for w in ws])
    dp = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    nn = (C.c_int * n)(*[int(v) for v in ns])
    if act_quant == 0:
        kl.check(kl.library().b200q_gemv_group(n, types, wp, dp, nn, k, elem_of(x.dtype), x.data_ptr(), _stream()), "b200q_gemv_group")
    else:
        kl.check(kl.library().b200q_gemv_group_act(n, types, wp, dp, nn, k, elem_of(x.dtype), x.data_ptr(), act_quant, _stream()),
                 "b200q_gemv_group_act")
    return outs


def gemm(dtype: GgmlDType, w: torch.Tensor, x: torch.Tensor, n: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """`b200q_gemm`: prefill tile GEMM on the tensor cores. x [m, k] bf16/f16 -> [m, n] of x's dtype."""
    _require_cuda(w, x)
    m, k = x.shape
    y = torch.empty((m, n), dtype=x.dtype, device=x.device) if out is None else out
    kl.check(kl.library().b200q_gemm(int(dtype), elem_of(x.dtype), w.data_ptr(), x.data_ptr(), y.data_ptr(), m, n, k,
                                     x.stride(0), y.stride(0), _stream()), "b200q_gemm")
    return y


def gemv_tc_workspace(dtype: GgmlDType, k: int, device="cuda") -> torch.Tensor:
    """Scratch for `gemv_tc`: `b200q_gemv_tc_workspace_bytes` bytes, 128-byte aligned (torch's allocations are)."""
    nbytes = int(kl.library().b200q_gemv_tc_workspace_bytes(int(dtype), k))
    if nbytes <= 0:
        raise kl.KernelLibraryError(f"b200q_gemv_tc does not take K = {k}")
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def gemv_tc(dtype: GgmlDType, w: torch.Tensor, x: torch.Tensor, n: int, out: torch.Tensor | None = None,
            workspace: torch.Tensor | None = None) -> torch.Tensor:
    """`b200q_gemv_tc`: 1..16 activation rows on the tensor cores (int8). x [m, k] (rows may be strided) -> [m, n] of
    x's dtype. `workspace` from `gemv_tc_workspace`; allocated per call when not given."""
    if not (w.is_cuda and x.is_cuda) or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("expected CUDA tensors and rows of unit stride")
    m, k = x.shape
    y = torch.empty((m, n), dtype=x.dtype, device=x.device) if out is None else out
    if y.stride(1) != 1:
        raise ValueError("expected output rows of unit stride")
    ws = gemv_tc_workspace(dtype, k, x.device) if workspace is None else workspace
    kl.check(kl.library().b200q_gemv_tc(int(dtype), elem_of(x.dtype), w.data_ptr(), x.data_ptr(), y.data_ptr(), m, n, k,
                                        x.stride(0), y.stride(0), ws.data_ptr(), ws.numel() * ws.element_size(), _stream()),
             "b200q_gemv_tc")
    return y


def set_weight_successor(w: torch.Tensor, next_w: torch.Tensor | None, next_dtype: GgmlDType | None = None, next_k: int = 0,
                         next_n: int = 0) -> None:
    """`b200q_set_weight_successor`: the decode launch after the one on `w` will read `next_w` [next_n, next_k]; every
    GEMV launch on `w` then prefetches the start of `next_w` into L2. ``next_w=None`` forgets `w`."""
    if next_w is None:
        kl.check(kl.library().b200q_set_weight_successor(w.data_ptr(), None, 0, 0, 0), "b200q_set_weight_successor")
    else:
        kl.check(kl.library().b200q_set_weight_successor(w.data_ptr(), next_w.data_ptr(), int(next_dtype), next_k, next_n),
                 "b200q_set_weight_successor")


def clear_weight_successors() -> None:
    kl.check(kl.library().b200q_clear_weight_successors(), "b200q_clear_weight_successors")


def gemv_plan(dtype: GgmlDType, k: int, n: int, b: int) -> dict:
    out = (C.c_int * 10)()
    kl.check(kl.library().b200q_gemv_plan(int(dtype), k, n, b, C.byref(out)), "b200q_gemv_plan")
    keys = ("staged", "grid", "smem", "stages", "rows_per_stage", "warps_per_row", "stage_bytes", "row_align",
            "items_per_lane", "reg_slots")
    return dict(zip(keys, (int(v) for v in out)))


def set_option(name: str, value: int) -> None:
    kl.check(kl.library().b200q_set_option(name.encode(), int(value)), f"b200q_set_option({name})")


def get_option(name: str) -> int:
    v = C.c_int()
    kl.check(kl.library().b200q_get_option(name.encode(), C.byref(v)), f"b200q_get_option({name})")
    return int(v.value)
