"""Host-side mirror of the reference's quantized-matmul operator for this path: `QTensor`, `QMatMul` and
`GgufMatMul` with the same names, argument meaning and error behaviour, on torch device memory.

Reference: `QTensor` / `QMatMul` (crates/inference-tensor/src/quantized/mod.rs:85-120,1117-1187,1625-1647),
`GgufMatMul::forward` and its dispatch (crates/inference-quant/src/gguf/mod.rs:435-571), the row-count policy of
`fast_mmvq::plain` / `fast_mmq::plain` (crates/inference-quant/src/gguf/fast_mmvq.rs:84-134,477-665,
fast_mmq.rs:604-715). Every forward runs the CUDA kernels of the C-ABI library; there is no CPU fallback.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops
from .dtypes import MATRIX_ROW_PADDING, GgmlDType, pad
from .kernel_library import KernelLibraryError

MMVQ_MAX_BATCH = 8  # rows the decode GEMV launchers take (fast_mmvq.rs:84)
TENSOR_CORE_MAX_ROWS = 16  # rows the small-batch tensor-core kernel takes (fast_mmvq.rs:86)
# 3..8 rows: the crossovers measured on B200 against the dp4a GEMV at the Llama-3-8B shapes. The tier's cost hardly
# grows with the row count, the GEMV's grows linearly; Q6_K's unpacking is the most expensive, so it needs more rows
# or a bigger matrix. 9..16 rows: always (the alternative is the prefill GEMM).


def _tensor_core_pays(dtype: GgmlDType, rows: int, n: int, k: int) -> bool:
    big = k >= 8192 or n >= 16384
    if dtype == GgmlDType.Q6K:
        return rows >= 7 or (rows >= 4 and big) or n >= 65536
    return rows >= 5 or big


_tc_workspaces: dict = {}


def _tc_workspace(dtype: GgmlDType, k: int, device: torch.device) -> torch.Tensor:
    """One scratch buffer per (device, stream, type, k), like the reference's per-thread, per-stream activation
    workspace (crates/inference-quant/src/gguf/thread_workspace.rs:94-146): its address is stable, so captured
    graphs can replay, and calls on one stream are ordered, so they never overlap on it."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, int(dtype), k)
    ws = _tc_workspaces.get(key)
    if ws is None:
        ws = _tc_workspaces[key] = ops.gemv_tc_workspace(dtype, k, device)
    return ws


def tensor_core_rows_supported(dtype: GgmlDType, k: int) -> bool:
    """Shapes `b200q_gemv_tc` takes: whole 256-value chunks and packed rows of a multiple of 16 bytes."""
    return k % 256 == 0 and dtype.row_bytes(k) % 16 == 0


def prefers_tensor_core_rows(dtype: GgmlDType, rows: int, n: int, k: int) -> bool:
    """The small-batch tensor-core tier (fast_mmvq.rs:118-134: 2..16 rows where a type has it). Here: 9..16 rows
    always, 3..8 rows from the measured crossover with the dp4a GEMV on; 1..2 rows stay on the one-launch GEMV."""
    if rows > TENSOR_CORE_MAX_ROWS or rows < 3 or not tensor_core_rows_supported(dtype, k):
        return False
    return rows > MMVQ_MAX_BATCH or _tensor_core_pays(dtype, rows, n, k)


class QTensor:
    """Packed GGUF blocks of a `[n, k]` weight on a CUDA device (rows contiguous, then the reference's padding)."""

    def __init__(self, data: torch.Tensor, dtype: GgmlDType, shape: tuple[int, int]):
        n, k = shape
        if k % dtype.block_size:
            # mod.rs:872-884: the last dimension must hold whole blocks
            raise ValueError(f"quantized tensor last dim {k} is not a multiple of the {dtype.name} block size {dtype.block_size}")
        need = n * dtype.row_bytes(k)
        if data.dtype != torch.uint8 or data.numel() < need:
            raise ValueError(f"{dtype.name} tensor of shape {shape} needs {need} bytes, got {data.numel()} of {data.dtype}")
        self.data, self.dtype, self.shape = data, dtype, (n, k)

    @classmethod
    def from_packed(cls, packed, dtype: GgmlDType, shape: tuple[int, int], device="cuda") -> "QTensor":
        """From host bytes (numpy uint8 or torch CPU tensor), uploaded with the trailing padding."""
        return cls(ops.upload_weights(packed, dtype, device), dtype, shape)

    @classmethod
    def quantize(cls, src: torch.Tensor, dtype: GgmlDType) -> "QTensor":
        """`QTensor::quantize(&tensor, dtype)` (mod.rs:903-918): an f32 `[n, k]` tensor packed on its device by the library's
        quantizer, byte for byte what the reference's host quantizer writes. `k` must hold whole blocks."""
        if src.dim() != 2:
            raise ValueError(f"quantize takes a matrix, got {tuple(src.shape)}")
        n, k = src.shape
        if k % dtype.block_size:
            raise ValueError(f"quantized tensor last dim {k} is not a multiple of the {dtype.name} block size {dtype.block_size}")
        x = src.detach().to(dtype=torch.float32).contiguous()
        if not x.is_cuda:
            x = x.cuda()
        return cls(ops.quantize_weights(x, dtype), dtype, (n, k))

    def dequantize(self, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """`QTensor::dequantize` (mod.rs:920-940): the values as a dense `[n, k]` tensor on the same device."""
        return ops.dequantize(self.dtype, self.data, self.shape[0], self.shape[1], out_dtype)

    def embedding(self, ids: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """The rows `ids` names, dequantized: the quantized embedding lookup (crates/inference-quant/src/gguf/mod.rs:546-548)."""
        return ops.get_rows(self.dtype, self.data, ids, self.shape[0], self.shape[1], out_dtype)

    @property
    def storage_size_in_bytes(self) -> int:
        return self.shape[0] * self.dtype.row_bytes(self.shape[1])

    def packed_bytes(self) -> torch.Tensor:
        """The blocks without the padding."""
        return self.data[: self.storage_size_in_bytes]

    @property
    def device(self) -> torch.device:
        return self.data.device


class QMatMul:
    """`y = x @ W^T` for a quantized `W`; x `[..., k]` contiguous -> y `[..., n]` in x's dtype (mod.rs:1625-1647)."""

    def __init__(self, qtensor: QTensor):
        self.qtensor = qtensor

    @classmethod
    def from_qtensor(cls, qtensor: QTensor) -> "QMatMul":
        return cls(qtensor)

    def forward(self, xs: torch.Tensor, act_quant: int = ops.ACT_QUANT_Q8_1) -> torch.Tensor:
        n, k = self.qtensor.shape
        if xs.dim() < 2:
            raise ValueError(f"input tensor has only one dimension {tuple(xs.shape)}")
        if not xs.is_contiguous():
            raise ValueError(f"input tensor is not contiguous {tuple(xs.shape)}")
        if xs.shape[-1] != k:
            raise ValueError(f"input tensor {tuple(xs.shape)} incompatible with {(n, k)}")
        if xs.device != self.qtensor.device:
            raise ValueError(f"input on {xs.device}, weights on {self.qtensor.device}")
        x2 = xs.reshape(-1, k)
        y = _forward_rows(self.qtensor, x2, act_quant)
        return y.reshape(*xs.shape[:-1], n)

    __call__ = forward


def prefers_mmvq(rows: int) -> bool:
    """Decode GEMV for up to MMVQ_MAX_BATCH rows where the tensor-core tier does not take them, the prefill GEMM above
    (fast_mmvq.rs:96-134)."""
    return rows <= MMVQ_MAX_BATCH


def _forward_rows(w: QTensor, x: torch.Tensor, act_quant: int) -> torch.Tensor:
    n, k = w.shape
    rows = x.shape[0]
    if rows == 0:
        return torch.empty((0, n), dtype=x.dtype, device=x.device)
    if act_quant == ops.ACT_QUANT_Q8_1 and prefers_tensor_core_rows(w.dtype, rows, n, k):
        return ops.gemv_tc(w.dtype, w.data, x, n, workspace=_tc_workspace(w.dtype, k, x.device))
    if prefers_mmvq(rows):
        if k % 128 == 0:
            try:
                return ops.gemv(w.dtype, w.data, x, n, act_quant=act_quant)
            except KernelLibraryError as exc:
                # B200Q_ERR_UNSUPPORTED: no staged plan for this call (weights not 16-byte aligned, the simple kernel
                # forced, no ring that fits). The library can still serve Q8_1 activations in two launches.
                if act_quant != ops.ACT_QUANT_Q8_1 or exc.status != -1:
                    raise
        elif act_quant != ops.ACT_QUANT_Q8_1:
            raise ValueError(f"the CPU path's activation format needs K a multiple of 128, got {k}")
        # shapes the one-launch kernel declines: the reference's own two-launch protocol
        vy = ops.quantize_q8_1(x, pad(k, MATRIX_ROW_PADDING))
        return ops.mmvq_plain(w.dtype, w.data, vy, n, k, rows, x.dtype)
    if x.dtype in (torch.bfloat16, torch.float16) and k % 64 == 0:
        return ops.gemm(w.dtype, w.data, x, n)
    if x.dtype == torch.float32 and k % 64 == 0:
        # the tensor-core path takes 16-bit activations; f32 inputs are narrowed as the reference narrows them for
        # its own CUDA path (crates/inference-quant/src/gguf/mod.rs:667-691 keeps bf16 when given bf16)
        return ops.gemm(w.dtype, w.data, x.to(torch.bfloat16), n).to(torch.float32)
    # K not a multiple of 64 (Q8_0 only): batches of the GEMV launcher
    outs = []
    for i in range(0, rows, MMVQ_MAX_BATCH):
        xb = x[i:i + MMVQ_MAX_BATCH].contiguous()
        vy = ops.quantize_q8_1(xb, pad(k, MATRIX_ROW_PADDING))
        outs.append(ops.mmvq_plain(w.dtype, w.data, vy, n, k, xb.shape[0], x.dtype))
    return torch.cat(outs, 0)


class GgufMatMul:
    """The `QuantMethod` of GGUF weights: forward = quantized matmul plus optional bias
    (crates/inference-quant/src/gguf/mod.rs:92-100,513-571; trait crates/inference-quant/src/lib.rs:2014-2291)."""

    def __init__(self, w: QMatMul, b: torch.Tensor | None = None):
        self.w, self.b = w, b

    @classmethod
    def from_qtensor(cls, q: QTensor, bias: torch.Tensor | None = None) -> "GgufMatMul":
        return cls(QMatMul.from_qtensor(q), bias)

    def quantized_act_type(self):
        return None  # CUDA GGUF takes activations as they are (gguf/mod.rs:667-691)

    def dtype_and_device(self):
        return self.w.qtensor.dtype, self.w.qtensor.device

    def is_distributed(self) -> bool:
        return False

    def get_qtensor(self) -> QTensor:
        return self.w.qtensor

    def forward_raw(self, x: torch.Tensor) -> torch.Tensor:
        y = self.w.forward(x)
        return y if self.b is None else y + self.b.to(y.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_raw(x)

    __call__ = forward

