"""GGUF block types on this path, with the ids and sizes the container format fixes
(crates/inference-tensor/src/quantized/mod.rs:582-624; block structs k_quants.rs:150-227)."""
from __future__ import annotations

import enum


class GgmlDType(enum.IntEnum):
    Q8_0 = 8
    Q4K = 12
    Q6K = 14

    @property
    def block_size(self) -> int:
        return 32 if self is GgmlDType.Q8_0 else 256

    @property
    def type_size(self) -> int:
        return {GgmlDType.Q8_0: 34, GgmlDType.Q4K: 144, GgmlDType.Q6K: 210}[self]

    @property
    def tag(self) -> str:
        return {GgmlDType.Q8_0: "q8_0", GgmlDType.Q4K: "q4_k", GgmlDType.Q6K: "q6_k"}[self]

    def row_bytes(self, k: int) -> int:
        if k % self.block_size:
            raise ValueError(f"{k} columns are not a multiple of the {self.name} block of {self.block_size}")
        return k // self.block_size * self.type_size


# element types of activations / outputs at the C ABI
ELEM_F32, ELEM_F16, ELEM_BF16 = 0, 1, 2
ELEM_TAG = {ELEM_F32: "f32", ELEM_F16: "f16", ELEM_BF16: "bf16"}
# the reference's `type_x` codes for the prefill activation quantizer (crates/inference-quant/src/gguf/fast_mmq.rs:671-676)
MMQ_TYPE_X = {ELEM_F32: 0, ELEM_F16: 1, ELEM_BF16: 30}
MATRIX_ROW_PADDING = 512  # activation rows are padded to this many values (kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:33)


def pad(k: int, to: int) -> int:
    return (k + to - 1) // to * to
