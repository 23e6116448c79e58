"""Row-count routing of the operator mirror (host logic only): which kernel `QMatMul` picks for a shape, mirroring
`prefers_mmvq` / `TENSOR_CORE_MAX_ROWS` of the reference (crates/inference-quant/src/gguf/fast_mmvq.rs:84-134)."""
import pytest

from inference_rs_b200 import GgmlDType
from inference_rs_b200 import qmatmul as qm

LLAMA_SHAPES = [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096), (4096, 128256)]  # (k, n)


@pytest.mark.parametrize("dtype", [GgmlDType.Q4K, GgmlDType.Q6K, GgmlDType.Q8_0])
def test_rows_1_2_stay_on_the_gemv_and_9_to_16_take_the_tensor_core_tier(dtype):
    for k, n in LLAMA_SHAPES:
        for rows in (1, 2):
            assert not qm.prefers_tensor_core_rows(dtype, rows, n, k) and qm.prefers_mmvq(rows)
        for rows in range(9, 17):
            assert qm.prefers_tensor_core_rows(dtype, rows, n, k)
        assert not qm.prefers_tensor_core_rows(dtype, 17, n, k) and not qm.prefers_mmvq(17)


def test_rows_3_to_8_follow_the_measured_crossovers():
    # light unpacking (Q4_K, Q8_0): from 5 rows everywhere, from 3 rows on big matrices
    for dtype in (GgmlDType.Q4K, GgmlDType.Q8_0):
        assert not qm.prefers_tensor_core_rows(dtype, 4, 4096, 4096)
        assert qm.prefers_tensor_core_rows(dtype, 5, 4096, 4096)
        assert qm.prefers_tensor_core_rows(dtype, 3, 28672, 4096) and qm.prefers_tensor_core_rows(dtype, 3, 4096, 14336)
    # Q6_K: from 7 rows everywhere, from 4 rows on big matrices, 3 rows only on the output head
    q6 = GgmlDType.Q6K
    assert not qm.prefers_tensor_core_rows(q6, 6, 4096, 4096) and qm.prefers_tensor_core_rows(q6, 7, 4096, 4096)
    assert qm.prefers_tensor_core_rows(q6, 4, 4096, 14336) and not qm.prefers_tensor_core_rows(q6, 3, 4096, 14336)
    assert qm.prefers_tensor_core_rows(q6, 3, 128256, 4096)


def test_shapes_the_tier_cannot_take_fall_back():
    assert qm.tensor_core_rows_supported(GgmlDType.Q4K, 256) and not qm.tensor_core_rows_supported(GgmlDType.Q4K, 128)
    # Q6_K rows are a multiple of 16 bytes only when K is a multiple of 2048
    assert qm.tensor_core_rows_supported(GgmlDType.Q6K, 14336) and not qm.tensor_core_rows_supported(GgmlDType.Q6K, 4096 + 256)
    assert qm.tensor_core_rows_supported(GgmlDType.Q8_0, 512) and not qm.tensor_core_rows_supported(GgmlDType.Q8_0, 96)
    assert not qm.prefers_tensor_core_rows(GgmlDType.Q6K, 12, 4096, 4096 + 256)
