"""GPU parity of the activation quantizers: bit-exact against the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import kquants as kq

from inference_rs_b200 import ops
from gpu_util import TORCH_DTYPES, as_f32_numpy, assert_device_ok, seeded_acts

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("rows,k", [(1, 4096), (3, 700), (16, 512), (17, 14336), (1, 32), (5, 96)])
def test_q8_1_blocks_are_bit_exact(dtype, rows, k):
    x = seeded_acts(rows, k, 1, TORCH_DTYPES[dtype])
    x[0, : min(k, 32)] = 0  # an all-zero block
    k_padded = (k + 511) // 512 * 512
    got = ops.quantize_q8_1(x.cuda(), k_padded).cpu().numpy()
    want = kq.quantize_q8_1_mmvq(as_f32_numpy(x), k_padded)
    assert got.shape == want.shape
    assert np.array_equal(got, want), f"{(got != want).sum()} bytes differ"
    assert_device_ok()


def test_q8_1_ties_and_extremes():
    # values that sit exactly on .5 after scaling, the largest magnitudes and denormal-sized inputs
    base = np.array([127.0] + [(i - 16.0) + 0.5 for i in range(1, 32)], np.float32)
    x = np.stack([base, -base, base * 1e-30, base * 3e30, np.zeros(32, np.float32)])
    got = ops.quantize_q8_1(torch.from_numpy(x).cuda(), 32).cpu().numpy()
    want = kq.quantize_q8_1_mmvq(x, 32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("layout,code", [("D4", 0), ("DS4", 1)])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("rows,k", [(1, 4096), (40, 512), (130, 1000), (512, 4096)])
def test_prefill_blocks_are_bit_exact(layout, code, dtype, rows, k):
    x = seeded_acts(rows, k, 2, TORCH_DTYPES[dtype])
    k_padded = (k + 511) // 512 * 512
    got = ops.quantize_mmq_q8_1(x.cuda(), layout, k_padded).cpu().numpy()
    want = kq.quantize_q8_1_mmq(as_f32_numpy(x), k_padded, code)
    assert np.array_equal(got, want), f"{(got != want).sum()} bytes differ"
    assert_device_ok()
