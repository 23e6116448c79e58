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


@pytest.mark.parametrize("layout", ["D4", "DS4"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("activation", ["relu", "silu", "gelu", "gelu_erf", "sigmoid"])
def test_glu_prefill_quantizer_equals_the_plain_one_on_the_product(layout, dtype, activation):
    """launch_mmq_quantize_glu_q8_1_*: the blocks of act(gate) * up (activation in f32, rounded to the input type; product in
    the input type) equal the plain quantizer's blocks of that product: bit for bit with ReLU, and with the
    transcendental activations wherever the host's and the device's exp / tanh / erf round alike (all scales within
    one f32 / f16 rounding, quants one step apart at most, in a small fraction of the positions)."""
    from inference_rs_b200 import ops
    rows, k = 9, 640
    g = torch.Generator().manual_seed(17)
    gate = (torch.randn(rows, k, generator=g) * 2.0).to(dtype)
    up = torch.randn(rows, k, generator=g).to(dtype)
    gf = gate.float()
    act = {"relu": torch.clamp(gf, min=0.0), "silu": gf / (1.0 + torch.exp(-gf)),
           "gelu": 0.5 * gf * (1.0 + torch.tanh(0.7978845608 * (gf + 0.044715 * gf * gf * gf))),
           "gelu_erf": gf * 0.5 * (1.0 + torch.erf(gf * 0.7071067811865476)), "sigmoid": 1.0 / (1.0 + torch.exp(-gf))}[activation]
    product = act.to(dtype) * up
    want = ops.quantize_mmq_q8_1(product.cuda(), layout).cpu().numpy().reshape(-1, 144)
    got = ops.quantize_mmq_q8_1_glu(gate.cuda(), up.cuda(), layout, activation).cpu().numpy().reshape(-1, 144)
    torch.cuda.synchronize()
    if activation == "relu":
        assert np.array_equal(got, want)
        if dtype == torch.float32:
            again = ops.quantize_mmq_q8_1_glu(gate.cuda(), up.cuda(), layout, activation, typed=False).cpu().numpy().reshape(-1, 144)
            assert np.array_equal(again, want)
        return
    sc = np.float32 if layout == "D4" else np.float16
    np.testing.assert_allclose(got[:, :16].copy().view(sc).astype(np.float32), want[:, :16].copy().view(sc).astype(np.float32),
                               rtol=2e-3, atol=1e-6)
    dq = got[:, 16:].view(np.int8).astype(np.int32) - want[:, 16:].view(np.int8).astype(np.int32)
    assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 5e-3
