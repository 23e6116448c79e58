"""GPU parity of the Q8_0 matvec against unquantized activations (`launch_mmvq_gguf_q8_0_{bf16,f32}_exact`), through the
C ABI: against x . dequant(W)^T accumulated in double by the oracle (only f32 summation order and output rounding
differ) and against the reference's own kernel (oracle/_ref) on the same buffers."""
import numpy as np
import pytest
import torch

from oracle import kquants as kq
from oracle import refkernels as rk

from inference_rs_b200 import ops
from gpu_util import DT, as_f32_numpy, assert_device_ok, real_packed, seeded_acts, seeded_weights

pytestmark = pytest.mark.gpu

EPS = {torch.bfloat16: 2.0 ** -8, torch.float32: 0.0}


def run_exact(n, k, b, dtype, packed=None, seed=0):
    if packed is None:
        packed = kq.quantize(kq.Q8_0, seeded_weights(n, k, 7000 + seed))
    x = seeded_acts(b, k, 7100 + seed, dtype)
    w_dev = ops.upload_weights(packed, DT[kq.Q8_0])
    got = as_f32_numpy(ops.mmvq_exact_q8_0(w_dev, x.cuda(), n)).astype(np.float64)
    torch.cuda.synchronize()
    ref = kq.matmul_dense(kq.Q8_0, as_f32_numpy(x), packed, n)
    scale = np.abs(ref).max() + 1e-30
    bad = np.abs(got - ref) > 2e-5 * scale + EPS[dtype] * 1.01 * np.abs(ref)
    assert not bad.any(), f"n={n} k={k} b={b} {dtype}: {bad.sum()} outputs off, worst {np.abs(got - ref).max():.3e} vs {scale:.3e}"
    if rk.available():
        theirs = as_f32_numpy(rk.exact_q8_0(w_dev, x.cuda(), n)).astype(np.float64)
        torch.cuda.synchronize()
        off = np.abs(got - theirs) > 4e-5 * scale + 2 * EPS[dtype] * 1.01 * np.abs(ref)
        assert not off.any(), f"{off.sum()} outputs differ from the reference's kernel, worst {np.abs(got - theirs).max():.3e}"
    assert_device_ok()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b", [1, 2, 5, 8])
def test_short_and_long_rows(dtype, b):
    for n, k in [(7, 32), (130, 512), (1000, 1024), (333, 2080), (64, 4096)]:
        run_exact(n, k, b, dtype, seed=b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_a_baseline_shape(dtype):
    run_exact(4096, 4096, 4, dtype, packed=real_packed(kq.Q8_0, 4096, 4096), seed=1)


def test_zero_inputs_give_zeros():
    packed = kq.quantize(kq.Q8_0, seeded_weights(40, 256, 3))
    w_dev = ops.upload_weights(packed, DT[kq.Q8_0])
    assert not ops.mmvq_exact_q8_0(w_dev, torch.zeros(3, 256, device="cuda"), 40).any()
    zero_w = ops.upload_weights(kq.quantize(kq.Q8_0, np.zeros((40, 256), np.float32)), DT[kq.Q8_0])
    assert not ops.mmvq_exact_q8_0(zero_w, seeded_acts(3, 256, 4, torch.float32).cuda(), 40).any()
    assert_device_ok()
