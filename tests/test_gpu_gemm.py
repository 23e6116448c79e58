"""GPU parity of the prefill GEMM (tcgen05 tile GEMM with in-kernel dequantization), through the C ABI.

  * against the same arithmetic in double (activations as given, weights dequantized by the oracle and rounded to the
    activation type as the kernel does): only f32 accumulation order and output rounding differ;
  * against the reference CPU path (Q8_K / Q8_0 activations): per tensor, max|d| <= 1e-3 + 1e-2 max|ref|. The kernel
    keeps activations unquantized, so it is closer to the dense product than the CPU path is.
"""
import numpy as np
import pytest
import torch

from oracle import kquants as kq

from inference_rs_b200 import ops
from gpu_util import DT, TYPES, as_f32_numpy, assert_device_ok, random_packed, seeded_acts, seeded_weights

pytestmark = pytest.mark.gpu


def rounded_weights(type_id, packed, k, dtype):
    w = kq.dequantize(type_id, packed, k)
    t = torch.from_numpy(w).to(dtype).float().numpy()
    return t.astype(np.float64)


def run_gemm(type_id, m, n, k, dtype=torch.bfloat16, packed=None, seed=0, check_cpu=True):
    real = packed is None
    if packed is None:
        packed = kq.quantize(type_id, seeded_weights(n, k, 3000 + seed))
    x = seeded_acts(m, k, 4000 + seed, dtype)
    w_dev = ops.upload_weights(packed, DT[type_id])
    y = ops.gemm(DT[type_id], w_dev, x.cuda(), n)
    torch.cuda.synchronize()
    assert_device_ok()
    got = as_f32_numpy(y).astype(np.float64)
    xf = as_f32_numpy(x).astype(np.float64)
    ref = xf @ rounded_weights(type_id, packed, k, dtype).T
    eps = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    scale = np.abs(ref).max()
    bad = np.abs(got - ref) > 1e-4 * scale + eps * 1.01 * np.abs(ref)
    assert not bad.any(), (f"{kq.TYPE_NAMES[type_id]} m={m} n={n} k={k}: {bad.sum()} outputs off, worst {np.abs(got - ref).max():.3e} "
                           f"vs scale {scale:.3e}; first at {np.argwhere(bad)[:4].tolist()}")
    if check_cpu:
        cpu = kq.matmul(type_id, as_f32_numpy(x), packed, n)
        rel = 1e-2 if real else 2e-2
        assert np.abs(got - cpu).max() <= 1e-3 + rel * np.abs(cpu).max()


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (40, 64, 512), (17, 130, 256), (300, 200, 1024), (512, 384, 768)])
def test_small_tiles_and_ragged_edges(type_id, m, n, k):
    run_gemm(type_id, m, n, k, seed=m + n)


@pytest.mark.parametrize("type_id", TYPES)
def test_f16_activations(type_id):
    run_gemm(type_id, 256, 256, 512, dtype=torch.float16)


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q6_K])
@pytest.mark.parametrize("k,n", [(4096, 4096), (14336, 4096), (4096, 6144)])
def test_prefill_shapes_m512(type_id, k, n):
    run_gemm(type_id, 512, n, k, packed=random_packed(type_id, n, k, seed=k + n), seed=1)


def test_two_subtiles_path_large_m():
    # M = 2048 with enough tiles takes the 256-token CTA tile
    run_gemm(kq.Q4_K, 2048, 4096, 4096, packed=random_packed(kq.Q4_K, 4096, 4096, seed=5), seed=2, check_cpu=False)


def test_rows_are_independent():
    type_id, n, k = kq.Q4_K, 512, 1024
    packed = random_packed(type_id, n, k, seed=9)
    w_dev = ops.upload_weights(packed, DT[type_id])
    x = seeded_acts(300, k, 7, torch.bfloat16).cuda()
    full = ops.gemm(DT[type_id], w_dev, x, n)
    part = ops.gemm(DT[type_id], w_dev, x[100:228].contiguous(), n)
    assert torch.equal(part, full[100:228])
    assert_device_ok()


def test_unsupported_inputs_are_refused():
    from inference_rs_b200 import kernel_library as kl
    w_dev = ops.upload_weights(random_packed(kq.Q4_K, 128, 256, 1), DT[kq.Q4_K])
    with pytest.raises(TypeError):
        ops.gemm(DT[kq.Q4_K], w_dev, torch.zeros(32, 256, device="cuda", dtype=torch.float64), 128)
    with pytest.raises(kl.KernelLibraryError, match="bf16 or f16"):
        ops.gemm(DT[kq.Q4_K], w_dev, torch.zeros(32, 256, device="cuda", dtype=torch.float32), 128)
