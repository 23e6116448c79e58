"""GPU parity of the prefill GEMM (tcgen05 tile GEMM with in-kernel dequantization), through the C ABI.

  * against the same arithmetic in double (activations as given, weights dequantized by the oracle and rounded to the
    activation type as the kernel does): only f32 accumulation order and output rounding differ;
  * against the reference CPU path (Q8_K / Q8_0 activations): per tensor, max|d| <= 1e-3 + 1e-2 max|ref|. The kernel
    keeps activations unquantized, so it is closer to the dense product than the CPU path is;
  * against the reference's own CUDA prefill path (oracle/_ref: its activation quantizer + MMQ tile GEMM, compiled
    from the reference checkout), per tensor at the bound the reference's own CUDA tests use, max|d| <= 0.02 max|ref|
    (crates/inference-quant/src/gguf/mod.rs:998-1037): that path quantizes the activations to int8 and multiplies block
    scales in half precision (mmq_gguf.cuh:2207-2211), so it sits 1.2 - 1.6 % of the largest output away from this kernel,
    which keeps activations in 16 bits and scales in f32 and is the closer of the two to the CPU path.

Shapes of the baseline's prefill sweep use ~N(0, 0.02) weights packed by the oracle's quantizer. At M = 2048 and 8192
the CPU comparisons run on a seeded sample of the token rows (output rows are independent; the oracle is scalar code)
and every row is covered by comparing the large call with calls on 512-token slices, bit for bit.
"""
import numpy as np
import pytest
import torch

from oracle import kquants as kq

from oracle import refkernels as rk

from inference_rs_b200 import ops
from gpu_util import DT, TYPES, as_f32_numpy, assert_device_ok, random_packed, real_packed, seeded_acts, seeded_weights

pytestmark = pytest.mark.gpu


def rounded_weights(type_id, packed, k, dtype):
    w = kq.dequantize(type_id, packed, k)
    t = torch.from_numpy(w).to(dtype).float().numpy()
    return t.astype(np.float64)


def run_gemm(type_id, m, n, k, dtype=torch.bfloat16, packed=None, seed=0, check_cpu=True, real=None, sample_rows=None):
    if real is None:
        real = packed is None
    if packed is None:
        packed = kq.quantize(type_id, seeded_weights(n, k, 3000 + seed))
    x = seeded_acts(m, k, 4000 + seed, dtype)
    w_dev = ops.upload_weights(packed, DT[type_id])
    x_dev = x.cuda()
    y = ops.gemm(DT[type_id], w_dev, x_dev, n)
    torch.cuda.synchronize()
    assert_device_ok()
    rows = np.arange(m)
    if sample_rows is not None and sample_rows < m:
        rows = np.sort(np.random.default_rng(seed).choice(m, size=sample_rows, replace=False))
        # rows outside the sample: the same bits as calls on 512-token slices
        for r0 in range(0, m, 512):
            part = ops.gemm(DT[type_id], w_dev, x_dev[r0:r0 + 512].contiguous(), n)
            assert torch.equal(part, y[r0:r0 + 512]), f"rows {r0}..{r0 + 512} differ from the slice run alone"
    got = as_f32_numpy(y)[rows].astype(np.float64)
    xf = as_f32_numpy(x)[rows].astype(np.float64)
    ref = xf @ rounded_weights(type_id, packed, k, dtype).T
    eps = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    scale = np.abs(ref).max()
    bad = np.abs(got - ref) > 1e-4 * scale + eps * 1.01 * np.abs(ref)
    assert not bad.any(), (f"{kq.TYPE_NAMES[type_id]} m={m} n={n} k={k}: {bad.sum()} outputs off, worst {np.abs(got - ref).max():.3e} "
                           f"vs scale {scale:.3e}; first at {np.argwhere(bad)[:4].tolist()}")
    if check_cpu:
        cpu = kq.matmul(type_id, as_f32_numpy(x)[rows], packed, n)
        rel = 1e-2 if real else 2e-2
        assert np.abs(got - cpu).max() <= 1e-3 + rel * np.abs(cpu).max()
    if rk.available() and k % 256 == 0:
        theirs = as_f32_numpy(rk.mmq_forward(type_id, w_dev, x_dev, n))[rows].astype(np.float64)
        torch.cuda.synchronize()
        assert np.abs(got - theirs).max() <= 2e-2 * np.abs(theirs).max(), "differs from the reference's MMQ"


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
    run_gemm(type_id, 512, n, k, packed=real_packed(type_id, n, k), seed=1, real=True)


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q6_K])
@pytest.mark.parametrize("k,n", [(4096, 4096), (14336, 4096)])
@pytest.mark.parametrize("m", [2048, 8192])
def test_prefill_shapes_large_m(type_id, k, n, m):
    # M = 2048 with enough tiles takes the 256-token CTA tile; M = 8192 is the compute-bound end of the sweep
    run_gemm(type_id, m, n, k, packed=real_packed(type_id, n, k), seed=m, real=True, sample_rows=192)


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q6_K])
def test_prefill_wide_shapes(type_id):
    # the gate+up shape (4096 x 28672) at 512 tokens, CPU path on a sample of the rows
    run_gemm(type_id, 512, 28672, 4096, packed=real_packed(type_id, 28672, 4096), seed=3, real=True, sample_rows=96)


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


# ---------------------------------------------------------------------------------------------------------------------
# The reference's prefill launcher pair: launch_mmq_quantize_q8_1_{D4,DS4} + launch_mmq_gguf_<type>
# ---------------------------------------------------------------------------------------------------------------------
def mmq_reference_math(type_id, x32, packed, k):
    """(d q) . dequant(W)^T in double, with the prefill quantizer's d and q per 32 values (d_inv = 127 / amax,
    q = roundf(x d_inv), d = 1 / d_inv; mmq_quantize.cu:158-198); the DS4 blocks Q4_K weights take store d as f16."""
    m = x32.shape[0]
    b = x32.reshape(m, k // 32, 32)
    amax = np.abs(b).max(axis=2, keepdims=True).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        d_inv = (np.float32(127.0) / amax).astype(np.float32)
        v = (b * d_inv).astype(np.float32)
        q = np.where(amax == 0, 0, np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)))
        d = np.where(amax == 0, 0, (np.float32(1.0) / d_inv).astype(np.float32)).astype(np.float32)
    if ops.MMQ_LAYOUT[DT[type_id]] == "DS4":
        d = d.astype(np.float16).astype(np.float32)
    return (d.astype(np.float64) * q).reshape(m, k), kq.dequantize(type_id, packed, k).astype(np.float64)


def run_mmq(type_id, m, n, k, dtype=torch.bfloat16, packed=None, seed=0, real=None, sample_rows=None):
    if real is None:
        real = packed is None
    if packed is None:
        packed = kq.quantize(type_id, seeded_weights(n, k, 8000 + seed))
    x = seeded_acts(m, k, 8100 + seed, dtype)
    w_dev = ops.upload_weights(packed, DT[type_id])
    layout = ops.MMQ_LAYOUT[DT[type_id]]
    vy = ops.quantize_mmq_q8_1(x.cuda(), layout)
    y = ops.mmq(DT[type_id], w_dev, vy, m, n, k, dtype)
    torch.cuda.synchronize()
    assert_device_ok()
    rows = np.arange(m)
    if sample_rows is not None and sample_rows < m:
        rows = np.sort(np.random.default_rng(seed).choice(m, size=sample_rows, replace=False))
    got = as_f32_numpy(y)[rows].astype(np.float64)
    xq, wd = mmq_reference_math(type_id, as_f32_numpy(x)[rows], packed, k)
    if k % 256 == 0 and DT[type_id].row_bytes(k) % 16 == 0:
        # the tile kernel rounds d q and the dequantized weights to bf16 before the tensor core multiplies them
        xq = torch.from_numpy(xq).to(torch.bfloat16).double().numpy()
        wd = torch.from_numpy(wd).to(torch.bfloat16).double().numpy()
    ref = xq @ wd.T
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -22}[dtype]
    scale = np.abs(ref).max()
    bad = np.abs(got - ref) > 1e-4 * scale + eps * 1.01 * np.abs(ref)
    assert not bad.any(), (f"{kq.TYPE_NAMES[type_id]} m={m} n={n} k={k}: {bad.sum()} outputs off, worst {np.abs(got - ref).max():.3e} "
                           f"vs scale {scale:.3e}; first at {np.argwhere(bad)[:4].tolist()}")
    cpu = kq.matmul(type_id, as_f32_numpy(x)[rows], packed, n)
    assert np.abs(got - cpu).max() <= 1e-3 + (1e-2 if (real and k >= 1024) else 2e-2) * np.abs(cpu).max()
    if rk.available():
        # the same blocks, followed by the 128 spare blocks the reference's host allocates behind them (fast_mmq.rs:686-692)
        vy_ref = torch.zeros(vy.numel() + 128 * 144, dtype=torch.uint8, device="cuda")
        vy_ref[: vy.numel()] = vy.reshape(-1)
        theirs = as_f32_numpy(rk.mmq(type_id, w_dev, vy_ref, m, n, k, dtype))[rows].astype(np.float64)
        torch.cuda.synchronize()
        assert np.abs(got - theirs).max() <= 2e-2 * np.abs(theirs).max(), "differs from the reference's MMQ on the same blocks"
    return y


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (40, 64, 512), (17, 130, 256), (300, 200, 1024), (512, 384, 768), (2048, 4096, 512)])
def test_mmq_launcher_small_tiles_and_ragged_edges(type_id, m, n, k):
    run_mmq(type_id, m, n, k, seed=m + n)


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_mmq_launcher_output_types(type_id, dtype):
    run_mmq(type_id, 200, 256, 512, dtype=dtype)


def test_mmq_launcher_shapes_the_tile_kernel_does_not_take():
    run_mmq(kq.Q8_0, 20, 100, 96, seed=1)      # K not a multiple of 256
    run_mmq(kq.Q6_K, 33, 64, 768, seed=2)      # 210-byte blocks: rows not a multiple of 16 bytes
    run_mmq(kq.Q8_0, 9, 64, 1056, seed=3)


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q6_K])
@pytest.mark.parametrize("k,n", [(4096, 4096), (14336, 4096)])
@pytest.mark.parametrize("m", [512, 2048])
def test_mmq_launcher_prefill_shapes(type_id, k, n, m):
    run_mmq(type_id, m, n, k, packed=real_packed(type_id, n, k), seed=m, real=True, sample_rows=128)
