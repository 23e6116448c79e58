"""GPU parity of the small-batch tensor-core kernel (`b200q_gemv_tc`, 1..16 activation rows, int8 MMA), through the C ABI.

The kernel's arithmetic is the reference tensor-core matvec tier's: activations quantized per 32 values to int8 with
d = f16(amax / 127), q = roundf(x / d) (mmvq_gguf/mmvq_quantize.cu:157-190), exact integer dot products per block,
block scales applied in f32. Gates:
  * against that arithmetic in double (weights dequantized by the oracle times d * q): only the f32 scale products,
    their summation order and the output rounding differ;
  * per tensor against the reference CPU path (Q8_K / Q8_0 activations): max|d| <= 1e-3 + 1e-2 max|ref|;
  * against the reference's own tensor-core matvec (oracle/_ref: launch_mmvq_tc_quantize_* +
    launch_mmvq_tc_gguf_{q4_k,q6_k}_*_plain, compiled from the reference checkout), the same arithmetic.
"""
import numpy as np
import pytest
import torch

from oracle import kquants as kq

from oracle import refkernels as rk

from inference_rs_b200 import kernel_library as kl
from inference_rs_b200 import ops
from gpu_util import (DT, Q8_1_VS_CPU_PASS_FLOOR, TYPES, as_f32_numpy, assert_device_ok, elementwise_pass_rate, random_packed,
                      real_packed, seeded_acts, seeded_weights)

pytestmark = pytest.mark.gpu

EPS = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -22}


def k_for(type_id, k):
    """Packed rows are fetched by TMA, whose row pitch must be a multiple of 16 bytes: any multiple of 256 for Q4_K
    (144-byte blocks) and Q8_0, multiples of 2048 for Q6_K (210-byte blocks)."""
    return -(-k // 2048) * 2048 if type_id == kq.Q6_K else k


def requantized(x32):
    """x [m, k] f32 -> d * q in f64 with the tier's block quantization."""
    m, k = x32.shape
    b = x32.reshape(m, k // 32, 32)
    amax = np.abs(b).max(axis=2, keepdims=True).astype(np.float32)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (b / d).astype(np.float32)
    q = np.where(amax == 0, 0, np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)))
    dh = d.astype(np.float16).astype(np.float64)
    return (dh * q.astype(np.float64)).reshape(m, k)


def run_tc(type_id, m, n, k, dtype=torch.bfloat16, packed=None, seed=0, check_cpu=True, scale=1.0, real=None):
    if real is None:
        real = packed is None
    if packed is None:
        packed = kq.quantize(type_id, seeded_weights(n, k, 5000 + seed))
    x = (seeded_acts(m, k, 6000 + seed, torch.float32) * scale).to(dtype)
    w_dev = ops.upload_weights(packed, DT[type_id])
    y = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    ops.gemv_tc(DT[type_id], w_dev, x.cuda(), n, out=y)
    torch.cuda.synchronize()
    assert_device_ok()
    got = as_f32_numpy(y).astype(np.float64)
    assert np.isfinite(got).all(), f"{np.isnan(got).sum()} outputs were never written"
    ref = requantized(as_f32_numpy(x)) @ kq.dequantize(type_id, packed, k).astype(np.float64).T
    size = np.abs(ref).max()
    bad = np.abs(got - ref) > 2e-5 * size + EPS[dtype] * 1.01 * np.abs(ref)
    assert not bad.any(), (f"{kq.TYPE_NAMES[type_id]} m={m} n={n} k={k}: {bad.sum()} outputs off, worst {np.abs(got - ref).max():.3e} "
                           f"vs size {size:.3e}; first at {np.argwhere(bad)[:4].tolist()}")
    if check_cpu:
        cpu = kq.matmul(type_id, as_f32_numpy(x), packed, n)
        # the two activation formats (a scale per 32 values here, per 256 on the CPU) differ by their own quantization
        # noise, which for short rows and hundreds of thousands of outputs reaches the 1 % line by itself
        rel = 1e-2 if (real and k >= 1024) else 2e-2
        assert np.abs(got - cpu).max() <= 1e-3 + rel * np.abs(cpu).max()
        if real and k >= 1024 and m * n >= 4096:
            assert elementwise_pass_rate(got, cpu) >= Q8_1_VS_CPU_PASS_FLOOR[type_id]
    if rk.available() and type_id != kq.Q8_0 and scale == 1.0:
        # the reference's tier (it has no Q8_0 instance) on the same quantized activations, laid out for it by the oracle
        # (its own quantizer is built with approximate division, so now and then one of its quants sits a step away):
        # only the order of the f32 scale products differs
        vy = torch.from_numpy(kq.quantize_mmvq_tc(as_f32_numpy(x))).cuda()
        theirs = as_f32_numpy(rk.tc_plain(type_id, w_dev, vy, n, k, m, dtype)).astype(np.float64)
        torch.cuda.synchronize()
        # (two separately rounded outputs may sit one unit of the output type apart: 2 eps)
        off = np.abs(got - theirs) > 1e-4 * size + 2 * EPS[dtype] * 1.01 * np.abs(ref)
        assert not off.any(), f"{off.sum()} outputs differ from the reference's tensor-core matvec, worst {np.abs(got - theirs).max():.3e} vs {size:.3e}"
    return y


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (3, 64, 512), (16, 130, 256), (5, 1000, 1024), (12, 148 * 128 + 77, 256),
                                   (16, 40000, 512), (8, 9000, 768), (9, 300, 2048)])
def test_ragged_row_ranges_and_every_row_split(type_id, m, n, k):
    # n < SM count (one row per CTA), n not a multiple of the CTA count, several tiles per CTA with a short last one;
    # m <= 4, <= 8 and above take different splits of the scaling work
    run_tc(type_id, m, n, k_for(type_id, k), seed=m + n)


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_other_activation_types(type_id, dtype):
    run_tc(type_id, 7, 512, k_for(type_id, 768), dtype=dtype)


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("k,n", [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096), (4096, 128256)])
def test_decode_sweep_shapes_batch_4_and_16(type_id, k, n):
    """BASELINE config 2 at batch 4 and 16 on all five shapes and three types, weights ~N(0, 0.02) packed by the oracle."""
    packed = real_packed(type_id, n, k)
    for m in (4, 16):
        run_tc(type_id, m, n, k, packed=packed, seed=m, real=True)


def test_zero_rows_and_large_magnitudes():
    type_id, n, k = kq.Q4_K, 256, 1024
    packed = random_packed(type_id, n, k, seed=8)
    w_dev = ops.upload_weights(packed, DT[type_id])
    x = seeded_acts(6, k, 3, torch.float32)
    x[2] = 0.0            # amax = 0: d = 0, all quants 0
    x[4] *= 1000.0
    x[5, 32:64] = 0.0     # one all-zero block inside a row
    y = ops.gemv_tc(DT[type_id], w_dev, x.cuda(), n)
    torch.cuda.synchronize()
    assert_device_ok()
    got = as_f32_numpy(y).astype(np.float64)
    ref = requantized(x.numpy()) @ kq.dequantize(type_id, packed, k).astype(np.float64).T
    assert (got[2] == 0).all()
    assert np.abs(got - ref).max() <= 2e-5 * np.abs(ref).max() + 1e-6 * np.abs(ref).max()


def test_agrees_with_the_decode_gemv_within_quantization_noise():
    # the GEMV's Q8_1 activations differ only in how the block sum is stored, so the two kernels agree closely
    type_id, n, k = kq.Q4_K, 2048, 2048
    packed = random_packed(type_id, n, k, seed=3)
    w_dev = ops.upload_weights(packed, DT[type_id])
    x = seeded_acts(8, k, 11, torch.bfloat16).cuda()
    a = ops.gemv_tc(DT[type_id], w_dev, x, n).float()
    b = ops.gemv(DT[type_id], w_dev, x, n).float()
    torch.cuda.synchronize()
    assert_device_ok()
    assert (a - b).abs().max().item() <= 1e-2 * b.abs().max().item()


def test_rows_beyond_m_are_not_written_and_strides_are_honoured():
    type_id, n, k = kq.Q6_K, 300, 2048
    packed = random_packed(type_id, n, k, seed=4)
    w_dev = ops.upload_weights(packed, DT[type_id])
    xbig = seeded_acts(16, k + 64, 5, torch.bfloat16).cuda()
    x = xbig[:5, :k]  # row stride k + 64
    ybig = torch.full((8, n + 20), 7.0, dtype=torch.bfloat16, device="cuda")
    y = ybig[:5, :n]
    ops.gemv_tc(DT[type_id], w_dev, x, n, out=y)
    ref = ops.gemv_tc(DT[type_id], w_dev, x.contiguous(), n)
    torch.cuda.synchronize()
    assert torch.equal(y, ref)
    assert (ybig[5:] == 7.0).all() and (ybig[:, n:] == 7.0).all()
    assert_device_ok()


def test_two_calls_with_one_workspace_give_the_same_result():
    type_id, n, k = kq.Q8_0, 1000, 1024
    packed = random_packed(type_id, n, k, seed=6)
    w_dev = ops.upload_weights(packed, DT[type_id])
    ws = ops.gemv_tc_workspace(DT[type_id], k)
    x1 = seeded_acts(16, k, 1, torch.bfloat16).cuda()
    x2 = seeded_acts(3, k, 2, torch.bfloat16).cuda()
    a1 = ops.gemv_tc(DT[type_id], w_dev, x1, n, workspace=ws)
    a2 = ops.gemv_tc(DT[type_id], w_dev, x2, n, workspace=ws)  # rows 3..15 of the workspace must be rewritten as zeros
    b1 = ops.gemv_tc(DT[type_id], w_dev, x1, n, workspace=ws)
    torch.cuda.synchronize()
    assert torch.equal(a1, b1)
    assert torch.equal(a2, ops.gemv_tc(DT[type_id], w_dev, x2, n))
    assert_device_ok()


@pytest.mark.parametrize("m", [3, 8, 16])
def test_results_do_not_depend_on_timing(m):
    # several warps add up a row's sums: the order is fixed, so repeated launches agree to the last bit, f32 included
    type_id, n, k = kq.Q4_K, 20000, 1024
    w_dev = ops.upload_weights(random_packed(type_id, n, k, seed=12), DT[type_id])
    x = seeded_acts(m, k, 13, torch.float32).cuda()
    first = ops.gemv_tc(DT[type_id], w_dev, x, n)
    for _ in range(5):
        assert torch.equal(ops.gemv_tc(DT[type_id], w_dev, x, n), first)
    assert_device_ok()


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("m,n,k", [(4, 4096, 4096), (16, 1024, 4096), (9, 6144, 2048), (3, 100, 4096)])
def test_matrices_with_few_rows_are_split_along_k(type_id, m, n, k):
    # few row tiles: the 256-k stages of a tile are shared out over several CTAs whose partial outputs are added in a
    # fixed order; same gates, bit-reproducible, and close to the unsplit kernel (different f32 summation order only)
    packed = random_packed(type_id, n, k, seed=n + k)
    y = run_tc(type_id, m, n, k, packed=packed, seed=m)
    w_dev = ops.upload_weights(packed, DT[type_id])
    x = (seeded_acts(m, k, 6000 + m, torch.float32)).to(torch.bfloat16).cuda()
    again = ops.gemv_tc(DT[type_id], w_dev, x, n)
    assert torch.equal(again, y)
    ops.set_option("tc_ksplit", 0)
    try:
        whole = ops.gemv_tc(DT[type_id], w_dev, x, n)
    finally:
        ops.set_option("tc_ksplit", 1)
    torch.cuda.synchronize()
    assert (whole.float() - y.float()).abs().max().item() <= 2.0 ** -7 * y.float().abs().max().item()
    assert_device_ok()


def test_unsupported_inputs_are_refused():
    w_dev = ops.upload_weights(random_packed(kq.Q4_K, 128, 256, 1), DT[kq.Q4_K])
    with pytest.raises(kl.KernelLibraryError, match="at most 16"):
        ops.gemv_tc(DT[kq.Q4_K], w_dev, torch.zeros(17, 256, device="cuda", dtype=torch.bfloat16), 128)
    w6 = ops.upload_weights(random_packed(kq.Q6_K, 64, 256, 1), DT[kq.Q6_K])
    with pytest.raises(kl.KernelLibraryError, match="multiple of 2048"):  # 210-byte rows
        ops.gemv_tc(DT[kq.Q6_K], w6, torch.zeros(4, 256, device="cuda", dtype=torch.bfloat16), 64)
    w8 = ops.upload_weights(random_packed(kq.Q8_0, 64, 96, 1), DT[kq.Q8_0])
    with pytest.raises(kl.KernelLibraryError):
        ops.gemv_tc(DT[kq.Q8_0], w8, torch.zeros(4, 96, device="cuda", dtype=torch.bfloat16), 64)
    ws = torch.empty(64, dtype=torch.uint8, device="cuda")
    with pytest.raises(kl.KernelLibraryError, match="workspace"):
        ops.gemv_tc(DT[kq.Q4_K], w_dev, torch.zeros(4, 256, device="cuda", dtype=torch.bfloat16), 128, workspace=ws)


# ---------------------------------------------------------------------------------------------------------------------
# The reference tier's own pair of launchers: launch_mmvq_tc_quantize_* + launch_mmvq_tc_gguf_{q4_k,q6_k}_*_plain
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,k", [(1, 256), (8, 1024), (9, 512), (16, 4096), (5, 1000)])
def test_reference_activation_layout_is_bit_exact(dtype, rows, k):
    x = seeded_acts(rows, k, 40 + rows, dtype)
    mine = ops.mmvq_tc_quantize(x.cuda()).cpu().numpy()
    torch.cuda.synchronize()
    want = kq.quantize_mmvq_tc(as_f32_numpy(x))
    assert mine.shape == want.shape and np.array_equal(mine, want)
    if rk.available():
        # the reference's build divides approximately (fast-math): scales identical, a quant may sit one step away
        theirs = rk.tc_quantize(x.cuda()).cpu().numpy()
        torch.cuda.synchronize()
        nb = (k + 31) // 32
        for h in range((rows + 7) // 8):
            a, b = mine[h * nb * 288:(h + 1) * nb * 288], theirs[h * nb * 288:(h + 1) * nb * 288]
            assert np.array_equal(a[nb * 256:nb * 272], b[nb * 256:nb * 272]), "scales differ"
            dq = a[:nb * 256].view(np.int8).astype(np.int32) - b[:nb * 256].view(np.int8).astype(np.int32)
            assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 2e-3


def run_tc_ref(type_id, m, n, k, dtype=torch.bfloat16, packed=None, seed=0):
    """quantize + plain through the reference's symbols, with activations built by the ORACLE's layout function as well
    as by the library's quantizer: both must give the tier's arithmetic."""
    if packed is None:
        packed = kq.quantize(type_id, seeded_weights(n, k, 5000 + seed))
    x = seeded_acts(m, k, 6000 + seed, dtype)
    w_dev = ops.upload_weights(packed, DT[type_id])
    vy_oracle = torch.from_numpy(kq.quantize_mmvq_tc(as_f32_numpy(x))).cuda()
    y = ops.mmvq_tc_plain(DT[type_id], w_dev, vy_oracle, n, k, m, dtype)
    y2 = ops.mmvq_tc_plain(DT[type_id], w_dev, ops.mmvq_tc_quantize(x.cuda()), n, k, m, dtype)
    torch.cuda.synchronize()
    assert_device_ok()
    assert torch.equal(y, y2)
    got = as_f32_numpy(y).astype(np.float64)
    ref = requantized(as_f32_numpy(x)) @ kq.dequantize(type_id, packed, k).astype(np.float64).T
    size = np.abs(ref).max()
    bad = np.abs(got - ref) > 2e-5 * size + EPS[dtype] * 1.01 * np.abs(ref)
    assert not bad.any(), f"{kq.TYPE_NAMES[type_id]} m={m} n={n} k={k}: {bad.sum()} outputs off, worst {np.abs(got - ref).max():.3e} vs {size:.3e}"
    cpu = kq.matmul(type_id, as_f32_numpy(x), packed, n)
    assert np.abs(got - cpu).max() <= 1e-3 + (1e-2 if k >= 1024 else 2e-2) * np.abs(cpu).max()
    if rk.available():
        theirs = as_f32_numpy(rk.tc_plain(type_id, w_dev, vy_oracle, n, k, m, dtype)).astype(np.float64)
        torch.cuda.synchronize()
        off = np.abs(got - theirs) > 1e-4 * size + 2 * EPS[dtype] * 1.01 * np.abs(ref)
        assert not off.any(), f"{off.sum()} outputs differ from the reference's kernel on the same scratch"
    return y


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q6_K])
@pytest.mark.parametrize("m,n,k", [(1, 128, 2048), (3, 64, 2048), (8, 1000, 2048), (9, 300, 4096), (16, 148 * 128 + 77, 2048), (12, 9000, 2048)])
def test_reference_launcher_pair(type_id, m, n, k):
    run_tc_ref(type_id, m, n, k, seed=m + n)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_reference_launcher_pair_other_types(dtype):
    run_tc_ref(kq.Q4_K, 7, 512, 1024, dtype=dtype)


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q6_K])
def test_reference_launcher_pair_at_baseline_shapes(type_id):
    for k, n in ((4096, 4096), (14336, 4096)):
        packed = real_packed(type_id, n, k)
        run_tc_ref(type_id, 16, n, k, packed=packed, seed=1)
        run_tc_ref(type_id, 4, n, k, packed=packed, seed=2)


def test_reference_launcher_pair_on_rows_the_tma_path_cannot_take():
    # Q6_K rows of 210 * k / 256 bytes are a multiple of 16 only when k is a multiple of 2048: other k take the plain kernel
    run_tc_ref(kq.Q6_K, 5, 200, 768, seed=3)
    run_tc_ref(kq.Q6_K, 16, 64, 1280, seed=4)
