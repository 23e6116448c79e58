"""The library's launchers beside the reference's own CUDA kernels (oracle/_ref: compiled for sm_100a from the reference
checkout by oracle/build_ref.py, with the reference's flags, fast-math included) on the same device buffers.

The matmul comparisons live with each kernel's parity tests (test_gpu_gemv.py, test_gpu_gemv_tc.py, test_gpu_gemm.py);
here: the activation quantizers. The reference's build uses approximate division, so a quant that sits on a rounding
boundary may come out one step away from the IEEE result the oracle and this library compute; scales must be identical.
"""
import numpy as np
import pytest
import torch

from oracle import refkernels as rk

from inference_rs_b200 import ops
from gpu_util import seeded_acts

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not rk.available(), reason="oracle/_ref was not built (no reference checkout)")]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,k", [(1, 4096), (8, 14336), (3, 544)])
def test_q8_1_blocks_match_the_reference_quantizer(dtype, rows, k):
    x = seeded_acts(rows, k, 11 + rows, dtype).cuda()
    mine = ops.quantize_q8_1(x).cpu().numpy().reshape(rows, -1, 36)
    theirs = rk.quantize_q8_1(x).cpu().numpy().reshape(rows, -1, 36)
    torch.cuda.synchronize()
    assert mine.shape == theirs.shape
    assert np.array_equal(mine[:, :, 0:2], theirs[:, :, 0:2]), "block scales differ"
    dq = mine[:, :, 4:].view(np.int8).astype(np.int32) - theirs[:, :, 4:].view(np.int8).astype(np.int32)
    assert np.abs(dq).max() <= 1
    assert (dq != 0).mean() < 2e-3, f"{(dq != 0).mean():.2e} of the quants differ"
    # the stored sum is half(sum(x)), from the same values on both sides
    sm = mine[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    st = theirs[:, :, 2:4].copy().view(np.float16).astype(np.float32)
    np.testing.assert_allclose(sm, st, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("layout", ["D4", "DS4"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_prefill_blocks_match_the_reference_quantizer(layout, dtype):
    rows, k = 37, 1024
    x = seeded_acts(rows, k, 5, dtype).cuda()
    mine = ops.quantize_mmq_q8_1(x, layout).cpu().numpy().reshape(-1, 144)
    theirs = rk.mmq_quantize(x, layout).cpu().numpy()[: mine.size].reshape(-1, 144)
    torch.cuda.synchronize()
    assert np.array_equal(mine[:, :16], theirs[:, :16]) or np.allclose(
        mine[:, :16].copy().view(np.float32 if layout == "D4" else np.float16).astype(np.float32),
        theirs[:, :16].copy().view(np.float32 if layout == "D4" else np.float16).astype(np.float32), rtol=2e-3, atol=1e-6)
    dq = mine[:, 16:].view(np.int8).astype(np.int32) - theirs[:, 16:].view(np.int8).astype(np.int32)
    assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 2e-3
