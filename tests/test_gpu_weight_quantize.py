"""GPU parity of the weight quantizers, dequantizers and the row gather (`b200q_quantize`, `b200q_dequantize`,
`b200q_get_rows`), through the C ABI: packed bytes identical to the oracle's (the reference CPU quantizer's default mode),
dequantized values identical to the oracle's `to_float`, and, for the two types the reference has device quantizers for,
identical to those (oracle/_ref) as well."""
import numpy as np
import pytest
import torch

from oracle import kquants as kq
from oracle import refkernels as rk

from inference_rs_b200 import QMatMul, QTensor, ops
from gpu_util import DT, TYPES, as_f32_numpy, assert_device_ok, seeded_acts, seeded_weights

pytestmark = pytest.mark.gpu


def edge_rows(k):
    """Rows the searches treat specially: zeros, one spike, constants of either sign, tiny and huge magnitudes, ties."""
    rng = np.random.default_rng(3)
    rows = [np.zeros(k), np.full(k, 0.25), np.full(k, -0.25), rng.standard_normal(k) * 1e-20, rng.standard_normal(k) * 1e4,
            np.where(np.arange(k) % 256 == 7, 3.0, 0.0), np.arange(k) % 16 - 7.5, rng.standard_normal(k) * 0.02,
            np.abs(rng.standard_normal(k)) * 0.02, -np.abs(rng.standard_normal(k)) * 0.02]
    return np.stack(rows).astype(np.float32)


@pytest.mark.parametrize("type_id", TYPES)
def test_packed_bytes_equal_the_oracle(type_id):
    for w in (seeded_weights(512, 1024, 11), edge_rows(1024), seeded_weights(3, 256, 12) * 50.0):
        mine = ops.quantize_weights(torch.from_numpy(w).cuda(), DT[type_id])
        torch.cuda.synchronize()
        want = kq.quantize(type_id, w).reshape(-1)
        got = mine.cpu().numpy()[: want.size]
        bad = np.nonzero(got != want)[0]
        if bad.size:
            blk, bb = bad[0] // kq.BLOCK_BYTES[type_id], kq.BLOCK_BYTES[type_id]
            raise AssertionError(f"{kq.TYPE_NAMES[type_id]}: {bad.size} bytes differ, first at {bad[:8].tolist()}; block {blk}: got "
                                 f"{got[blk * bb:(blk + 1) * bb].tolist()} want {want[blk * bb:(blk + 1) * bb].tolist()}")
        assert not mine.cpu().numpy()[want.size:].any(), "the padding behind the blocks must be zero"
    assert_device_ok()


@pytest.mark.parametrize("type_id", TYPES)
def test_config_1_weights_quantized_by_the_library(type_id):
    """BASELINE config 1: f32 4096 x 4096 ~N(0, 0.02), seed 0, packed by the product's own quantizer; the bytes equal the
    oracle's and the matmul on them is within the stated tolerance of the CPU path."""
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(4096, 4096, generator=g) * 0.02)
    q = QTensor.quantize(w.cuda(), DT[type_id])
    torch.cuda.synchronize()
    want = kq.quantize(type_id, w.numpy())
    assert np.array_equal(q.packed_bytes().cpu().numpy(), want.reshape(-1))
    x = seeded_acts(4, 4096, 1, torch.float32)
    y = QMatMul.from_qtensor(q).forward(x.cuda(), act_quant=ops.ACT_QUANT_CPU)
    cpu = kq.matmul(type_id, x.numpy(), want, 4096)
    assert (np.abs(as_f32_numpy(y) - cpu) <= 1e-3 + 1e-2 * np.abs(cpu)).all()
    assert_device_ok()


@pytest.mark.parametrize("type_id", [kq.Q6_K, kq.Q8_0])
def test_packed_bytes_equal_the_reference_device_quantizers(type_id):
    if not rk.available():
        pytest.skip("oracle/_ref was not built")
    w = torch.from_numpy(seeded_weights(300, 2048, 13)).cuda()
    mine = ops.quantize_weights(w, DT[type_id])
    theirs, _ = (rk.encode_q6_k if type_id == kq.Q6_K else rk.encode_q8_0)(w)
    torch.cuda.synchronize()
    if type_id == kq.Q8_0:
        assert torch.equal(mine[: theirs.numel()], theirs.reshape(-1))
    else:
        # the reference's device Q6_K quantizer follows its fused-multiply-add mode (Quantizer::IkLlama), this library's the
        # default one: theirs must equal the oracle in that mode, this library's the oracle in the default mode
        assert np.array_equal(theirs.cpu().numpy().reshape(-1), kq.quantize(type_id, w.cpu().numpy(), mode=kq.IKLLAMA).reshape(-1))
        assert np.array_equal(mine.cpu().numpy()[: theirs.numel()], kq.quantize(type_id, w.cpu().numpy()).reshape(-1))


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_dequantize_and_row_gather(type_id, dtype):
    n, k = 257, 768
    packed = kq.quantize(type_id, seeded_weights(n, k, 14))
    q = QTensor.from_packed(packed, DT[type_id], (n, k))
    want = torch.from_numpy(kq.dequantize(type_id, packed, k)).to(dtype)
    got = q.dequantize(dtype)
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), want)
    ids = torch.tensor([[0, 256, 5], [5, 17, 255]], dtype=torch.int64)
    rows = q.embedding(ids, dtype)
    torch.cuda.synchronize()
    assert rows.shape == (2, 3, k) and torch.equal(rows.cpu(), want[ids])
    assert_device_ok()


def test_quantize_errors_and_bad_row_ids():
    from inference_rs_b200 import kernel_library as kl
    with pytest.raises(ValueError, match="not a multiple"):
        QTensor.quantize(torch.zeros(4, 100), DT[kq.Q4_K])
    with pytest.raises(TypeError):
        ops.quantize_weights(torch.zeros(4, 256, dtype=torch.float16, device="cuda"), DT[kq.Q4_K])
    q = QTensor.quantize(torch.from_numpy(seeded_weights(8, 256, 1)).cuda(), DT[kq.Q8_0])
    rows = q.embedding(torch.tensor([1, 99]))
    torch.cuda.synchronize()
    assert not rows[1].any() and rows[0].any()
    st = kl.device_status()
    assert st[0] == 6 and st[2] == 1, st  # code 6: row id outside the table; detail = position of the id
    kl.check(kl.library().b200q_reset_device_status(), "reset")
