"""Pins the CPU oracle to the reference.

The known answers are the reference's own: FNV-1a-64 hashes of the packed bytes of its LCG layer in
`IkLlama` mode (crates/inference-quant/src/gguf/requantize.rs:1071-1152, `PINNED_IK`), read from that
file as text. The other checks repeat the reference's CPU property tests against the restatement
(crates/inference-tensor/src/quantized/mod.rs:1654-1685, 1719-1764, 1883-1918) and cross-check the
dequantizers with gguf-py.
"""
import numpy as np
import pytest

from oracle import kquants as kq

# (name, plain, with importance matrix) from PINNED_IK
PINNED_IK = {
    "q4_k": (14679928973253263191, 14544912929349767743),
    "q6_k": (15677125580282521591, 18396251129581993316),
    "q8_0": (11372417339874904451, 11372417339874904451),
}


def test_lcg_layer_shape_and_range():
    vals, imat = kq.pinned_layer()
    assert vals.shape == (8, 512) and imat.shape == (512,)
    assert np.abs(vals).max() <= 0.2 + 1e-6 and imat.min() >= 0.05


@pytest.mark.parametrize("type_id", [kq.Q8_0, kq.Q4_K, kq.Q6_K])
def test_quantizers_write_the_reference_bytes(type_id):
    vals, _ = kq.pinned_layer()
    name = kq.TYPE_NAMES[type_id]
    assert kq.fnv1a64(kq.quantize(type_id, vals, kq.IKLLAMA)) == PINNED_IK[name][0]


def test_q6_k_imatrix_bytes():
    vals, imat = kq.pinned_layer()
    assert kq.fnv1a64(kq.quantize_q6_k_imatrix(vals, imat, kq.IKLLAMA)) == PINNED_IK["q6_k"][1]


def test_q8_0_is_mode_independent():
    vals, _ = kq.pinned_layer()
    assert np.array_equal(kq.quantize(kq.Q8_0, vals, kq.LLAMACPP), kq.quantize(kq.Q8_0, vals, kq.IKLLAMA))


def test_f16_conversion_matches_numpy():
    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5, np.inf, -np.inf], np.float32),
    ]).astype(np.float32)
    got = kq.narrow_f16(x)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)
    allbits = np.arange(65536, dtype=np.uint16)
    back = kq.widen_f16(allbits)
    want_back = allbits.view(np.float16).astype(np.float32)
    ok = (back == want_back) | (np.isnan(back) & np.isnan(want_back))
    assert ok.all()


def test_bf16_conversion_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.005859375, 1.01171875, -3.1415927, 1e-40, 3.3e38], np.float32)
    bits = kq.narrow_bf16(x)
    import torch
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, want)
    assert np.array_equal(kq.widen_bf16(bits), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_block32_quantizer_ties_round_away_from_zero():
    # mod.rs:1654-1685: a block whose max is 127 so values are their own quants, ties at every half
    x = np.array([127.0 if i == 0 else (i - 16.0) + (0.5 if i % 2 == 0 else 0.49999997) for i in range(32)], np.float32)
    packed = kq.quantize(kq.Q8_0, x[None, :])[0]
    assert kq.lib().orc_f16_to_f32(int(packed[:2].view(np.uint16)[0])) == 1.0
    q = packed[2:].view(np.int8)
    want = [127] + [int(np.sign(v) * np.floor(abs(v) + 0.5)) for v in x[1:]]
    assert q.tolist() == want
    z = kq.quantize(kq.Q8_0, np.zeros((1, 32), np.float32))
    assert not z.any()


@pytest.mark.parametrize("type_id", [kq.Q8_0, kq.Q4_K, kq.Q6_K])
def test_rows_quantize_alone_as_in_a_tensor(type_id):
    # mod.rs:1719-1764: many rows at once give the bytes each row gets alone
    rng = np.random.default_rng(7)
    w = rng.standard_normal((33, 512)).astype(np.float32)
    whole = kq.quantize(type_id, w)
    for r in (0, 17, 32):
        assert np.array_equal(whole[r], kq.quantize(type_id, w[r:r + 1])[0])


@pytest.mark.parametrize("type_id", [kq.Q8_0, kq.Q4_K, kq.Q6_K])
def test_dequantize_matches_gguf_py(type_id):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((6, 1024)) * 0.02).astype(np.float32)
    packed = kq.quantize(type_id, w)
    ours = kq.dequantize(type_id, packed, 1024)
    qt = {kq.Q8_0: gguf.GGMLQuantizationType.Q8_0, kq.Q4_K: gguf.GGMLQuantizationType.Q4_K,
          kq.Q6_K: gguf.GGMLQuantizationType.Q6_K}[type_id]
    theirs = quants.dequantize(packed, qt)
    np.testing.assert_allclose(ours, theirs, rtol=1e-6, atol=1e-9)
    # and the round trip stays close to the weights
    err = np.abs(ours - w).max()
    assert err < {kq.Q8_0: 5e-4, kq.Q4_K: 8e-3, kq.Q6_K: 2e-3}[type_id]


def test_q8_0_packing_matches_gguf_py():
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.default_rng(5)
    w = rng.standard_normal((4, 256)).astype(np.float32)
    theirs = quants.quantize(w, gguf.GGMLQuantizationType.Q8_0)
    assert np.array_equal(kq.quantize(kq.Q8_0, w), theirs)


@pytest.mark.parametrize("type_id", [kq.Q8_0, kq.Q4_K, kq.Q6_K])
@pytest.mark.parametrize("m", [1, 3, 9, 33])
def test_quantized_matmul_matches_dequantized_weights(type_id, m):
    # mod.rs:1883-1918: ||err||_2 < 0.02 ||ref||_2 against x @ dequant(W)^T, K=512, N=48
    rng = np.random.default_rng(100 + m)
    w = rng.standard_normal((48, 512)).astype(np.float32)
    x = rng.standard_normal((m, 512)).astype(np.float32)
    packed = kq.quantize(type_id, w)
    got = kq.matmul(type_id, x, packed, 48)
    ref = kq.matmul_dense(type_id, x, packed, 48)
    assert np.linalg.norm(got - ref) < 0.02 * np.linalg.norm(ref)
    # one thread and many give the same bits
    assert np.array_equal(got, kq.matmul(type_id, x, packed, 48, threads=1))


@pytest.mark.parametrize("type_id", [kq.Q8_0, kq.Q4_K, kq.Q6_K])
def test_q8_1_arithmetic_close_to_cpu_path(type_id):
    rng = np.random.default_rng(11)
    k, n = 1024, 40
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((2, k)).astype(np.float32)
    packed = kq.quantize(type_id, w)
    acts = kq.quantize_q8_1_mmvq(x)
    gpu_math = kq.matmul_q8_1(type_id, acts, 2, k, 1024, packed, n)
    cpu = kq.matmul(type_id, x, packed, n)
    assert np.abs(gpu_math - cpu).max() <= 1e-3 + 1e-2 * np.abs(cpu).max()


def test_q8_1_mmvq_blocks():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((3, 700)).astype(np.float32)
    x[1, :32] = 0.0
    acts = kq.quantize_q8_1_mmvq(x).reshape(3, -1, 36)
    assert acts.shape[1] == 1024 // 32
    d = acts[:, :, 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    s = acts[:, :, 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    q = acts[:, :, 4:].view(np.int8).astype(np.float32)
    xp = np.zeros((3, 1024), np.float32)
    xp[:, :700] = x
    xb = xp.reshape(3, -1, 32)
    assert np.abs(q * d[..., None] - xb).max() <= 0.5 * d.max() * 1.01
    np.testing.assert_allclose(s, xb.sum(-1), rtol=2e-3, atol=2e-3)
    assert not acts[1, 0].any() and not acts[:, 22:, :].any()  # zero block, zero padding


def test_q8_1_mmq_layout():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((5, 256)).astype(np.float32)
    for layout in (0, 1):
        blocks = kq.quantize_q8_1_mmq(x, 256, layout)
        assert blocks.shape == (2, 5, 144)
        q = blocks[:, :, 16:].view(np.int8).astype(np.float32).reshape(2, 5, 4, 32)
        if layout == 0:
            d = blocks[:, :, :16].copy().view(np.float32)
        else:
            ds = blocks[:, :, :16].copy().view(np.float16).astype(np.float32).reshape(2, 5, 4, 2)
            d = ds[..., 0]
            np.testing.assert_allclose(ds[..., 1], x.reshape(5, 2, 4, 32).transpose(1, 0, 2, 3).sum(-1), rtol=2e-3, atol=2e-3)
        xr = x.reshape(5, 2, 4, 32).transpose(1, 0, 2, 3)
        assert np.abs(q * d[..., None] - xr).max() <= 0.51 * d.max()
