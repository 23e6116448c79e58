"""The fused decode launchers (launch_mmvq_gguf_<type>_<elem>_fused_glu / _fused_qkv) against three references on the
same Q8_1 activation blocks: the CPU oracle's integer matmul with the epilogue restated in torch on the host, this
library's plain launchers followed by the same epilogue, and the reference's own fused CUDA kernels (oracle/_ref).

Rounding order of the gated epilogue (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:829-836): gate and up
are rounded to the output type, the activation is evaluated in f32 on the rounded gate and rounded, and the product is
formed in the output type. Outputs that went through those three roundings are compared within two spacings of the
output type (one rounding boundary apart on either side).
"""
import numpy as np
import pytest
import torch

from oracle import kquants as kq
from oracle import refkernels as rk

from inference_rs_b200 import ops
from gpu_util import DT, TYPES, random_packed, real_packed, seeded_acts, seeded_weights, assert_device_ok

pytestmark = pytest.mark.gpu

EPS = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -23}


def epilogue(gate: torch.Tensor, up: torch.Tensor, activation: str, dtype: torch.dtype) -> torch.Tensor:
    """act(gate) * up with the reference's rounding order; gate / up f32 or already of `dtype`."""
    g = gate.to(dtype).float()
    u = up.to(dtype)
    if activation == "silu":
        a = g / (1.0 + torch.exp(-g))
    elif activation == "gelu":
        a = 0.5 * g * (1.0 + torch.tanh(0.7978845608 * (g + 0.044715 * g * g * g)))
    elif activation == "relu":
        a = torch.clamp(g, min=0.0)
    elif activation == "gelu_erf":
        a = g * 0.5 * (1.0 + torch.erf(g * 0.7071067811865476))
    else:
        a = 1.0 / (1.0 + torch.exp(-g))
    return a.to(dtype) * u


def close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, scale: float = 2.0, floor: float = 4e-6):
    """|got - want| within `scale` spacings of the larger magnitude; outputs that are small through cancellation carry the
    f32 summation-order difference of the dot products, `floor` of the largest output."""
    g, w = got.float().cpu(), want.float().cpu()
    tol = scale * 2 * EPS[dtype] * torch.maximum(g.abs(), w.abs()) + floor * float(w.abs().max()) + 1e-6
    bad = (g - w).abs() > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} differ; worst {float(((g - w).abs() - tol).max()):.3e} over tolerance"


def weights_for(type_id, n, k, real):
    return real_packed(type_id, n, k) if real else random_packed(type_id, n, k, n + k)


GLU_SHAPES = [
    # k, n, real weights
    (4096, 14336, True),    # llama3-8b ffn_gate / ffn_up
    (512, 77, True),        # ragged rows: the plain fallback and the tail of the ring
    (8192, 28672, False),   # llama3-70b ffn: several warps per row for the K-quants
    (14336, 200, True),     # long rows, few of them
]


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("k,n,real", GLU_SHAPES)
@pytest.mark.parametrize("b", [1, 2, 5, 8])
def test_fused_glu_equals_plain_launches_and_epilogue(type_id, k, n, real, b):
    dtype = torch.bfloat16
    if real and n >= 14336:
        gate_np, up_np = real_packed(type_id, n, k), real_packed(type_id, n, k)[::-1].copy()
    else:
        gate_np, up_np = weights_for(type_id, n, k, real), weights_for(type_id, n + 1, k, real)[1:]
    wg, wu = ops.upload_weights(gate_np, DT[type_id]), ops.upload_weights(up_np, DT[type_id])
    x = seeded_acts(b, k, 3 * b + n, dtype).cuda()
    vy = ops.quantize_q8_1(x)
    got = ops.mmvq_fused_glu(DT[type_id], wg, wu, vy, n, k, b, dtype)
    g = ops.mmvq_plain(DT[type_id], wg, vy, n, k, b, torch.float32)
    u = ops.mmvq_plain(DT[type_id], wu, vy, n, k, b, torch.float32)
    torch.cuda.synchronize()
    assert_device_ok()
    close(got, epilogue(g, u, "silu", dtype), dtype, scale=3.0 if dtype != torch.float32 else 64.0)


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("activation", ["silu", "gelu", "relu", "gelu_erf", "sigmoid"])
def test_fused_glu_against_the_oracle(type_id, dtype, activation):
    k, n, b = 1024, 301, 3
    gate_np = kq.quantize(type_id, seeded_weights(n, k, 21))
    up_np = kq.quantize(type_id, seeded_weights(n, k, 22))
    # activations large enough that the gate leaves the linear part of every activation function
    x = (seeded_acts(b, k, 23, torch.float32) * 4.0).to(dtype)
    k_padded = 1024
    acts = kq.quantize_q8_1_mmvq(x.float().numpy(), k_padded)
    g = torch.from_numpy(kq.matmul_q8_1(type_id, acts, b, k, k_padded, gate_np, n))
    u = torch.from_numpy(kq.matmul_q8_1(type_id, acts, b, k, k_padded, up_np, n))
    want = epilogue(g, u, activation, dtype)
    wg, wu = ops.upload_weights(gate_np, DT[type_id]), ops.upload_weights(up_np, DT[type_id])
    vy = ops.quantize_q8_1(x.cuda())
    assert np.array_equal(vy.cpu().numpy().reshape(-1)[: acts.size], acts.reshape(-1))
    got = ops.mmvq_fused_glu(DT[type_id], wg, wu, vy, n, k, b, dtype, activation)
    torch.cuda.synchronize()
    assert_device_ok()
    # f32 outputs carry the summation-order difference of the dot products (1e-5 of the products' size)
    close(got, want, dtype, scale=2.0 if dtype != torch.float32 else 64.0)


@pytest.mark.skipif(not rk.available(), reason="oracle/_ref was not built (no reference checkout)")
@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("b", [1, 4, 8])
@pytest.mark.parametrize("activation", ["silu", "gelu"])
def test_fused_glu_against_the_reference_kernel(type_id, b, activation):
    k, n, dtype = 4096, 14336, torch.bfloat16
    gate_np, up_np = real_packed(type_id, n, k), real_packed(type_id, n, k)[::-1].copy()
    wg, wu = ops.upload_weights(gate_np, DT[type_id]), ops.upload_weights(up_np, DT[type_id])
    x = seeded_acts(b, k, 40 + b, dtype).cuda()
    vy = ops.quantize_q8_1(x)
    theirs = rk.fused_glu(type_id, wg, wu, x, n, activation, vy=vy)
    got = ops.mmvq_fused_glu(DT[type_id], wg, wu, vy, n, k, b, dtype, activation)
    torch.cuda.synchronize()
    assert_device_ok()
    # the reference's build evaluates exp and tanh approximately (fast-math): one more spacing. Its Q4_K min term uses
    # the block sums as Q8_1 stores them (f16), this library's the integer sums: 4e-5 of the largest dot product, as in
    # the plain matvec's comparison, which the epilogue carries into the product
    close(got, theirs, dtype, scale=3.0, floor=2e-4)


QKV_SHAPES = [
    # k, nq, nk, nv
    (4096, 4096, 1024, 1024),    # llama3-8b attention
    (8192, 8192, 1024, 1024),    # llama3-70b attention
    (512, 100, 36, 7),           # ragged
]


@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("k,nq,nk,nv", QKV_SHAPES)
@pytest.mark.parametrize("b", [1, 3, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_qkv_equals_three_plain_launches(type_id, k, nq, nk, nv, b, dtype):
    packed = [random_packed(type_id, n, k, 7 * i + n) if k >= 4096 else kq.quantize(type_id, seeded_weights(n, k, 50 + i))
              for i, n in enumerate((nq, nk, nv))]
    ws = [ops.upload_weights(p, DT[type_id]) for p in packed]
    x = seeded_acts(b, k, 60 + b, dtype).cuda()
    vy = ops.quantize_q8_1(x)
    outs = ops.mmvq_fused_qkv(DT[type_id], ws[0], ws[1], ws[2], vy, nq, nk, nv, k, b, dtype)
    torch.cuda.synchronize()
    assert_device_ok()
    for w, n, out in zip(ws, (nq, nk, nv), outs):
        plain = ops.mmvq_plain(DT[type_id], w, vy, n, k, b, dtype)
        assert out.shape == (b, n)
        close(out, plain, dtype, scale=1.0 if dtype != torch.float32 else 64.0)


@pytest.mark.parametrize("type_id", TYPES)
def test_fused_qkv_against_the_oracle(type_id):
    k, ns, b, dtype = 768, (96, 40, 33), 2, torch.float32
    packed = [kq.quantize(type_id, seeded_weights(n, k, 70 + i)) for i, n in enumerate(ns)]
    x = seeded_acts(b, k, 71, dtype)
    k_padded = 1024
    acts = kq.quantize_q8_1_mmvq(x.numpy(), k_padded)
    ws = [ops.upload_weights(p, DT[type_id]) for p in packed]
    outs = ops.mmvq_fused_qkv(DT[type_id], ws[0], ws[1], ws[2], ops.quantize_q8_1(x.cuda()), *ns, k, b, dtype)
    torch.cuda.synchronize()
    assert_device_ok()
    for p, n, out in zip(packed, ns, outs):
        want = kq.matmul_q8_1(type_id, acts, b, k, k_padded, p, n)
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-4, atol=1e-5)


@pytest.mark.skipif(not rk.available(), reason="oracle/_ref was not built (no reference checkout)")
@pytest.mark.parametrize("type_id", TYPES)
@pytest.mark.parametrize("b", [1, 8])
def test_fused_qkv_against_the_reference_kernel(type_id, b):
    k, ns, dtype = 4096, (4096, 1024, 1024), torch.bfloat16
    ws = [ops.upload_weights(random_packed(type_id, n, k, 80 + i), DT[type_id]) for i, n in enumerate(ns)]
    x = seeded_acts(b, k, 81 + b, dtype).cuda()
    vy = ops.quantize_q8_1(x)
    theirs = rk.fused_qkv(type_id, ws[0], ws[1], ws[2], x, *ns, vy=vy)
    outs = ops.mmvq_fused_qkv(DT[type_id], ws[0], ws[1], ws[2], vy, *ns, k, b, dtype)
    torch.cuda.synchronize()
    assert_device_ok()
    for mine, ref in zip(outs, theirs):
        close(mine, ref, dtype, scale=1.0, floor=4e-5)
