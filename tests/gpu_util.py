"""Helpers shared by the GPU parity tests: seeded inputs, oracle calls, tolerances."""
from __future__ import annotations

import numpy as np
import torch

from oracle import kquants as kq

import inference_rs_b200 as pkg
from inference_rs_b200 import ops

DT = {kq.Q8_0: pkg.GgmlDType.Q8_0, kq.Q4_K: pkg.GgmlDType.Q4K, kq.Q6_K: pkg.GgmlDType.Q6K}
TYPES = [kq.Q4_K, kq.Q6_K, kq.Q8_0]
TORCH_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def seeded_weights(n: int, k: int, seed: int) -> np.ndarray:
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, k, generator=g) * 0.02).numpy()


def seeded_acts(m: int, k: int, seed: int, dtype: torch.dtype) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(m, k, generator=g).to(dtype)


def as_f32_numpy(x: torch.Tensor) -> np.ndarray:
    return x.detach().float().cpu().numpy()


def random_packed(type_id: int, n: int, k: int, seed: int) -> np.ndarray:
    """Random but well-formed blocks (random quants and sub-scales, scales of the size N(0, 0.02) weights give):
    lets full-size shapes be tested without running the quantizer over hundreds of millions of weights."""
    rng = np.random.default_rng(seed)
    nb = n * (k // kq.BLOCK_ELEMS[type_id])
    bb = kq.BLOCK_BYTES[type_id]
    raw = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    if type_id == kq.Q8_0:
        d = (rng.uniform(2e-4, 6e-4, nb)).astype(np.float16)
        raw[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    elif type_id == kq.Q4_K:
        d = (rng.uniform(5e-5, 2e-4, nb)).astype(np.float16)
        dm = (rng.uniform(5e-5, 2e-4, nb)).astype(np.float16)
        raw[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        raw[:, 2:4] = dm.view(np.uint8).reshape(nb, 2)
    else:
        d = (rng.uniform(-3e-5, 3e-5, nb)).astype(np.float16)
        raw[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
    return raw.reshape(n, -1)


def elementwise_pass_rate(got: np.ndarray, ref: np.ndarray, rtol=1e-2, atol=1e-3) -> float:
    return float((np.abs(got - ref) <= atol + rtol * np.abs(ref)).mean())


def assert_device_ok():
    from inference_rs_b200 import kernel_library as kl
    torch.cuda.synchronize()
    st = kl.device_status()
    assert st[0] == 0, f"device status word reports a failed wait: {st}"
