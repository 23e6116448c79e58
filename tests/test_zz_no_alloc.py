"""The entry point for callers that cannot allocate device memory: `b200q_gemv_static_scratch`.

Such a caller (a serving loop whose device memory all belongs to its own pool, or a thread that must not call
cudaMalloc because that stalls every stream of the device) cannot provide the Q8_1 scratch buffer the two-launch decode
path needs, so the library keeps one inside its own image. The output must equal what the existing pair of launchers
(`launch_mmvq_gguf_quantize_q8_1_*` then `launch_mmvq_gguf_*_plain`) gives with caller-allocated scratch, call after
call, and sizes beyond the fixed array must be refused. This file sorts last so that a stop-at-first-failure run has
already been through every other test.
"""
import pytest
import torch

from oracle import kquants as kq

from inference_rs_b200 import kernel_library as kl
from inference_rs_b200 import ops
from gpu_util import DT, random_packed, seeded_acts

pytestmark = pytest.mark.gpu


def static_gemv(type_id, w_dev, x, n):
    b, k = x.shape
    dst = torch.empty((b, n), dtype=x.dtype, device=x.device)
    rc = kl.library().b200q_gemv_static_scratch(int(DT[type_id]), ops.elem_of(x.dtype), w_dev.data_ptr(), x.data_ptr(),
                                                dst.data_ptr(), k, n, n, b, torch.cuda.current_stream().cuda_stream)
    kl.check(rc, "b200q_gemv_static_scratch")
    return dst


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q6_K, kq.Q8_0])
def test_static_scratch_matches_caller_allocated_scratch_twice(type_id):
    n, k = 1000, 2048
    w_dev = ops.upload_weights(random_packed(type_id, n, k, seed=77), DT[type_id])
    # two calls in a row, the second with fewer rows and other values: it must not see anything of the first
    for b, seed in ((3, 1), (1, 2)):
        x = seeded_acts(b, k, seed, torch.bfloat16).cuda()
        want = ops.mmvq_plain(DT[type_id], w_dev, ops.quantize_q8_1(x), n, k, b, torch.bfloat16)
        got = static_gemv(type_id, w_dev, x, n)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call with {b} rows: static-scratch output differs from the two-launch path"
    assert kl.device_status()[0] == 0


def test_static_scratch_handles_padding_and_f32():
    # K = 768 pads to 1024: the padded blocks are rewritten as zeros on every call
    type_id, n, k = kq.Q6_K, 64, 768
    w_dev = ops.upload_weights(random_packed(type_id, n, k, seed=5), DT[type_id])
    x = seeded_acts(2, k, 9, torch.float32).cuda()
    want = ops.mmvq_plain(DT[type_id], w_dev, ops.quantize_q8_1(x), n, k, 2, torch.float32)
    for _ in range(2):
        assert torch.equal(static_gemv(type_id, w_dev, x, n), want)


def test_sizes_beyond_the_fixed_array_are_refused():
    w_dev = ops.upload_weights(random_packed(kq.Q8_0, 8, 256, seed=1), DT[kq.Q8_0])
    with pytest.raises(kl.KernelLibraryError, match="at most 8 activation rows"):
        static_gemv(kq.Q8_0, w_dev, torch.zeros(9, 256, device="cuda"), 8)
    big_k = 32768 + 512
    w_big = ops.upload_weights(random_packed(kq.Q8_0, 1, big_k, seed=1), DT[kq.Q8_0])
    with pytest.raises(kl.KernelLibraryError, match="32768"):
        static_gemv(kq.Q8_0, w_big, torch.zeros(1, big_k, device="cuda"), 1)
