"""Host logic of the tensor-parallel split (no GPU): shard ranges, packed slicing, and a two-rank gloo run in which each
rank multiplies its shard with the CPU oracle and the partial outputs are sum-all-reduced, as the row-parallel layer
does on GPUs. Follows the reference's own CPU-side TP tests (crates/inference-quant/src/gguf/weight_source.rs:2189-2243,
distributed/layers.rs:3249-3325), which check slicing and bias placement without running a collective."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kquants as kq

from inference_rs_b200 import GgmlDType
from inference_rs_b200.tensor_parallel import Shard, SumAllReduce, compute_kv_shard, shard_range, slice_blocked_data
from inference_rs_b200 import workloads

DT = {kq.Q8_0: GgmlDType.Q8_0, kq.Q4_K: GgmlDType.Q4K, kq.Q6_K: GgmlDType.Q6K}


def test_shard_range_matches_the_reference_rules():
    assert shard_range(Shard.simple(0, 0, 1), (8, 512)) is None
    assert shard_range(Shard.simple(0, 1, 2), (8, 512)) == (0, 4, 4)
    assert shard_range(Shard.simple(1, 3, 4), (8, 1024)) == (1, 768, 256)
    assert shard_range(Shard.at(0, 0, 8), (8, 512)) is None
    assert shard_range(Shard.at(1, 256, 256), (8, 512)) == (1, 256, 256)
    with pytest.raises(ValueError, match="not divisible by world size 3"):
        shard_range(Shard.simple(0, 0, 3), (8, 512))
    with pytest.raises(ValueError, match="outside world size"):
        shard_range(Shard.simple(0, 2, 2), (8, 512))
    with pytest.raises(ValueError, match="exceeds dimension"):
        shard_range(Shard.at(1, 300, 300), (8, 512))
    with pytest.raises(ValueError, match="Cannot shard dimension 2"):
        shard_range(Shard.simple(2, 0, 2), (8, 512))


@pytest.mark.parametrize("type_id", [kq.Q8_0, kq.Q4_K, kq.Q6_K])
def test_packed_shards_equal_quantizing_the_slices(type_id):
    rng = np.random.default_rng(1)
    n, k = 16, 1024
    w = rng.standard_normal((n, k)).astype(np.float32)
    packed = kq.quantize(type_id, w)
    dt = DT[type_id]
    # output-dimension shard = whole rows
    rows = slice_blocked_data(packed, (n, k), dt.block_size, dt.type_size, 0, 4, 8)
    assert np.array_equal(rows.reshape(8, -1), packed[4:12])
    # input-dimension shard = whole blocks of every row, contiguous; blocks are self-contained, so it equals quantizing
    # the column slice on its own
    cols = slice_blocked_data(packed, (n, k), dt.block_size, dt.type_size, 1, 512, 256)
    assert np.array_equal(cols.reshape(n, -1), kq.quantize(type_id, w[:, 512:768]))
    assert cols.size == n * dt.row_bytes(256)
    with pytest.raises(ValueError, match="block alignment"):
        slice_blocked_data(packed, (n, k), dt.block_size, dt.type_size, 1, 16, 256)
    with pytest.raises(ValueError, match="exceeds dimension"):
        slice_blocked_data(packed, (n, k), dt.block_size, dt.type_size, 0, 10, 10)


def test_kv_head_shards():
    assert compute_kv_shard(8, 128, 3, 8) == Shard.simple(0, 3, 8)
    assert compute_kv_shard(8, 128, 1, 2) == Shard.simple(0, 1, 2)
    # 2 KV heads over 8 ranks: each head replicated on 4 ranks
    assert compute_kv_shard(2, 128, 5, 8) == Shard.at(0, 128, 128)
    assert compute_kv_shard(8, 128, 0, 1) == Shard.simple(0, 0, 1)


def test_70b_projections_shard_in_whole_superblocks():
    for world in (2, 4, 8):
        for p in workloads.LLAMA3_70B.layer_projections():
            s = workloads.shard(p, world)
            assert s.k % p.dtype.block_size == 0
            assert s.weight_bytes * world == p.weight_bytes


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _row_parallel_rank(rank, world, port, type_id, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)  # same data on every rank
        n, k = 24, 1024
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        x = rng.standard_normal((3, k)).astype(np.float32)
        packed = kq.quantize(type_id, w)
        dt = DT[type_id]
        _, start, length = shard_range(Shard.simple(1, rank, world), (n, k))
        mine = slice_blocked_data(packed, (n, k), dt.block_size, dt.type_size, 1, start, length)
        partial = kq.matmul(type_id, x[:, start:start + length], mine, n)
        total = SumAllReduce().sum_all_reduce(torch.from_numpy(partial))
        full = kq.matmul(type_id, x, packed, n)
        ret[rank] = float(np.abs(total.numpy() - full).max() / np.abs(full).max())
        # a non-contiguous partial is refused, as in the reference
        try:
            SumAllReduce().sum_all_reduce(torch.from_numpy(partial).t())
            ret[rank + world] = "no error"
        except ValueError:
            ret[rank + world] = "refused"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("type_id", [kq.Q4_K, kq.Q8_0])
def test_row_parallel_partials_sum_to_the_full_matmul_over_gloo(type_id):
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_row_parallel_rank, args=(world, port, type_id, ret), nprocs=world, join=True)
        for r in range(world):
            assert ret[r] < 1e-5, ret[r]
            assert ret[r + world] == "refused"
