"""Tensor parallelism of the quantized matmul path, mirroring the reference:

* `Shard`, `shard_range`, `slice_blocked_data` (crates/inference-quant/src/uqff/mod.rs:111-163,226-320): a shard of
  packed data along the output dimension keeps whole rows; along the input dimension it keeps whole blocks and each
  row's byte sub-range is copied into a new contiguous buffer;
* `ColumnParallelLayer` / `RowParallelLayer` / `ReplicatedLayer` (crates/inference-quant/src/distributed/layers.rs:
  814-1190,1193-1700,1708): column-parallel splits the output rows (bias sharded with them), row-parallel splits the
  input columns and sum-all-reduces the partial outputs before the bias is added once;
* `SumAllReduce` (crates/inference-quant/src/distributed/mod.rs:392-458,516-670): an out-of-place sum all-reduce of the
  `[batch, hidden]` partial outputs in the activation type, here `torch.distributed.all_reduce` (NCCL over NVLink on
  GPUs, gloo on CPU ranks).

One process per GPU; rank = CUDA ordinal, as the reference requires (distributed/mod.rs:262-271).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from .dtypes import GgmlDType
from .qmatmul import GgufMatMul, QTensor


@dataclass(frozen=True)
class Shard:
    """`Shard::Simple {dim, rank, world_size}` or, with `offset`/`length`, `Shard::Offset {dim, offset, len}`."""
    dim: int
    rank: int = 0
    world_size: int = 1
    offset: int | None = None
    length: int | None = None

    @classmethod
    def simple(cls, dim: int, rank: int, world_size: int) -> "Shard":
        return cls(dim=dim, rank=rank, world_size=world_size)

    @classmethod
    def at(cls, dim: int, offset: int, length: int) -> "Shard":
        return cls(dim=dim, offset=offset, length=length)


def shard_range(shard: Shard, dims: tuple[int, ...]):
    """None for a full load, else (dim, start, len); errors as the reference's (uqff/mod.rs:111-163)."""
    if shard.dim >= len(dims):
        raise ValueError(f"Cannot shard dimension {shard.dim} of rank-{len(dims)} tensor.")
    size = dims[shard.dim]
    if shard.offset is not None:
        end = shard.offset + shard.length
        if end > size:
            raise ValueError(f"Shard range {shard.offset}..{end} exceeds dimension {shard.dim} of size {size}.")
        if shard.offset == 0 and shard.length == size:
            return None
        return shard.dim, shard.offset, shard.length
    if shard.world_size == 0:
        raise ValueError("Shard world size must be non-zero.")
    if shard.rank >= shard.world_size:
        raise ValueError(f"Shard rank {shard.rank} is outside world size {shard.world_size}.")
    if shard.world_size == 1:
        return None
    if size % shard.world_size:
        raise ValueError(f"Weight shard dim {shard.dim} of size {size} is not divisible by world size {shard.world_size}.")
    length = size // shard.world_size
    return shard.dim, shard.rank * length, length


def slice_blocked_data(data: np.ndarray, dims: tuple[int, int], block: int, block_bytes: int, dim: int, start: int,
                       length: int) -> np.ndarray:
    """The bytes of `[start, start + length)` along `dim` of packed `[rows, cols]` data, contiguous
    (uqff/mod.rs:226-320, two-dimensional case)."""
    if block == 0 or block_bytes == 0:
        raise ValueError("Packed block sizes must be non-zero.")
    rows, last = dims
    size = dims[dim]
    if start + length > size:
        raise ValueError(f"Packed shard range {start}..{start + length} exceeds dimension {dim} of size {size}.")
    if last % block:
        raise ValueError(f"Cannot shard block-quantized data: last dim {last} is not a multiple of block size {block}.")
    row_bytes = last // block * block_bytes
    data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    if data.size < rows * row_bytes:
        raise ValueError(f"Packed tensor needs {rows * row_bytes} bytes for shape {list(dims)}, but only {data.size} are available.")
    mat = data[: rows * row_bytes].reshape(rows, row_bytes)
    if dim == 1:
        if start % block or length % block:
            raise ValueError(f"Sharding the packed dim requires block alignment: start {start}, len {length}, block {block}.")
        off, sub = start // block * block_bytes, length // block * block_bytes
        return np.ascontiguousarray(mat[:, off:off + sub]).reshape(-1)
    return np.ascontiguousarray(mat[start:start + length]).reshape(-1)


def load_linear_shard(packed: np.ndarray, dtype: GgmlDType, shape: tuple[int, int], shard: Shard, device="cuda") -> QTensor:
    """`GgufWeightSource::load_linear(key, device, shard)` for bytes already in memory
    (crates/inference-quant/src/gguf/weight_source.rs:627-669,877-908): shard first, then upload."""
    rng = shard_range(shard, shape)
    if rng is None:
        return QTensor.from_packed(packed, dtype, shape, device)
    dim, start, length = rng
    sub = slice_blocked_data(packed, shape, dtype.block_size, dtype.type_size, dim, start, length)
    new_shape = (length, shape[1]) if dim == 0 else (shape[0], length)
    return QTensor.from_packed(sub, dtype, new_shape, device)


class SumAllReduce:
    """Sum of the ranks' partial outputs; contiguous inputs only, as the reference's CUDA op (distributed/mod.rs:516-670)."""

    def __init__(self, group=None):
        self.group = group

    def world_size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def sum_all_reduce(self, xs: torch.Tensor) -> torch.Tensor:
        if self.world_size() == 1:
            return xs
        if not xs.is_contiguous():
            raise ValueError("sum_all_reduce expects a contiguous tensor")
        out = xs.clone()  # out of place, like the reference's all_reduce(src, &mut dst)
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out


class PeerSumAllReduce(SumAllReduce):
    """`SumAllReduce` through `b200q_peer_allreduce`: one small kernel per call over NVLink peer memory instead of an
    NCCL collective, for the latency-bound `[rows, hidden]` sums of decode. The exchange buffers come from torch's
    symmetric memory (one allocation per rank, mapped into every rank of the group); vectors larger than `capacity`
    bytes fall through to NCCL. All ranks must make the same calls in the same order."""

    def __init__(self, group=None, capacity: int = 1 << 20, device=None):
        super().__init__(group)
        import ctypes
        import os

        # plain peer mappings are all this needs; no NVLink multicast object is bound to the buffer
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        from . import kernel_library as kl
        self._kl = kl
        self.capacity = (capacity + 15) & ~15
        pg = group if group is not None else dist.group.WORLD
        nbytes = int(kl.library().b200q_peer_allreduce_buffer_bytes(self.capacity))
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, pg)
        self.buffer.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=pg)  # nobody signals before everybody's flags are zero
        self.rank, self.world = int(self.handle.rank), int(self.handle.world_size)
        if self.world > 8:
            raise ValueError("b200q_peer_allreduce takes at most 8 ranks")
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)

    def sum_all_reduce(self, xs: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return xs
        if not xs.is_contiguous():
            raise ValueError("sum_all_reduce expects a contiguous tensor")
        nbytes = xs.numel() * xs.element_size()
        # which collective runs is decided from what every rank shares (size and type), never from a rank's own
        # addresses: ranks that disagreed would wait for each other in two different exchanges
        if nbytes > self.capacity or nbytes % 16 or xs.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            return super().sum_all_reduce(xs)
        from .ops import _stream, elem_of
        if xs.data_ptr() % 16:
            xs = xs.clone()  # torch allocations are aligned
        out = torch.empty_like(xs)
        self._kl.check(self._kl.library().b200q_peer_allreduce(self._ptrs, self.rank, self.world, self.capacity, elem_of(xs.dtype),
                                                               xs.data_ptr(), out.data_ptr(), xs.numel(), _stream()),
                       "b200q_peer_allreduce")
        return out

    def check_status(self) -> None:
        """Raises if a kernel on this device recorded a failed wait (a peer that never arrived leaves the output
        unwritten and only the device status word says so). Synchronizes the device: not for captured steps."""
        st = self._kl.device_status()
        if st[0] != 0:
            raise self._kl.KernelLibraryError(f"device status word reports a failed wait: code {st[0]}, block {st[1]}, detail {st[2]}, "
                                              f"{st[3]} failures")

    def gemv_sum(self, dtype: GgmlDType, w: torch.Tensor, x: torch.Tensor, n: int, out: torch.Tensor | None = None) -> torch.Tensor:
        """`b200q_gemv_allreduce`: this rank's row-parallel matmul (x `[rows <= 8, k / w]` contiguous) and the sum over
        the ranks in one launch. Raises `KernelLibraryError` where the fused launch does not apply (shape, alignment,
        capacity): callers then use `ops.gemv` + `sum_all_reduce_`."""
        from .ops import _stream, elem_of
        rows, k = x.shape
        y = torch.empty((rows, n), dtype=x.dtype, device=x.device) if out is None else out
        self._kl.check(self._kl.library().b200q_gemv_allreduce(int(dtype), elem_of(x.dtype), w.data_ptr(), x.data_ptr(), y.data_ptr(), k, n,
                                                               rows, self._ptrs, self.rank, self.world, self.capacity, _stream()),
                       "b200q_gemv_allreduce")
        return y

    def sum_all_reduce_(self, xs: torch.Tensor) -> torch.Tensor:
        """In place (no allocation: for captured decode steps)."""
        from .ops import _stream, elem_of
        self._kl.check(self._kl.library().b200q_peer_allreduce(self._ptrs, self.rank, self.world, self.capacity, elem_of(xs.dtype),
                                                               xs.data_ptr(), xs.data_ptr(), xs.numel(), _stream()),
                       "b200q_peer_allreduce")
        return xs


class ColumnParallelLayer:
    """Output rows `[rank * n / w, (rank + 1) * n / w)` of the weight; the bias is sharded with them (layers.rs:1193-1700)."""

    def __init__(self, packed: np.ndarray, dtype: GgmlDType, shape: tuple[int, int], rank: int, world_size: int,
                 bias: torch.Tensor | None = None, device="cuda"):
        q = load_linear_shard(packed, dtype, shape, Shard.simple(0, rank, world_size), device)
        if bias is not None and world_size > 1:
            n = shape[0] // world_size
            bias = bias[rank * n:(rank + 1) * n]
        self.weight = GgufMatMul.from_qtensor(q, None if bias is None else bias.to(device))
        self.rank, self.world_size = rank, world_size

    def is_distributed(self) -> bool:
        return self.world_size > 1

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.weight.forward(x)

    __call__ = forward


class RowParallelLayer:
    """Input columns `[rank * k / w, (rank + 1) * k / w)` of the weight in whole blocks; matmul, contiguous, sum
    all-reduce, then the bias once (layers.rs:814-1190, forward_raw :1036-1046)."""

    def __init__(self, packed: np.ndarray, dtype: GgmlDType, shape: tuple[int, int], rank: int, world_size: int,
                 bias: torch.Tensor | None = None, device="cuda", group=None, all_reduce: SumAllReduce | None = None):
        q = load_linear_shard(packed, dtype, shape, Shard.simple(1, rank, world_size), device)
        self.weight = GgufMatMul.from_qtensor(q, None)  # a row shard never carries the bias (layers.rs:869-878)
        self.bias = None if bias is None else bias.to(device)
        # layers of one model share one exchange object (pass a PeerSumAllReduce for the peer-memory kernel)
        self.all_reduce = all_reduce if all_reduce is not None else SumAllReduce(group)
        self.rank, self.world_size = rank, world_size

    def is_distributed(self) -> bool:
        return self.world_size > 1

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x holds this rank's slice of the input features: `[..., k / w]`."""
        y = self._fused_forward(x)
        if y is None:
            y = self.weight.forward_raw(x).contiguous()
            y = self.all_reduce.sum_all_reduce(y)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def _fused_forward(self, x: torch.Tensor):
        """Matmul and exchange in one launch (`b200q_gemv_allreduce`) where the exchange object offers it and the call
        fits it: up to 8 rows, a sum within the exchange's capacity. The conditions only involve what all ranks share
        (shapes, types), so every rank takes the same path. None = not applicable."""
        ar = self.all_reduce
        if not isinstance(ar, PeerSumAllReduce) or ar.world == 1 or not x.is_contiguous():
            return None
        q = self.weight.get_qtensor()
        n, k = q.shape
        x2 = x.reshape(-1, k)
        rows = x2.shape[0]
        nbytes = rows * n * x.element_size()
        if rows < 1 or rows > 8 or k % 128 or nbytes % 16 or nbytes > ar.capacity or x.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            return None
        from . import ops
        if not ops.gemv_plan(q.dtype, k, n, rows)["staged"]:
            return None
        if x2.data_ptr() % 16:
            x2 = x2.clone()  # a rank's own addresses never change the path: misaligned rows are copied (torch allocations are aligned)
        return ar.gemv_sum(q.dtype, q.data, x2, n).reshape(*x.shape[:-1], n)

    __call__ = forward


class ReplicatedLayer:
    """The whole weight on every rank (layers.rs:1708)."""

    def __init__(self, packed: np.ndarray, dtype: GgmlDType, shape: tuple[int, int], bias: torch.Tensor | None = None,
                 device="cuda"):
        self.weight = GgufMatMul.from_qtensor(QTensor.from_packed(packed, dtype, shape, device),
                                              None if bias is None else bias.to(device))

    def is_distributed(self) -> bool:
        return False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.weight.forward(x)

    __call__ = forward


def compute_kv_shard(total_kv_heads: int, head_dim: int, rank: int, world_size: int) -> Shard:
    """KV heads per rank; with fewer KV heads than ranks each head is replicated over `world / heads` ranks
    (layers.rs:2566-2606)."""
    if world_size == 1:
        return Shard.simple(0, 0, 1)
    if total_kv_heads >= world_size:
        if total_kv_heads % world_size:
            raise ValueError(f"KV heads ({total_kv_heads}) must be divisible by tensor parallel size ({world_size}).")
        return Shard.simple(0, rank, world_size)
    if world_size % total_kv_heads:
        raise ValueError(f"Tensor parallel size ({world_size}) must be divisible by KV heads ({total_kv_heads}).")
    replication = world_size // total_kv_heads
    head = (rank // replication) % total_kv_heads
    return Shard.at(0, head * head_dim, head_dim)
