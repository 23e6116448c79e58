"""The matmul shapes of the benchmark configurations: per-layer projections of Llama-3-shaped models under the
Q4_K_M mix the baseline names (attn_v, ffn_down and output in Q6_K, everything else Q4_K), and the decode sweep."""
from __future__ import annotations

from dataclasses import dataclass

from .dtypes import GgmlDType


@dataclass(frozen=True)
class Projection:
    name: str
    dtype: GgmlDType
    k: int           # input features (columns of the packed weight)
    n: int           # output features (rows of the packed weight)
    split: str       # tensor-parallel split: "col" (rows of W), "row" (columns of W, whole superblocks), "none"

    @property
    def weight_bytes(self) -> int:
        return self.n * self.dtype.row_bytes(self.k)


@dataclass(frozen=True)
class ModelShape:
    name: str
    layers: int
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    ffn: int
    vocab: int

    def layer_projections(self) -> list[Projection]:
        h, kv = self.hidden, self.kv_heads * self.head_dim
        q4, q6 = GgmlDType.Q4K, GgmlDType.Q6K
        return [
            Projection("attn_q", q4, h, self.q_heads * self.head_dim, "col"),
            Projection("attn_k", q4, h, kv, "col"),
            Projection("attn_v", q6, h, kv, "col"),
            Projection("attn_output", q4, self.q_heads * self.head_dim, h, "row"),
            Projection("ffn_gate", q4, h, self.ffn, "col"),
            Projection("ffn_up", q4, h, self.ffn, "col"),
            Projection("ffn_down", q6, self.ffn, h, "row"),
        ]

    def output_projection(self) -> Projection:
        return Projection("output", GgmlDType.Q6K, self.hidden, self.vocab, "col")

    def weight_bytes_per_token(self) -> int:
        return self.layers * sum(p.weight_bytes for p in self.layer_projections()) + self.output_projection().weight_bytes


LLAMA3_8B = ModelShape("llama3-8b", 32, 4096, 32, 8, 128, 14336, 128256)
LLAMA3_70B = ModelShape("llama3-70b", 80, 8192, 64, 8, 128, 28672, 128256)

# decode sweep (K x N) of the baseline's second configuration
SWEEP_SHAPES = [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096), (4096, 128256)]


def shard(p: Projection, world: int) -> Projection:
    """The per-rank projection under tensor parallelism: column split divides N, row split divides K in whole blocks
    (crates/inference-quant/src/uqff/mod.rs:111-140)."""
    if world == 1 or p.split == "none":
        return p
    if p.split == "col":
        if p.n % world:
            raise ValueError(f"{p.name}: {p.n} rows do not divide over {world} ranks")
        return Projection(p.name, p.dtype, p.k, p.n // world, p.split)
    if p.k % (world * p.dtype.block_size):
        raise ValueError(f"{p.name}: {p.k} columns do not divide over {world} ranks in whole blocks")
    return Projection(p.name, p.dtype, p.k // world, p.n, p.split)
