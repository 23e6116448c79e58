"""Llama-shaped GGUF files for the matmul path: the tensor-name map between the GGUF and the checkpoint naming, a writer
for a random-initialised model in the Q4_K_M mix, and a loader that hands the projections to `QTensor`.

The reference maps GGUF tensor names to its layers' checkpoint-style names when it loads a llama-family file
(crates/inference-gguf/src/normal_bindings.rs:887-914: `blk.N.attn_q` -> `model.layers.N.self_attn.q_proj`, ...; the
non-layer tensors `token_embd`, `output_norm`, `output` in the same function). Only what the matmul path needs is here:
the seven projections per layer, the output head and the embedding table.
"""
from __future__ import annotations

import re
from typing import BinaryIO

import numpy as np

from .dtypes import GgmlDType
from .gguf_file import Content, GgufError, Value, write
from .workloads import ModelShape

# GGUF suffix -> checkpoint suffix inside `model.layers.N.` (normal_bindings.rs:887-914 and the norm names above them)
LAYER_TENSORS = {
    "attn_q": "self_attn.q_proj",
    "attn_k": "self_attn.k_proj",
    "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj",
    "ffn_gate": "mlp.gate_proj",
    "ffn_up": "mlp.up_proj",
    "ffn_down": "mlp.down_proj",
    "attn_norm": "input_layernorm",
    "ffn_norm": "post_attention_layernorm",
}
TOP_TENSORS = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}
_BLK = re.compile(r"^blk\.(\d+)\.([a-z_]+)\.(weight|bias)$")


def checkpoint_name(gguf_name: str) -> str | None:
    """`blk.3.attn_q.weight` -> `model.layers.3.self_attn.q_proj.weight`; None for names the llama map does not know."""
    m = _BLK.match(gguf_name)
    if m:
        layer, key, suffix = m.groups()
        if key not in LAYER_TENSORS:
            return None
        return f"model.layers.{layer}.{LAYER_TENSORS[key]}.{suffix}"
    base, _, suffix = gguf_name.rpartition(".")
    if base in TOP_TENSORS and suffix in ("weight", "bias"):
        return f"{TOP_TENSORS[base]}.{suffix}"
    return None


def gguf_name(checkpoint: str) -> str | None:
    """The inverse of `checkpoint_name`."""
    m = re.match(r"^model\.layers\.(\d+)\.(.+)\.(weight|bias)$", checkpoint)
    if m:
        layer, mid, suffix = m.groups()
        for key, val in LAYER_TENSORS.items():
            if val == mid:
                return f"blk.{layer}.{key}.{suffix}"
        return None
    base, _, suffix = checkpoint.rpartition(".")
    for key, val in TOP_TENSORS.items():
        if val == base and suffix in ("weight", "bias"):
            return f"{key}.{suffix}"
    return None


def metadata_for(model: ModelShape, layers: int) -> list[tuple[str, Value]]:
    """The llama.* keys a loader reads for the matmul shapes (llama.cpp's key names)."""
    return [
        ("general.architecture", Value.string("llama")),
        ("general.name", Value.string(f"{model.name}-random-init")),
        ("general.file_type", Value.u32(15)),  # MOSTLY_Q4_K_M
        ("llama.block_count", Value.u32(layers)),
        ("llama.embedding_length", Value.u32(model.hidden)),
        ("llama.feed_forward_length", Value.u32(model.ffn)),
        ("llama.attention.head_count", Value.u32(model.q_heads)),
        ("llama.attention.head_count_kv", Value.u32(model.kv_heads)),
        ("llama.vocab_size", Value.u32(model.vocab)),
    ]


def write_random_llama(out: BinaryIO, model: ModelShape, layers: int, make_weight, include_output: bool = True) -> list[str]:
    """Writes `layers` layers of `model`'s projections (and the output head) in the Q4_K_M mix. `make_weight(name,
    projection)` returns the packed bytes of one matrix (uint8 numpy, `n * row_bytes`): quantized random weights from
    `ops.quantize_weights`, or blocks generated any other way. Returns the tensor names in file order."""
    tensors = []
    for li in range(layers):
        for p in model.layer_projections():
            name = f"blk.{li}.{p.name}.weight"
            tensors.append((name, int(p.dtype), (p.n, p.k), make_weight(name, p)))
    if include_output:
        p = model.output_projection()
        tensors.append(("output.weight", int(p.dtype), (p.n, p.k), make_weight("output.weight", p)))
    write(out, metadata_for(model, layers), tensors)
    return [t[0] for t in tensors]


def model_shape(content: Content) -> tuple[ModelShape, int]:
    """The shapes a llama GGUF declares, and its layer count."""
    md = {k: v.plain() for k, v in content.metadata.items()}
    if md.get("general.architecture") != "llama":
        raise GgufError(f"not a llama file: general.architecture = {md.get('general.architecture')!r}")
    try:
        hidden, heads = md["llama.embedding_length"], md["llama.attention.head_count"]
        shape = ModelShape(str(md.get("general.name", "llama")), md["llama.block_count"], hidden, heads,
                           md.get("llama.attention.head_count_kv", heads), hidden // heads, md["llama.feed_forward_length"],
                           md.get("llama.vocab_size", 0))
    except KeyError as e:
        raise GgufError(f"llama file lacks metadata key {e.args[0]}") from None
    return shape, shape.layers


def load_projections(f: BinaryIO, content: Content, device="cuda"):
    """`{checkpoint name: QTensor}` of every quantized matrix the llama map knows, checked against the declared shapes."""
    shape, layers = model_shape(content)
    expect = {p.name: (p.n, p.k, p.dtype) for p in shape.layer_projections()}
    out = {}
    for name, info in content.tensor_infos.items():
        target = checkpoint_name(name)
        if target is None or info.ggml_dtype not in (int(GgmlDType.Q8_0), int(GgmlDType.Q4K), int(GgmlDType.Q6K)):
            continue
        m = _BLK.match(name)
        if m:
            if int(m.group(1)) >= layers:
                raise GgufError(f"{name}: the file declares {layers} layers")
            n, k, _ = expect[m.group(2)]
            if tuple(info.shape) != (n, k):
                raise GgufError(f"{name}: shape {tuple(info.shape)}, the metadata implies {(n, k)}")
        out[target] = content.tensor(f, name, device)
    return out
