"""Llama-shaped GGUF files for the matmul path: the tensor-name map (crates/inference-gguf/src/normal_bindings.rs:887-914),
a random-initialised model written in the Q4_K_M mix with the oracle's quantizer, read back byte for byte; on the GPU the
projections loaded from the file give the same matmuls as the bytes that were written."""
import io
import zlib

import numpy as np
import pytest
import torch

from oracle import kquants as kq

import inference_rs_b200 as pkg
from inference_rs_b200 import llama_gguf as lg
from inference_rs_b200.gguf_file import Content, GgufError, Value, write
from inference_rs_b200.workloads import ModelShape

TINY = ModelShape("tiny-llama", 2, 256, 4, 2, 64, 512, 1024)
KQ_TYPE = {pkg.GgmlDType.Q4K: kq.Q4_K, pkg.GgmlDType.Q6K: kq.Q6_K, pkg.GgmlDType.Q8_0: kq.Q8_0}


def quantized_random(name, p):
    g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
    w = (torch.randn(p.n, p.k, generator=g) * 0.02).numpy()
    return kq.quantize(KQ_TYPE[p.dtype], w).reshape(-1)


def written_file():
    buf = io.BytesIO()
    packed = {}

    def make(name, p):
        packed[name] = quantized_random(name, p)
        return packed[name]

    names = lg.write_random_llama(buf, TINY, TINY.layers, make)
    buf.seek(0)
    return buf, names, packed


def test_name_map_both_directions():
    pairs = [("blk.0.attn_q.weight", "model.layers.0.self_attn.q_proj.weight"),
             ("blk.31.attn_k.weight", "model.layers.31.self_attn.k_proj.weight"),
             ("blk.7.attn_v.weight", "model.layers.7.self_attn.v_proj.weight"),
             ("blk.7.attn_output.weight", "model.layers.7.self_attn.o_proj.weight"),
             ("blk.2.ffn_gate.weight", "model.layers.2.mlp.gate_proj.weight"),
             ("blk.2.ffn_up.weight", "model.layers.2.mlp.up_proj.weight"),
             ("blk.2.ffn_down.weight", "model.layers.2.mlp.down_proj.weight"),
             ("blk.2.attn_norm.weight", "model.layers.2.input_layernorm.weight"),
             ("blk.2.ffn_norm.weight", "model.layers.2.post_attention_layernorm.weight"),
             ("token_embd.weight", "model.embed_tokens.weight"), ("output_norm.weight", "model.norm.weight"),
             ("output.weight", "lm_head.weight")]
    for g, c in pairs:
        assert lg.checkpoint_name(g) == c
        assert lg.gguf_name(c) == g
    assert lg.checkpoint_name("blk.0.ffn_gate_exps.weight") is None  # MoE tensors are not on this path
    assert lg.checkpoint_name("rope_freqs.weight") is None
    assert lg.gguf_name("model.layers.0.self_attn.rotary_emb.inv_freq") is None


def test_random_llama_file_round_trips_byte_for_byte():
    buf, names, packed = written_file()
    content = Content.read(buf)
    shape, layers = lg.model_shape(content)
    assert (layers, shape.hidden, shape.ffn, shape.q_heads, shape.kv_heads, shape.head_dim, shape.vocab) == (2, 256, 512, 4, 2, 64, 1024)
    assert list(content.tensor_infos) == names and len(names) == 2 * 7 + 1
    for p in TINY.layer_projections():
        info, raw = content.tensor_bytes(buf, f"blk.1.{p.name}.weight")
        assert info.ggml_dtype == int(p.dtype) and tuple(info.shape) == (p.n, p.k)
        assert np.array_equal(raw, packed[f"blk.1.{p.name}.weight"])
    info, raw = content.tensor_bytes(buf, "output.weight")
    assert info.ggml_dtype == int(pkg.GgmlDType.Q6K) and np.array_equal(raw, packed["output.weight"])


def test_gguf_py_reads_the_same_file():
    gguf = pytest.importorskip("gguf")
    import os
    import tempfile
    buf, names, packed = written_file()
    with tempfile.NamedTemporaryFile(suffix=".gguf", delete=False) as tmp:
        tmp.write(buf.getvalue())
        path = tmp.name
    try:
        reader = gguf.GGUFReader(path)
        got = {t.name: t for t in reader.tensors}
        assert set(got) == set(names)
        t = got["blk.0.ffn_down.weight"]
        assert int(t.tensor_type) == int(pkg.GgmlDType.Q6K)
        assert np.array_equal(np.asarray(t.data).reshape(-1).view(np.uint8), packed["blk.0.ffn_down.weight"])
    finally:
        os.unlink(path)


def test_not_a_llama_file_and_shape_mismatch_are_refused():
    buf = io.BytesIO()
    write(buf, [("general.architecture", Value.string("qwen2"))], [])
    buf.seek(0)
    with pytest.raises(GgufError):
        lg.model_shape(Content.read(buf))
    buf = io.BytesIO()
    write(buf, [("general.architecture", Value.string("llama")), ("llama.block_count", Value.u32(1))], [])
    buf.seek(0)
    with pytest.raises(GgufError, match="llama.embedding_length"):
        lg.model_shape(Content.read(buf))


@pytest.mark.gpu
def test_projections_loaded_from_the_file_multiply_like_the_written_bytes():
    from inference_rs_b200 import ops
    from inference_rs_b200.qmatmul import QMatMul
    buf, names, packed = written_file()
    content = Content.read(buf)
    weights = lg.load_projections(buf, content, "cuda")
    assert len(weights) == len(names)
    g = torch.Generator().manual_seed(3)
    for li in range(TINY.layers):
        for p in TINY.layer_projections():
            q = weights[lg.checkpoint_name(f"blk.{li}.{p.name}.weight")]
            assert q.shape == (p.n, p.k) and q.dtype == p.dtype
            x = torch.randn(1, p.k, generator=g).to(torch.bfloat16).cuda()
            got = QMatMul.from_qtensor(q).forward(x)
            direct = ops.gemv(p.dtype, ops.upload_weights(packed[f"blk.{li}.{p.name}.weight"], p.dtype), x, p.n)
            assert torch.equal(got, direct)
            ref = kq.matmul(KQ_TYPE[p.dtype], x.float().cpu().numpy(), packed[f"blk.{li}.{p.name}.weight"].reshape(p.n, -1), p.n)
            err = np.abs(got.float().cpu().numpy() - ref).max()
            assert err <= 1e-3 + 2e-2 * np.abs(ref).max()  # a few hundred outputs per tensor: the reference's own 2 % gate
    torch.cuda.synchronize()
