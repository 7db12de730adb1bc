"""CPU tests of the checkpoint reader / writer: the safetensors container (header, offsets, dtypes,
bit-exact payload), error handling on damaged files, sharded directories with an index, and the
tensor names of an MLX-community-style 4-bit model directory.  No kernel runs here; the model is
built on the CPU and only its tensors are compared."""

import json
import os
import struct

import pytest
import torch

from metile_b200 import synth
from metile_b200.integrations import blocks, checkpoint


def _same(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape
    view = torch.uint16 if a.dtype is torch.bfloat16 else a.dtype
    assert torch.equal(a.view(view), b.view(view))


def test_safetensors_round_trip_is_bit_exact(tmp_path):
    packed, scales, biases = synth.affine_weight(3, 32, 128)
    tensors = {"a.weight": packed, "a.scales": scales, "a.biases": biases,
               "norm.weight": synth.norm_weight(4, 128), "ids": torch.arange(7, dtype=torch.int32),
               "half": torch.randn(3, 5).to(torch.float16), "single": torch.randn(2, 2)}
    path = tmp_path / "model.safetensors"
    checkpoint.write_safetensors(path, tensors, {"format": "mlx"})
    loaded = checkpoint.read_safetensors(path)
    assert loaded.pop("__metadata__") == {"format": "mlx"}
    assert sorted(loaded) == sorted(tensors)
    for name in tensors:
        _same(loaded[name], tensors[name])
    # The header is what the format says: length prefix, JSON, offsets relative to its end.
    raw = path.read_bytes()
    (length,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + length])
    begin, end = header["a.weight"]["data_offsets"]
    assert header["a.weight"]["dtype"] == "U32" and header["a.scales"]["dtype"] == "BF16"
    assert raw[8 + length + begin:8 + length + end] == packed.numpy().tobytes()


def test_damaged_files_are_refused(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError, match="length prefix"):
        checkpoint.read_safetensors(path)
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="exceeds the file"):
        checkpoint.read_safetensors(path)
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(ValueError, match="inconsistent offsets"):
        checkpoint.read_safetensors(path)
    header = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(ValueError, match="unsupported dtype"):
        checkpoint.read_safetensors(path)


@pytest.mark.parametrize("shards", [1, 3])
@pytest.mark.parametrize("tied", [False, True])
def test_model_directory_round_trip(tmp_path, shards, tied):
    model = blocks.random_model(seed=5, device="cpu", layers=2, quantized_embedding=True, tie_word_embeddings=tied)
    config = checkpoint.save_torch_lm(model, tmp_path, shards=shards)
    assert config["quantization"] == {"group_size": 64, "bits": 4} and config["tie_word_embeddings"] is tied
    names = checkpoint.read_checkpoint_tensors(tmp_path)
    assert "model.layers.1.mlp.down_proj.scales" in names and "model.embed_tokens.biases" in names
    assert ("lm_head.weight" in names) is (not tied)
    assert os.path.exists(tmp_path / "model.safetensors.index.json") is (shards > 1)
    loaded = checkpoint.load_torch_lm(tmp_path, device="cpu")
    before, after = dict(model.named_buffers()), dict(loaded.named_buffers())
    assert sorted(before) == sorted(after)
    for name in before:
        _same(after[name], before[name])
    assert loaded.layers[0].self_attn.heads == 4 and loaded.layers[0].self_attn.kv_heads == 2
    if tied:
        assert loaded.lm_head.weight.data_ptr() == loaded.embed_tokens.weight.data_ptr()


def test_quantized_embedding_dequantises_the_rows_it_gathers():
    packed, scales, biases = synth.affine_weight(9, 16, 128)
    embedding = blocks.QuantizedEmbedding(packed, scales, biases)
    tokens = torch.tensor([[3, 0, 15]])
    out = embedding(tokens)
    assert out.shape == (1, 3, 128) and out.dtype == torch.bfloat16
    row = 3
    q = torch.tensor([(int(packed[row, k // 8].item()) >> (4 * (k % 8))) & 15 for k in range(128)], dtype=torch.float32)
    expected = (q * scales[row].float().repeat_interleave(64) + biases[row].float().repeat_interleave(64)).to(torch.bfloat16)
    _same(out[0, 0], expected)


def test_wrong_format_is_refused(tmp_path):
    model = blocks.random_model(seed=6, device="cpu", layers=1)
    checkpoint.save_torch_lm(model, tmp_path)
    config = json.loads((tmp_path / "config.json").read_text())
    config["quantization"]["bits"] = 8
    (tmp_path / "config.json").write_text(json.dumps(config))
    with pytest.raises(ValueError, match="4-bit"):
        checkpoint.load_torch_lm(tmp_path, device="cpu")


def test_projection_biases_and_dense_embedding_round_trip(tmp_path):
    """A Qwen2-style model (additive q / k / v biases) with a dense embedding and its own lm_head."""
    model = blocks.random_model(seed=7, device="cpu", layers=1)
    attention = model.layers[0].self_attn
    for index, name in enumerate(("q_proj", "k_proj", "v_proj")):
        linear = getattr(attention, name)
        linear.bias = synth.activations(40 + index, 1, linear.out_features).reshape(-1)
    config = checkpoint.save_torch_lm(model, tmp_path)
    assert config["model_type"] == "qwen2" and config["tie_word_embeddings"] is False
    names = checkpoint.read_checkpoint_tensors(tmp_path)
    assert "model.layers.0.self_attn.k_proj.bias" in names and "model.embed_tokens.scales" not in names
    loaded = checkpoint.load_torch_lm(tmp_path, device="cpu")
    _same(loaded.layers[0].self_attn.v_proj.bias, attention.v_proj.bias)
    _same(loaded.embed_tokens.weight, model.embed_tokens.weight)
    assert loaded.layers[0].self_attn.o_proj.bias is None


def test_tied_embeddings_need_a_quantised_embedding(tmp_path):
    model = blocks.random_model(seed=8, device="cpu", layers=1)
    checkpoint.save_torch_lm(model, tmp_path)
    config = json.loads((tmp_path / "config.json").read_text())
    config["tie_word_embeddings"] = True
    (tmp_path / "config.json").write_text(json.dumps(config))
    tensors = checkpoint.read_safetensors(tmp_path / "model.safetensors")
    tensors.pop("__metadata__", None)
    for name in [n for n in tensors if n.startswith("lm_head.")]:
        del tensors[name]
    checkpoint.write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(ValueError, match="tied word embeddings"):
        checkpoint.load_torch_lm(tmp_path, device="cpu")
