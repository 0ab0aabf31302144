"""GGUF reader on the host (no GPU): header, metadata, tensor directory, names, byte-exact tensor reads and
the tensor-parallel shards cut at load, against a file written by the third-party gguf-py writer."""
import struct

import numpy as np
import pytest

from boostr_b200 import gguf as G
from boostr_b200.format import QuantFormat as F
from boostr_b200.tensor_parallel import DistributedError, shard_bytes
from gguf_fixture import HID, LAYER_TENSORS, VOC, write_gguf

pytest.importorskip("gguf")


@pytest.fixture(scope="module")
def fixture(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("gguf") / "tiny.gguf")
    packed = write_gguf(path, layers=2)
    return path, packed


def test_header_metadata_and_directory(fixture):
    path, packed = fixture
    g = G.Gguf.open(path)
    assert g.version == 3
    assert g.metadata["general.architecture"] == "llama" and g.metadata["llama.block_count"] == 2
    assert g.data_offset % 32 == 0
    info = g.tensors["blk.1.ffn_down.weight"]
    assert info.type_name == "Q6_K" and info.ggml_type == F.Q6_K.ggml_type_id
    assert info.row_major_shape() == (HID, 2048)          # GGML order reversed (reader.rs:497-499)
    assert info.size_bytes() == F.Q6_K.storage_bytes(HID * 2048)
    assert g.tensors["output_norm.weight"].type_name == "F16"
    for name, (fmt, n, k, b) in packed.items():
        assert g.quant_format(name) is F.parse(fmt)
        assert np.array_equal(g.read_tensor_bytes(name), b), name
    g.close()


def test_custom_alignment(tmp_path):
    path = str(tmp_path / "a64.gguf")
    packed = write_gguf(path, layers=1, alignment=64)
    g = G.Gguf.open(path)
    assert g.metadata["general.alignment"] == 64 and g.data_offset % 64 == 0
    name = "blk.0.attn_v.weight"
    assert np.array_equal(g.read_tensor_bytes(name), packed[name][3])


def test_from_bytes_and_errors(fixture):
    path, packed = fixture
    data = open(path, "rb").read()
    g = G.Gguf.from_bytes(data)
    assert set(g.tensors) >= set(packed)
    with pytest.raises(G.GgufError, match="invalid GGUF magic"):
        G.Gguf.from_bytes(b"GGML" + data[4:])
    with pytest.raises(G.GgufError, match="unsupported GGUF version"):
        G.Gguf.from_bytes(data[:4] + struct.pack("<I", 9) + data[8:])
    with pytest.raises(G.GgufError, match="tensor not found"):
        g.read_tensor_bytes("blk.9.attn_q.weight")
    with pytest.raises(G.GgufError, match="not a quantized format"):
        g.quant_format("output_norm.weight")
    with pytest.raises(G.GgufError, match="unexpected end"):
        G.Gguf.from_bytes(data[:40])


def test_name_map():
    m = G.gguf_to_hf_name
    assert m("token_embd.weight") == "model.embed_tokens.weight"
    assert m("output_norm.weight") == "model.norm.weight"
    assert m("output.weight") == "lm_head.weight"
    assert m("blk.7.attn_v.weight") == "model.layers.7.self_attn.v_proj.weight"
    assert m("blk.0.attn_output.weight") == "model.layers.0.self_attn.o_proj.weight"
    assert m("blk.31.ffn_down.weight") == "model.layers.31.mlp.down_proj.weight"
    assert m("blk.2.ffn_gate.5.weight") == "model.layers.2.block_sparse_moe.experts.5.gate_proj.weight"
    assert m("blk.3.attn_q.bias") == "model.layers.3.self_attn.q_proj.bias"
    assert m("rope_freqs.weight") == "rope_freqs.weight"
    assert G.parallel_dim("model.layers.0.self_attn.q_proj.weight") == 0
    assert G.parallel_dim("model.layers.0.mlp.down_proj.weight") == 1
    assert G.parallel_dim("lm_head.weight") == 0
    assert G.parallel_dim("model.norm.weight") is None


@pytest.mark.parametrize("world", [1, 2, 4])
def test_shards_cut_at_load_match_the_shard_packer(fixture, world):
    path, packed = fixture
    g = G.Gguf.open(path)
    for name, (fmt, n, k, b) in packed.items():
        dim = G.parallel_dim(G.gguf_to_hf_name(name))
        for rank in range(world):
            qt = g.load_tensor_quantized(name, device="cpu", rank=rank, world=world, dim=dim if world > 1 else None)
            want = b if world == 1 else shard_bytes(fmt, b, n, k, dim, rank, world)
            assert np.array_equal(qt.storage.numpy(), want), (name, rank)
            assert qt.shape == ((n, k) if world == 1 else (n // world, k) if dim == 0 else (n, k // world))
    with pytest.raises(DistributedError, match="not divisible"):
        g.load_tensor_quantized("output.weight", device="cpu", rank=0, world=7, dim=0)
    assert VOC % 7


def test_varmap_takes_each_tensor_once(fixture):
    path, _ = fixture
    vm = G.GgufVarMap(G.Gguf.open(path), device="cpu")
    assert vm.contains("model.layers.0.self_attn.q_proj.weight")
    norm = vm.take_tensor("model.norm.weight")
    assert norm.dtype.is_floating_point and norm.shape == (HID,)
    qt = vm.take_quant_tensor("lm_head.weight")
    assert qt.format is F.Q6_K and qt.shape == (VOC, HID)
    with pytest.raises(G.GgufError, match="tensor not found"):
        vm.take_quant_tensor("lm_head.weight")
    assert len(LAYER_TENSORS) == 7
