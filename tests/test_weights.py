"""safetensors reading and writing, loading by name, the one error that lists
everything wrong, and the random-weights mode (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from conftest import TINY_A, TINY_B
from zinfer_b200.config import Qwen3Config, qwen3_model_spec
from zinfer_b200.engine.model import declared_tensors
from zinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_tensors, random_tensors,
                                 write_model_dir, write_safetensors)


def _raw_file(path, header: dict, data: bytes):
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + data)


def test_round_trip_and_bf16_bit_patterns(tmp_path):
    # 1.0, -1.0, 2.0 are 0x3f80, 0xbf80, 0x4000 in bfloat16 (src/tensor/formats/bfloat16.zig:23-29)
    t = {"a": torch.tensor([1.0, -1.0, 2.0], dtype=torch.bfloat16), "b": torch.arange(6, dtype=torch.float32).reshape(2, 3),
         "c": torch.tensor([[1, 2]], dtype=torch.int32)}
    p = str(tmp_path / "m.safetensors")
    write_safetensors(p, t, metadata={"format": "pt"})
    with SafetensorsFile(p) as f:
        assert f.metadata == {"format": "pt"} and set(f.names()) == {"a", "b", "c"}
        assert f.tensor("a").view(torch.uint16).tolist() == [0x3F80, 0xBF80, 0x4000]
        assert torch.equal(f.tensor("b"), t["b"]) and torch.equal(f.tensor("c"), t["c"])
        with pytest.raises(KeyError):
            f.tensor("zzz")


@pytest.mark.parametrize("header,data,match", [
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 12]}}, b"\0" * 12, "needs 8 bytes"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, "beyond the data"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
      "b": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 6, "overlaps"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8, "unused bytes before"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 8, "unused bytes after"),
    ({"a": {"dtype": "Q9", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 4, "unsupported dtype"),
    ({"a": {"dtype": "F32", "shape": [1]}}, b"\0" * 4, "lacks 'data_offsets'"),
    ({"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}, b"\0" * 4, "invalid shape"),
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 0]}}, b"\0" * 4, "invalid data_offsets"),
    ({"__metadata__": {"k": 3}}, b"", "__metadata__"),
])
def test_malformed_files_are_refused(tmp_path, header, data, match):
    p = str(tmp_path / "bad.safetensors")
    _raw_file(p, header, data)
    with pytest.raises(SafetensorsError, match=match):
        SafetensorsFile(p)


def test_truncated_and_garbage_headers(tmp_path):
    p = str(tmp_path / "x.safetensors")
    open(p, "wb").write(b"\1\2\3")
    with pytest.raises(SafetensorsError, match="shorter"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds the file"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        SafetensorsFile(p)


def test_random_model_folder_loads_back(tmp_path):
    for raw in (TINY_A, TINY_B):
        cfg = Qwen3Config.from_dict(raw)
        d = write_model_dir(str(tmp_path / f"m{cfg.hidden_size}"), cfg, seed=5)
        assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
        specs = declared_tensors(qwen3_model_spec(cfg))
        got = load_tensors(d, specs, torch.bfloat16, "cpu")
        assert set(got) == {n for n, s in specs.items() if not s.optional}
        for n, t in got.items():
            assert tuple(t.shape) == specs[n].shape and t.dtype == torch.bfloat16
        # same seed, same values; another seed, other values; norm weights near one, matrices near zero
        again = random_tensors(specs, 5, torch.bfloat16)
        assert all(torch.equal(again[n], got[n]) for n in got)
        other = random_tensors(specs, 6, torch.bfloat16)
        assert not torch.equal(other["model.norm.weight"], got["model.norm.weight"])
        nw = got["model.layers.0.input_layernorm.weight"].float()
        assert 0.9 <= nw.min() and nw.max() <= 1.1
        assert abs(got["model.layers.0.mlp.down_proj.weight"].float().std() - 0.02) < 0.004
    assert ("lm_head.weight" in got) and "lm_head.weight" not in load_tensors(
        str(tmp_path / "m64"), declared_tensors(qwen3_model_spec(Qwen3Config.from_dict(TINY_A))), torch.bfloat16, "cpu")


def test_stored_32_bit_stays_32_bit_and_float32_run_widens(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_A)
    d16 = write_model_dir(str(tmp_path / "bf"), cfg, seed=1, dtype=torch.bfloat16)
    d32 = write_model_dir(str(tmp_path / "f32"), cfg, seed=1, dtype=torch.float32)
    specs = declared_tensors(qwen3_model_spec(cfg))
    assert all(t.dtype == torch.float32 for t in load_tensors(d32, specs, torch.bfloat16, "cpu").values())
    wide = load_tensors(d16, specs, torch.float32, "cpu")
    narrow = load_tensors(d16, specs, torch.bfloat16, "cpu")
    assert all(t.dtype == torch.float32 and torch.equal(t, narrow[n].float()) for n, t in wide.items())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_B)
    specs = declared_tensors(qwen3_model_spec(cfg))
    t = random_tensors(specs, 3, torch.bfloat16)
    del t["model.layers.1.self_attn.k_norm.weight"]
    del t["lm_head.weight"]
    t["model.layers.0.mlp.up_proj.weight"] = torch.zeros(7, 3, dtype=torch.bfloat16)
    t["model.layers.9.extra.weight"] = torch.zeros(2, dtype=torch.bfloat16)
    t["model.norm.weight"] = torch.zeros(cfg.hidden_size, dtype=torch.int32)
    d = tmp_path / "m"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), t)
    with pytest.raises(WeightsError) as ei:
        load_tensors(str(d), specs, torch.bfloat16, "cpu")
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.k_norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert len(e.wrong_shape) == 1 and "up_proj" in e.wrong_shape[0] and "[7, 3]" in e.wrong_shape[0]
    assert len(e.wrong_kind) == 1 and "model.norm.weight" in e.wrong_kind[0]
    msg = str(e)
    for part in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "k_norm", "extra"):
        assert part in msg


def test_tied_head_needs_no_separate_tensor_and_tolerates_one(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_A)   # tied
    specs = declared_tensors(qwen3_model_spec(cfg))
    assert specs["lm_head.weight"].optional
    t = random_tensors(specs, 3, torch.bfloat16, include_optional=True)
    d = tmp_path / "m"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), t)
    assert "lm_head.weight" in load_tensors(str(d), specs, torch.bfloat16, "cpu")
    untied = declared_tensors(qwen3_model_spec(Qwen3Config.from_dict({**TINY_A, "tie_word_embeddings": False})))
    del t["lm_head.weight"]
    write_safetensors(str(d / "model.safetensors"), t)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_tensors(str(d), untied, torch.bfloat16, "cpu")


# ------------------------------------------------------------------------- shards
def test_sharded_folder_loads_back_equal_to_the_single_file(tmp_path):
    from zinfer_b200.weights import Checkpoint

    cfg = Qwen3Config.from_dict(TINY_B)
    specs = declared_tensors(qwen3_model_spec(cfg))
    one = write_model_dir(str(tmp_path / "one"), cfg, seed=9)
    three = write_model_dir(str(tmp_path / "three"), cfg, seed=9, shards=3)
    files = sorted(os.listdir(three))
    assert files == ["config.json", "model-00001-of-00003.safetensors", "model-00002-of-00003.safetensors",
                     "model-00003-of-00003.safetensors", "model.safetensors.index.json"]
    index = json.load(open(os.path.join(three, "model.safetensors.index.json")))
    assert set(index["weight_map"]) == {n for n, s in specs.items() if not s.optional}
    assert len(set(index["weight_map"].values())) == 3
    sizes = [os.path.getsize(os.path.join(three, f)) for f in files[1:4]]
    assert max(sizes) < 2.5 * min(sizes), "the shards are far from equal in size"
    a, b = load_tensors(one, specs, torch.bfloat16, "cpu"), load_tensors(three, specs, torch.bfloat16, "cpu")
    assert list(a) == list(b) and all(torch.equal(a[n], b[n]) for n in a)
    with Checkpoint(three) as ck:
        assert len(ck.files) == 3 and ck.info("model.norm.weight").shape == (cfg.hidden_size,)


def test_one_error_over_all_shards(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_B)
    specs = declared_tensors(qwen3_model_spec(cfg))
    t = random_tensors(specs, 3, torch.bfloat16)
    del t["model.layers.1.self_attn.k_norm.weight"]                        # would lie in a middle shard
    del t["lm_head.weight"]                                                 # in the last
    t["model.embed_tokens.weight"] = torch.zeros(5, 5, dtype=torch.bfloat16)   # in the first
    t["model.layers.9.extra.weight"] = torch.zeros(2, dtype=torch.bfloat16)
    from zinfer_b200.weights import write_sharded

    d = tmp_path / "m"
    d.mkdir()
    write_sharded(str(d), t, 3)
    with pytest.raises(WeightsError) as ei:
        load_tensors(str(d), specs, torch.bfloat16, "cpu")
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.k_norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert len(e.wrong_shape) == 1 and "embed_tokens" in e.wrong_shape[0]


def test_broken_shard_sets_are_refused(tmp_path):
    from zinfer_b200.weights import Checkpoint, CheckpointError

    cfg = Qwen3Config.from_dict(TINY_A)
    d = write_model_dir(str(tmp_path / "m"), cfg, seed=2, shards=2)
    index_path = os.path.join(d, "model.safetensors.index.json")
    index = json.load(open(index_path))
    # a shard that the index names is absent
    os.rename(os.path.join(d, "model-00002-of-00002.safetensors"), os.path.join(d, "elsewhere"))
    with pytest.raises(CheckpointError, match="model-00002-of-00002.safetensors"):
        Checkpoint(d)
    os.rename(os.path.join(d, "elsewhere"), os.path.join(d, "model-00002-of-00002.safetensors"))
    # the index places a tensor in a shard that does not hold it
    bad = json.loads(json.dumps(index))
    bad["weight_map"]["model.norm.weight"] = "model-00001-of-00002.safetensors"
    json.dump(bad, open(index_path, "w"))
    with pytest.raises(CheckpointError, match="model.norm.weight"):
        Checkpoint(d)
    # an index that is no index
    open(index_path, "w").write('{"weight_map": []}')
    with pytest.raises(CheckpointError, match="weight_map"):
        Checkpoint(d)
    # a folder without weights
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        Checkpoint(str(tmp_path))
    # a tensor held by two shards
    json.dump(index, open(index_path, "w"))
    import shutil
    shutil.copy(os.path.join(d, "model-00001-of-00002.safetensors"), os.path.join(d, "copy.safetensors"))
    index["weight_map"]["model.embed_tokens.weight"] = "copy.safetensors"
    json.dump(index, open(index_path, "w"))
    with pytest.raises(CheckpointError, match="two shards"):
        Checkpoint(d)
