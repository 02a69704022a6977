"""Weights: the safetensors container, loading by name, the one error that lists every
difference, stored dtypes, sharded folders, and the random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import qwen3_b200 as q
from qwen3_b200.weights import Checkpoint, SafetensorsFile
from helpers import tiny


def specs_of(cfg):
    return q.build_model(q.config_from_dict(cfg).plan())


def test_random_model_folder_round_trip(tmp_path):
    config = q.config_from_dict(tiny("B"))
    tensors = q.write_random_model(str(tmp_path / "m"), config, seed=3)
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
    assert q.load_config(str(tmp_path / "m")) == config
    model = q.build_model(config.plan())
    loaded = q.load_weights(str(tmp_path / "m"), model.weight_specs(), model.ignorable_names())
    assert set(loaded) == set(tensors) and len(loaded) == 2 + 11 * 3 + 1
    for name, t in tensors.items():
        assert loaded[name].dtype == torch.bfloat16 and torch.equal(loaded[name], t), name


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    model = specs_of(tiny("A"))
    a = q.random_weights(model.weight_specs(), seed=5)
    b = q.random_weights(dict(reversed(list(model.weight_specs().items()))), seed=5)
    c = q.random_weights(model.weight_specs(), seed=6)
    for name in a:
        assert torch.equal(a[name], b[name])
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"].float()
    n = a["model.layers.1.input_layernorm.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = q.config_from_dict(tiny("B"))
    model = q.build_model(config.plan())
    tensors = q.random_weights(model.weight_specs(), seed=1)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 256, dtype=torch.bfloat16)   # transposed
    tensors["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    tensors["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2, dtype=torch.bfloat16)
    tensors["rotary.inv_freq"] = torch.zeros(4, dtype=torch.float32)
    q.write_model_folder(str(tmp_path / "m"), config, tensors)
    with pytest.raises(q.WeightError) as e:
        q.load_weights(str(tmp_path / "m"), model.weight_specs(), model.ignorable_names())
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.mlp.up_proj.weight", "rotary.inv_freq"]
    assert [n for n, _, _ in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight",
                                                 "model.layers.2.self_attn.q_norm.weight"]
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (2)", "[96, 256] != model [256, 96]"):
        assert piece in text


def test_tied_checkpoint_ignores_lm_head_and_untied_needs_it(tmp_path):
    tied = q.config_from_dict(tiny("A"))
    model = q.build_model(tied.plan())
    tensors = q.random_weights(model.weight_specs(), seed=1)
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    q.write_model_folder(str(tmp_path / "tied"), tied, tensors)
    loaded = q.load_weights(str(tmp_path / "tied"), model.weight_specs(), model.ignorable_names())
    assert "lm_head.weight" not in loaded
    untied = q.config_from_dict(tiny("A", tie_word_embeddings=False))
    model = q.build_model(untied.plan())
    with pytest.raises(q.WeightError):
        tensors.pop("lm_head.weight")
        q.write_model_folder(str(tmp_path / "untied"), untied, tensors)
        q.load_weights(str(tmp_path / "untied"), model.weight_specs(), model.ignorable_names())


def test_stored_dtypes_are_kept(tmp_path):
    path = str(tmp_path / "x.safetensors")
    tensors = {"half": torch.randn(3, 5).to(torch.bfloat16), "full": torch.randn(7), "table": torch.arange(6, dtype=torch.int32).view(2, 3),
               "empty": torch.zeros(0, 4, dtype=torch.float32)}
    q.save_file(tensors, path, metadata={"format": "pt"})
    f = SafetensorsFile(path)
    assert f.metadata == {"format": "pt"}
    for name, t in tensors.items():
        got = f.tensor(name)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)
    specs = {"full": q.WeightSpec((7,), "norm"), "table": q.WeightSpec((2, 3), "int_table")}
    os.rename(path, str(tmp_path / "model.safetensors"))
    with pytest.raises(q.WeightError) as e:
        q.load_weights(str(tmp_path), specs)
    assert e.value.unexpected == ["empty", "half"]
    got = q.load_weights(str(tmp_path), specs, ignorable=["empty", "half"])
    assert got["full"].dtype == torch.float32 and got["table"].dtype == torch.int32
    with pytest.raises(q.WeightError, match="wrong dtypes"):
        q.load_weights(str(tmp_path), {"full": q.WeightSpec((7,), "int_table")}, ignorable=["empty", "half", "table"])


def write_raw(path, header: bytes, data: bytes = b""):
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + data)


def test_malformed_files_are_refused(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(q.SafetensorsFormatError, match="8-byte"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(q.SafetensorsFormatError, match="not plausible"):
        SafetensorsFile(p)
    write_raw(p, b"[1, 2]")
    with pytest.raises(q.SafetensorsFormatError, match="start with"):
        SafetensorsFile(p)
    write_raw(p, b"{not json}")
    with pytest.raises(q.SafetensorsFormatError, match="JSON"):
        SafetensorsFile(p)
    write_raw(p, json.dumps({"a": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}).encode(), b"\0" * 4)
    with pytest.raises(q.SafetensorsFormatError, match="F16"):
        SafetensorsFile(p)
    write_raw(p, json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode(), b"\0" * 8)
    with pytest.raises(q.SafetensorsFormatError, match="claims bytes"):
        SafetensorsFile(p)
    write_raw(p, json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode(), b"\0" * 8)
    with pytest.raises(q.SafetensorsFormatError, match="claims bytes"):
        SafetensorsFile(p)


def make_sharded(folder, tensors, split):
    os.makedirs(folder, exist_ok=True)
    names = list(tensors)
    shards = {"model-00001-of-00002.safetensors": names[:split], "model-00002-of-00002.safetensors": names[split:]}
    weight_map, total = {}, 0
    for shard, members in shards.items():
        total += q.save_file({n: tensors[n] for n in members}, os.path.join(folder, shard))
        weight_map.update({n: shard for n in members})
    index = {"metadata": {"total_size": total}, "weight_map": weight_map}
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    return index


def test_sharded_folder_and_its_checks(tmp_path):
    config = q.config_from_dict(tiny("A"))
    model = q.build_model(config.plan())
    tensors = q.random_weights(model.weight_specs(), seed=2)
    folder = str(tmp_path / "sharded")
    index = make_sharded(folder, tensors, 9)
    loaded = q.load_weights(folder, model.weight_specs(), model.ignorable_names())
    for name, t in tensors.items():
        assert torch.equal(loaded[name], t)
    index_path = os.path.join(folder, "model.safetensors.index.json")

    def rewrite(change):
        bad = json.loads(json.dumps(index))
        change(bad)
        with open(index_path, "w") as f:
            json.dump(bad, f)

    rewrite(lambda i: i["metadata"].update(total_size=5))
    with pytest.raises(q.SafetensorsFormatError, match="total_size"):
        Checkpoint(folder)
    rewrite(lambda i: i["weight_map"].pop("model.norm.weight"))
    with pytest.raises(q.SafetensorsFormatError, match="does not map"):
        Checkpoint(folder)
    rewrite(lambda i: i["weight_map"].update({"ghost.weight": "model-00001-of-00002.safetensors"}))
    with pytest.raises(q.SafetensorsFormatError, match="not in shard"):
        Checkpoint(folder)
    rewrite(lambda i: i["weight_map"].update({"model.norm.weight": "../elsewhere.safetensors"}))
    with pytest.raises(q.SafetensorsFormatError, match="plain"):
        Checkpoint(folder)
    rewrite(lambda i: i["weight_map"].update({"model.norm.weight": "model-00003-of-00003.safetensors"}))
    with pytest.raises(q.SafetensorsFormatError, match="missing"):
        Checkpoint(folder)
    rewrite(lambda i: None)
    open(os.path.join(folder, "model.safetensors"), "wb").write(b"")
    with pytest.raises(q.SafetensorsFormatError, match="both"):
        Checkpoint(folder)
    with pytest.raises(q.SafetensorsFormatError, match="neither"):
        Checkpoint(str(tmp_path))
