"""The safetensors container, loading by name with one error for everything wrong, random weights."""
import json
import struct

import numpy as np
import pytest
import torch

from machserve_b200.config import config_from_json
from machserve_b200.parts import declared_tensors
from machserve_b200.weights import (
    SafetensorsError, TensorDecl, WeightsError, load_weights, normal_values, open_model_files, write_safetensors,
)
from tests.helpers import TINY, make_model_dir


def test_round_trip_keeps_storage_dtypes(tmp_path):
    t = {
        "a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
        "b": torch.tensor([1.5, -2.25], dtype=torch.bfloat16),
        "h": torch.tensor([0.5, 3.0], dtype=torch.float16),
        "i": torch.tensor([[1, 2], [3, 4]], dtype=torch.int64),
    }
    write_safetensors(tmp_path / "model.safetensors", t)
    decls = [TensorDecl("a", (2, 3)), TensorDecl("b", (2,)), TensorDecl("h", (2,)), TensorDecl("i", (2, 2), init="table")]
    with pytest.warns(UserWarning, match="float16 and are rounded to bfloat16"):
        kept = load_weights(tmp_path, decls, torch.bfloat16)
    # stored in 32 bits stays float32; 16-bit floats are kept as bfloat16; integer tables are int32
    assert kept["a"].dtype == torch.float32 and torch.equal(kept["a"], t["a"])
    assert kept["b"].dtype == torch.bfloat16 and torch.equal(kept["b"], t["b"])
    assert kept["h"].dtype == torch.bfloat16 and kept["h"].tolist() == [0.5, 3.0]
    assert kept["i"].dtype == torch.int32 and kept["i"].tolist() == [[1, 2], [3, 4]]
    wide = load_weights(tmp_path, decls, torch.float32)
    assert all(wide[n].dtype == torch.float32 for n in "abh") and wide["i"].dtype == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, model_root):
    cfg = config_from_json(TINY["A"]["config"])
    decls = declared_tensors(cfg.model_spec())
    entries, files = open_model_files(make_model_dir(model_root, "A"))
    tensors = {n: e.file.tensor(n) for n, e in entries.items()}
    for f in files:
        f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 100)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as ei:
        load_weights(tmp_path, decls)
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert e.wrong_shape == [("model.layers.0.mlp.down_proj.weight", (64, 128), (64, 100))]
    msg = str(e)
    assert "missing (2)" in msg and "unexpected (1)" in msg and "[64, 100]" in msg and "[64, 128]" in msg


def test_optional_tensors_may_be_absent(tmp_path, model_root):
    """q/k/v biases are used if the file has them; a tied head needs no tensor of its own."""
    cfg = config_from_json(TINY["A"]["config"])
    decls = declared_tensors(cfg.model_spec())
    entries, files = open_model_files(make_model_dir(model_root, "A"))
    assert "lm_head.weight" not in entries  # tied: the random model holds none
    tensors = {n: e.file.tensor(n) for n, e in entries.items() if not n.endswith("proj.bias")}
    for f in files:
        f.close()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    got = load_weights(tmp_path, decls)
    assert "model.layers.0.self_attn.q_proj.bias" not in got and len(got) == len(tensors)
    # untied: the head's tensor is required
    decls_b = declared_tensors(config_from_json(TINY["B"]["config"]).model_spec())
    assert [d for d in decls_b if d.name == "lm_head.weight"][0].required


def _write_raw(path, header: dict, data: bytes):
    blob = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + data)


def test_malformed_files_are_errors_not_crashes(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too short"):
        open_model_files(tmp_path)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="larger than"):
        open_model_files(tmp_path)
    p.write_bytes(struct.pack("<Q", 100) + b"{}")
    with pytest.raises(SafetensorsError, match="past the end"):
        open_model_files(tmp_path)
    _write_raw(p, {"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 32]}}, b"\0" * 16)
    with pytest.raises(SafetensorsError, match="outside the data section"):
        open_model_files(tmp_path)
    _write_raw(p, {"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}, b"\0" * 16)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        open_model_files(tmp_path)
    _write_raw(p, {"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        open_model_files(tmp_path)
    blob = b'{"x":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"x":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    p.write_bytes(struct.pack("<Q", len(blob)) + blob + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="twice"):
        open_model_files(tmp_path)
    p.unlink()
    with pytest.raises(SafetensorsError, match="no \\*.safetensors"):
        open_model_files(tmp_path)


def test_shards_are_read_together(tmp_path):
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {"a": torch.ones(2)})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {"b": torch.zeros(3)})
    got = load_weights(tmp_path, [TensorDecl("a", (2,)), TensorDecl("b", (3,))], torch.float32)
    assert got["a"].tolist() == [1, 1] and got["b"].tolist() == [0, 0, 0]
    write_safetensors(tmp_path / "model-00003.safetensors", {"a": torch.ones(2)})
    with pytest.raises(SafetensorsError, match="both"):
        open_model_files(tmp_path)


def test_shard_index_is_honoured_and_checked(tmp_path):
    """model.safetensors.index.json, when present, says which shards belong to the model and where each tensor lies."""
    decls = [TensorDecl("a", (2,)), TensorDecl("b", (3,))]

    def index(weight_map, **meta):
        (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": meta, "weight_map": weight_map}))

    write_safetensors(tmp_path / "s1.safetensors", {"a": torch.ones(2)})
    write_safetensors(tmp_path / "s2.safetensors", {"b": torch.zeros(3)})
    index({"a": "s1.safetensors", "b": "s2.safetensors"}, total_size=20)
    got = load_weights(tmp_path, decls, torch.float32)
    assert got["a"].tolist() == [1, 1] and got["b"].tolist() == [0, 0, 0]
    index({"a": "s1.safetensors", "b": "s2.safetensors"}, total_size=24)
    with pytest.raises(SafetensorsError, match="total_size is 24, the shards hold 20"):
        open_model_files(tmp_path)
    index({"a": "s2.safetensors", "b": "s2.safetensors"})
    with pytest.raises(SafetensorsError, match="does not name: s1.safetensors"):
        open_model_files(tmp_path)
    index({"a": "s1.safetensors", "b": "s1.safetensors", "c": "s2.safetensors"})
    with pytest.raises(SafetensorsError, match="tensor 'b' is indexed in s1.safetensors"):
        open_model_files(tmp_path)
    index({"a": "s1.safetensors"})
    with pytest.raises(SafetensorsError, match="does not name: s2.safetensors"):
        open_model_files(tmp_path)
    index({"a": "s1.safetensors", "b": "s2.safetensors", "c": "s2.safetensors"})
    with pytest.raises(SafetensorsError, match="no shard holds: c"):
        open_model_files(tmp_path)
    index({"a": "s1.safetensors", "b": "s3.safetensors"})
    with pytest.raises(SafetensorsError, match="s3.safetensors that it names is missing"):
        open_model_files(tmp_path)
    for bad in ("../s1.safetensors", "/etc/passwd", "s1.bin", 7):
        index({"a": bad, "b": "s2.safetensors"})
        with pytest.raises(SafetensorsError, match="must name a .safetensors file of this folder"):
            open_model_files(tmp_path)
    (tmp_path / "model.safetensors.index.json").write_text("{\"weight_map\": 3}")
    with pytest.raises(SafetensorsError, match="'weight_map' is missing"):
        open_model_files(tmp_path)
    # a single file is read on its own, whatever index lies beside it
    assert set(open_model_files(tmp_path / "s1.safetensors")[0]) == {"a"}


def test_random_weights_depend_on_seed_and_name_only(model_root, tmp_path):
    a = normal_values(7, "x.weight", 1000)
    assert np.array_equal(a, normal_values(7, "x.weight", 1000))
    assert np.array_equal(a[:100], normal_values(7, "x.weight", 100))
    assert not np.array_equal(a, normal_values(8, "x.weight", 1000))
    assert not np.array_equal(a, normal_values(7, "y.weight", 1000))
    big = normal_values(1, "big", 200000)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1.0) < 0.01
    d = make_model_dir(model_root, "B")
    cfg = json.loads((d / "config.json").read_text())
    assert cfg["architectures"] == ["Qwen2ForCausalLM"] and cfg["intermediate_size"] == 200
    entries, files = open_model_files(d)
    w = entries["model.layers.2.input_layernorm.weight"].file.tensor("model.layers.2.input_layernorm.weight")
    assert abs(float(w.mean()) - 1.0) < 0.1  # norm weights are 1 + noise
    assert "lm_head.weight" in entries and entries["lm_head.weight"].shape == (320, 96)
    for f in files:
        f.close()
