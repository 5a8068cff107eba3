"""serialize.py, one test per behaviour of rust-nn src/serialize.rs:300-440: the rnnb byte format, model save / load,
the safetensors export / import."""
import pytest
import torch

from rust_neural_network_b200 import nn, serialize as S


def test_serialize_deserialize_round_trip():
    t1 = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    t2 = torch.tensor([5.0, 6.0])
    loaded = S.deserialize(S.serialize([("weight", t1), ("bias", t2)]))
    assert len(loaded) == 2
    assert loaded[0][0] == "weight" and tuple(loaded[0][1].shape) == (2, 2)
    assert loaded[0][1].reshape(-1).tolist() == [1.0, 2.0, 3.0, 4.0]
    assert loaded[1][0] == "bias" and loaded[1][1].tolist() == [5.0, 6.0]


def test_save_load_model_round_trip():
    model = nn.Sequential().add(nn.Linear(4, 8)).add(nn.ReLU()).add(nn.Linear(8, 2))
    before = [p.detach().clone() for p in model.parameters()]
    blob = S.save_model(model)
    assert blob.startswith(b"RNNB")
    with torch.no_grad():
        for p in model.parameters():
            p.zero_()
    assert S.load_model(model, blob) == len(before)
    for a, b in zip(before, model.parameters()):
        assert torch.equal(a, b.detach())


def test_safetensors_export_import_round_trip():
    t1 = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    t2 = torch.arange(5.0, 11.0).reshape(2, 3)
    loaded = dict(S.safetensors_import(S.safetensors_export([("layer1.weight", t1), ("layer2.weight", t2)])))
    assert len(loaded) == 2
    assert tuple(loaded["layer1.weight"].shape) == (2, 2) and torch.equal(loaded["layer1.weight"], t1)
    assert tuple(loaded["layer2.weight"].shape) == (2, 3) and torch.equal(loaded["layer2.weight"], t2)


def test_empty_model():
    blob = S.serialize([])
    assert blob.startswith(b"RNNB")
    assert S.deserialize(blob) == []


def test_3d_tensors_keep_their_shape():
    loaded = S.deserialize(S.serialize([("x", torch.ones(2, 3, 4))]))
    assert tuple(loaded[0][1].shape) == (2, 3, 4)


def test_safetensors_one_element_tensor():
    loaded = S.safetensors_import(S.safetensors_export([("scalar", torch.tensor([42.0]))]))
    assert loaded[0][0] == "scalar" and loaded[0][1].tolist() == [42.0]


def test_invalid_magic_is_rejected():
    with pytest.raises(S.SerializationError):
        S.deserialize(b"XXXXrest of data")


def test_file_io_round_trip(tmp_path):
    model = nn.Sequential().add(nn.Linear(3, 5))
    path = str(tmp_path / "m.rnnb")
    S.write_file(path, S.save_model(model))
    assert S.load_model(model, S.read_file(path)) == 2


def test_save_model_named_uses_the_callers_names():
    model = nn.Sequential().add(nn.Linear(3, 5))
    loaded = S.deserialize(S.save_model_named(model, ["weight", "bias"]))
    assert [n for n, _ in loaded] == ["weight", "bias"]
    short = S.deserialize(S.save_model_named(model, ["weight"]))   # a short list: the rest keep their default names
    assert [n for n, _ in short] == ["weight", "param_1"]
