"""The safetensors container, binding by name, the one error message, random weights (no GPU)."""
import json
import os
import struct

import pytest
import torch

import tiny_models as tm
from litellmengine_b200.config import config_from_dict, load_config
from litellmengine_b200.parts import model_parameters
from litellmengine_b200.weights import (DictSource, ParamSpec, RandomSource, SafetensorsError,
                                        SafetensorsFile, SafetensorsSource, WeightError, bind_weights,
                                        write_random_model, write_safetensors)


def test_container_round_trip(tmp_path):
    t = {"a": torch.arange(6, dtype=torch.float32).view(2, 3), "b": torch.ones(4, dtype=torch.bfloat16) * 1.5,
         "idx": torch.tensor([1, 2, 3], dtype=torch.int64), "s": torch.tensor(2.0)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, {"k": "v"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
    for n in t:
        assert f.dtype(n) == t[n].dtype and f.shape(n) == tuple(t[n].shape) and torch.equal(f.tensor(n), t[n])
    # the layout is the public one: 8-byte length, JSON, data
    raw = open(path, "rb").read()
    (n,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + n])
    assert hdr["a"] == {"dtype": "F32", "shape": [2, 3], "data_offsets": hdr["a"]["data_offsets"]}


def test_container_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 2]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 2)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))
    empty = tmp_path / "empty_folder"
    empty.mkdir()
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        SafetensorsSource(str(empty))


def test_one_error_lists_everything_wrong():
    cfg = tm.TINY_B
    params = model_parameters(config_from_dict(cfg).plan())
    w = tm.make_weights(cfg, 1)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(3, 3)
    w["model.layers.9.extra.weight"] = torch.zeros(1)
    with pytest.raises(WeightError) as e:
        bind_weights(params, DictSource(w), torch.float32, "cpu", where="unit")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (192, 96), (3, 3))]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (1)", "expected [192, 96], found [3, 3]", "unit"):
        assert needle in text


def test_untied_model_needs_its_head_and_tied_model_aliases():
    pb = model_parameters(config_from_dict(tm.TINY_B).plan())
    w = tm.make_weights(tm.TINY_B, 1)
    del w["lm_head.weight"]
    with pytest.raises(WeightError) as e:
        bind_weights(pb, DictSource(w), torch.float32, "cpu")
    assert e.value.missing == ["lm_head.weight"]
    pa = model_parameters(config_from_dict(tm.TINY_A).plan())
    out = bind_weights(pa, DictSource(tm.make_weights(tm.TINY_A, 0)), torch.float32, "cpu")
    assert out["lm_head.weight"] is out["model.embed_tokens.weight"]
    # a tied model that does ship a head uses it
    wa = tm.make_weights(tm.TINY_A, 0)
    wa["lm_head.weight"] = torch.zeros(256, 64)
    out = bind_weights(pa, DictSource(wa), torch.float32, "cpu")
    assert out["lm_head.weight"].abs().sum() == 0


def test_stored_types_are_kept():
    params = {"m": ParamSpec((2, 2)), "m32": ParamSpec((2, 2)), "n": ParamSpec((2,), role="scale"),
              "i": ParamSpec((2,), role="index"), "h": ParamSpec((2, 2))}
    src = DictSource({"m": torch.ones(2, 2, dtype=torch.bfloat16), "m32": torch.ones(2, 2),
                      "n": torch.ones(2, dtype=torch.bfloat16), "i": torch.tensor([1, 2], dtype=torch.int64),
                      "h": torch.ones(2, 2, dtype=torch.float16)})
    out = bind_weights(params, src, torch.bfloat16, "cpu")
    assert out["m"].dtype == torch.bfloat16          # bfloat16 stays bfloat16
    assert out["m32"].dtype == torch.float32         # stored in 32-bit stays so
    assert out["n"].dtype == torch.float32           # norm weights multiply in 32-bit
    assert out["i"].dtype == torch.int32             # integer tables as int32
    assert out["h"].dtype == torch.float32
    out = bind_weights(params, src, torch.float32, "cpu")
    assert all(out[k].dtype == torch.float32 for k in ("m", "m32", "n", "h"))
    with pytest.raises(WeightError, match="integer table"):
        bind_weights({"i": ParamSpec((2,), role="index")}, DictSource({"i": torch.ones(2)}), torch.float32, "cpu")


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    cfg = config_from_dict(tm.TINY_A)
    d = write_random_model(cfg, str(tmp_path / "m"), seed=5, dtype=torch.bfloat16)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert load_config(d) == cfg
    src = SafetensorsSource(d)
    params = model_parameters(cfg.plan())
    assert "lm_head.weight" not in src.names()       # tied: the head is not stored
    out = bind_weights(params, src, torch.bfloat16, "cpu")
    q = out["model.layers.0.self_attn.q_proj.weight"].float()
    assert q.dtype == torch.float32 and abs(float(q.std()) - 0.02) < 0.002 and abs(float(q.mean())) < 0.002
    n = out["model.norm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.01 and 0.003 < float(n.std()) < 0.02
    # seeded: same seed same numbers, other seed other numbers; one tensor does not depend on the rest
    again = RandomSource(params, 5, torch.bfloat16).get("model.layers.1.mlp.down_proj.weight")
    assert torch.equal(again, out["model.layers.1.mlp.down_proj.weight"])
    other = RandomSource(params, 6, torch.bfloat16).get("model.layers.1.mlp.down_proj.weight")
    assert not torch.equal(other, again)
    alone = RandomSource({"model.norm.weight": params["model.norm.weight"]}, 5, torch.float32).get("model.norm.weight")
    assert torch.equal(alone.to(torch.bfloat16).float(), n)


def test_a_folder_of_shards(tmp_path):
    """Several files: those the index names if there is one, else every *.safetensors; a tensor
    that two files hold is refused by name, and so is a folder without any."""
    a = {"w1": torch.ones(2, 2), "w2": torch.zeros(3)}
    b = {"w3": torch.full((2,), 7.0)}
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), a)
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    src = SafetensorsSource(str(tmp_path))
    assert sorted(src.names()) == ["w1", "w2", "w3"] and torch.equal(src.get("w3"), b["w3"]) and src.shape("w1") == (2, 2)
    # a stray file beside the shards is read too, unless an index says which files belong to the model
    write_safetensors(str(tmp_path / "stray.safetensors"), {"w1": torch.ones(2, 2)})
    with pytest.raises(SafetensorsError, match="'w1' is in both"):
        SafetensorsSource(str(tmp_path))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        "w1": "model-00001-of-00002.safetensors", "w2": "model-00001-of-00002.safetensors",
        "w3": "model-00002-of-00002.safetensors"}}))
    assert sorted(SafetensorsSource(str(tmp_path)).names()) == ["w1", "w2", "w3"]
    (tmp_path / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(SafetensorsError, match="no weight_map"):
        SafetensorsSource(str(tmp_path))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(SafetensorsError, match="no .safetensors file"):
        SafetensorsSource(str(empty))
    with pytest.raises(SafetensorsError, match="cannot list"):
        SafetensorsSource(str(tmp_path / "nowhere"))
