"""Weights: safetensors round trips, the one error that lists everything, random-weights folders (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_gemma2 as plain
import tiny_configs
from rust_deeplearning_b200.config.base import architecture_for
from rust_deeplearning_b200.weights.loader import WeightError, load_weights, random_tensor, stored_dtype
from rust_deeplearning_b200.weights.random_init import write_random_model
from rust_deeplearning_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, WeightFiles, write_safetensors


def spec_of(cfg):
    arch = architecture_for(cfg)
    return arch.build_spec(arch.parse_config(cfg))


def test_safetensors_round_trip_and_format(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
               "empty": torch.zeros(0, 4)}
    path = str(tmp_path / "t.safetensors")
    write_safetensors(path, tensors, {"k": "v"})
    f = SafetensorsFile(path)
    assert f.metadata == {"k": "v"}
    for name, t in tensors.items():
        got = f.tensor(name)
        assert got.dtype == t.dtype and got.shape == t.shape and torch.equal(got, t)
    # the layout is the published one: u64 header length, JSON, data (hub/main/src/core/safetensors.rs:59-87)
    blob = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    b, e = header["a"]["data_offsets"]
    assert np.array_equal(np.frombuffer(blob[8 + hlen + b:8 + hlen + e], dtype="<f4"), tensors["a"].numpy().ravel())
    # and the plain reader of the tests reads what the library wrote
    floats = str(tmp_path / "floats.safetensors")
    write_safetensors(floats, {"a": tensors["a"], "b": tensors["b"]})
    assert np.allclose(plain.read_safetensors(floats)["b"], tensors["b"].double().numpy())


def test_broken_files_are_refused(tmp_path):
    path = str(tmp_path / "t.safetensors")
    write_safetensors(path, {"a": torch.randn(4, 4)})
    blob = bytearray(open(path, "rb").read())
    (hlen,) = struct.unpack("<Q", blob[:8])
    for mutate, what in (
        (lambda b: b[:20], "short"),
        (lambda b: struct.pack("<Q", 10 ** 9) + b[8:], "header length"),
        (lambda b: b[:-8], "data range"),
        (lambda b: b[:8] + b"{" * hlen + b[8 + hlen:], "JSON"),
    ):
        bad = str(tmp_path / "bad.safetensors")
        open(bad, "wb").write(bytes(mutate(bytes(blob))))
        with pytest.raises(SafetensorsError):
            SafetensorsFile(bad)
    with pytest.raises(SafetensorsError):
        WeightFiles(str(tmp_path / "nothing_here"))
    # header entries with sizes that are no whole numbers, negative, or too large for 64 bits; names that are no strings
    import json
    header = json.loads(blob[8:8 + hlen])
    for key, value in (("shape", [2 ** 70]), ("shape", [-4, -4]), ("shape", [1.5, 4]), ("shape", "4x4"), ("shape", [True, 16]),
                       ("data_offsets", [0, 2 ** 70]), ("data_offsets", [0.0, 64.0]), ("data_offsets", [5]), ("dtype", ["F32"]),
                       ("dtype", None)):
        h = json.loads(json.dumps(header))
        h["a"][key] = value
        hb = json.dumps(h).encode()
        bad = str(tmp_path / "bad_entry.safetensors")
        open(bad, "wb").write(struct.pack("<Q", len(hb)) + hb + bytes(blob[8 + hlen:]))
        with pytest.raises(SafetensorsError):
            SafetensorsFile(bad)


@pytest.mark.parametrize("name", ["A", "B"])
def test_random_model_folder_is_reproducible_and_loads(tmp_path, name):
    cfg, seed = tiny_configs.config(name)
    a = write_random_model(str(tmp_path / "a"), cfg, seed, "bfloat16")
    b = write_random_model(str(tmp_path / "b"), cfg, seed, "bfloat16")
    c = write_random_model(str(tmp_path / "c"), cfg, seed + 1, "bfloat16")
    ra, rb, rc = (open(os.path.join(d, "model.safetensors"), "rb").read() for d in (a, b, c))
    assert ra == rb and ra != rc
    assert json.load(open(os.path.join(a, "config.json")))["torch_dtype"] == "bfloat16"
    spec = spec_of(cfg)
    w16 = load_weights(spec, a, torch.bfloat16, "cpu")
    w32 = load_weights(spec, a, torch.float32, "cpu")
    assert set(w16) == set(spec.tensor_specs())
    for n, t in spec.tensor_specs().items():
        assert w16[n].dtype is torch.bfloat16 and w32[n].dtype is torch.float32 and tuple(w16[n].shape) == t.shape
        assert torch.equal(w16[n].float(), w32[n])
    std = w32["model.layers.0.mlp.up_proj.weight"].std().item()
    assert 0.015 < std < 0.025                                     # N(0, 0.02)
    # a tensor's values depend on (seed, its name) only
    t = spec.tensor_specs()["model.norm.weight"]
    assert torch.equal(random_tensor(t, seed, torch.bfloat16), w16["model.norm.weight"])


def test_a_vector_stored_in_32_bits_stays_32_bit(tmp_path):
    cfg, seed = tiny_configs.config("A")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed, "bfloat16")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    del f
    write_safetensors(path, tensors)
    spec = spec_of(cfg)
    w = load_weights(spec, folder, torch.bfloat16, "cpu")
    assert w["model.norm.weight"].dtype is torch.float32
    assert w["model.layers.0.input_layernorm.weight"].dtype is torch.bfloat16
    assert w["model.embed_tokens.weight"].dtype is torch.bfloat16
    assert stored_dtype(spec.tensor_specs()["model.embed_tokens.weight"], "F32", torch.bfloat16) is torch.bfloat16


def test_one_error_lists_missing_unexpected_and_misshaped(tmp_path):
    cfg, seed = tiny_configs.config("A")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed, "float32")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.bias_q"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(path, tensors)
    with pytest.raises(WeightError) as e:
        load_weights(spec_of(cfg), folder, torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.bias_q"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    assert [w[0] for w in err.wrong_dtype] == ["model.layers.0.input_layernorm.weight"]
    text = str(err)
    for piece in ("missing (2)", "unexpected (1)", "expected [64, 64], file has [64, 63]", "wrong dtype"):
        assert piece in text


def test_declared_extras_are_skipped_and_others_only_warn_when_asked(tmp_path):
    """Buffers the architecture declares (rotary frequencies, the head's copy of a tied table) load
    silently; any other extra tensor is an error by default and a listed warning with strict=False
    (the reference warns and skips: rustml/nlp/main/src/core/weight_map.rs:360-362)."""
    cfg, seed = tiny_configs.config("A")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed, "float32")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(path, tensors)
    spec = spec_of(cfg)
    w = load_weights(spec, folder, torch.float32, "cpu")
    assert set(w) == set(spec.tensor_specs())
    tensors["something.else"] = torch.zeros(3)
    write_safetensors(path, tensors)
    with pytest.raises(WeightError) as e:
        load_weights(spec, folder, torch.float32, "cpu")
    assert e.value.unexpected == ["something.else"]
    with pytest.warns(UserWarning, match="something.else"):
        w = load_weights(spec, folder, torch.float32, "cpu", strict=False)
    assert set(w) == set(spec.tensor_specs())
    # an untied model reads lm_head.weight, so there it is not an extra
    untied = dict(cfg, tie_word_embeddings=False)
    assert "lm_head.weight" in spec_of(untied).tensor_specs() and "lm_head.weight" not in spec_of(untied).ignored_tensors


def test_random_values_depend_on_seed_name_and_index_only():
    """Counter-based values: a prefix of a longer tensor with the same key is the shorter tensor; two
    names or two seeds give different numbers; the numbers are N(0, std)."""
    from rust_deeplearning_b200.parts.spec import TensorSpec
    from rust_deeplearning_b200.weights import counter_random as cr
    a = random_tensor(TensorSpec("x.weight", (40, 50)), 3, torch.float32)
    again = random_tensor(TensorSpec("x.weight", (40, 50)), 3, torch.float32)
    longer = random_tensor(TensorSpec("x.weight", (80, 50)), 3, torch.float32)
    assert torch.equal(a, again) and torch.equal(a, longer[:40])
    assert not torch.equal(a, random_tensor(TensorSpec("y.weight", (40, 50)), 3, torch.float32))
    assert not torch.equal(a, random_tensor(TensorSpec("x.weight", (40, 50)), 4, torch.float32))
    odd = cr.normal(7, cr.tensor_key(3, "x.weight"), 0.02)
    assert np.array_equal(odd, a.reshape(-1)[:7].numpy())
    big = cr.normal(200001, cr.tensor_key(0, "z"), 0.5).astype(np.float64)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 0.5) < 0.01
    assert abs(np.mean(big ** 4) / big.var() ** 2 - 3.0) < 0.1          # the fourth moment of a normal
    # bfloat16 is the float32 value rounded to nearest even
    assert torch.equal(random_tensor(TensorSpec("x.weight", (40, 50)), 3, torch.bfloat16), a.to(torch.bfloat16))


def test_sharded_folder(tmp_path):
    cfg, seed = tiny_configs.config("A")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed, "bfloat16")
    single = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(single)
    names = sorted(f.names())
    shards = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    weight_map = {}
    for shard, members in shards.items():
        write_safetensors(os.path.join(folder, shard), {n: f.tensor(n).clone() for n in members})
        weight_map.update({n: shard for n in members})
    whole = {n: f.tensor(n).clone() for n in names}
    del f
    os.remove(single)
    json.dump({"weight_map": weight_map}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    w = load_weights(spec_of(cfg), folder, torch.bfloat16, "cpu")
    assert all(torch.equal(w[n], whole[n]) for n in names)
