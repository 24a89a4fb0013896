"""Random weights made on the device are the weights a folder written on the host holds: the same
(configuration, seed) is the same model, bit for bit, wherever its numbers are made."""
import pytest
import torch

import model_helpers as mh
import tiny_configs
from rust_deeplearning_b200 import Engine, load_model, random_model, write_random_model
from rust_deeplearning_b200.config.base import architecture_for
from rust_deeplearning_b200.weights.loader import load_weights, random_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_device_and_host_make_the_same_weights(tmp_path, name, dtype):
    cfg, seed = tiny_configs.config(name)
    arch = architecture_for(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    torch_dtype = getattr(torch, dtype)
    folder = write_random_model(str(tmp_path / "host"), cfg, seed, dtype)                  # numbers made by numpy
    on_device = random_weights(spec, seed, torch_dtype, "cuda:0")                          # numbers made by the kernel
    from_folder = load_weights(spec, folder, torch_dtype, "cuda:0")
    assert set(on_device) == set(from_folder)
    for n in on_device:
        assert on_device[n].dtype is from_folder[n].dtype
        assert torch.equal(on_device[n], from_folder[n]), f"{n}: host and device values differ"
    names = sorted(on_device)
    same_shape = [(a, b) for a in names for b in names if a < b and on_device[a].shape == on_device[b].shape]
    assert same_shape and all(not torch.equal(on_device[a], on_device[b]) for a, b in same_shape)   # values differ by name
    # a folder written with the numbers made on the device is the same file
    folder2 = write_random_model(str(tmp_path / "device"), cfg, seed, dtype, device="cuda:0")
    assert open(f"{folder}/model.safetensors", "rb").read() == open(f"{folder2}/model.safetensors", "rb").read()
    # and the two models give the same logits, bit for bit
    ids = mh.prompt(900, 21, cfg["vocab_size"])
    out = []
    for model in (random_model(cfg, seed, dtype), load_model(folder, dtype)):
        eng = Engine(model, max_tokens=256)
        out.append(eng.step([eng.new_sequence()], [ids], "all").clone())
    assert torch.equal(out[0], out[1])
