"""Configuration, spec, tensor names and random weights of the Lederax design (no device needed)."""
import copy

import pytest
import torch

import plain_lederax as plain
from qwen_triton_b200.config import ConfigError, LederaxConfig, config_from_dict, load_preset
from qwen_triton_b200.engine.model import expected_tensors
from qwen_triton_b200.weights import Checkpoint, WeightsError, open_checkpoint, random_tensor, write_random_model

RAW = {
    "architecture": "Lederax", "vocab": 50, "width": 48, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5, "groups": 4},
    "layers": [
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16, "scale": 0.3, "mask": {"size": 5}, "v_mix": False}},
        {"type": "attention", "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 24}},
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.2, "v_mix": True}},
        {"type": "attention", "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 8}},
         "mixer": {"heads": 3, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.4, "mask": {"size": 9}, "v_mix": True}},
    ],
}


def test_registry_reads_the_single_architecture_name_and_round_trips():
    config = config_from_dict(RAW)
    assert isinstance(config, LederaxConfig)
    assert (config.vocab_size, config.hidden_size, config.num_hidden_layers) == (50, 48, 3)
    assert config.layers[0].window == 5 and config.layers[1].window is None and config.layers[0].mlp is None
    assert config_from_dict(config.to_hf_dict()) == config
    for name in ("lederax-tiny-a", "lederax-tiny-b"):
        preset = load_preset(name)
        assert config_from_dict(preset.to_hf_dict()) == preset


def test_spec_carries_every_constant_as_a_parameter():
    spec = config_from_dict(RAW).model_spec()
    assert spec.embedding["scale"] == 3.0 and spec.final_norm["groups"] == 4 and spec.final_norm["name"] == "final.norm"
    first, second, third = (layer.mixer for layer in spec.layers)
    assert (first["v_blend"], second["v_blend"], third["v_blend"]) == (None, "source", "blend")
    assert first["window"] == 5 and second["window"] is None
    assert (second["head_dim"], second["v_head_dim"], second["scale"]) == (16, 8, 0.2)
    assert spec.layers[0].feed_forward is None and spec.layers[2].feed_forward["top"] == 1


def test_tensor_names_shapes_and_what_may_be_absent():
    expected = expected_tensors(config_from_dict(RAW).model_spec())
    assert tuple(expected["embed"].shape) == (50, 48) and tuple(expected["head"].shape) == (50, 48)
    assert tuple(expected["l0.mix.q"].shape) == (32, 48) and tuple(expected["l0.mix.v"].shape) == (32, 48)
    assert tuple(expected["l0.mix.o"].shape) == (48, 64) and tuple(expected["l0.mix.k.b"].shape) == (16,)
    assert "l0.mix.o.b" not in expected and tuple(expected["l1.mix.r1"].shape) == (2,)
    assert expected["l1.mlp.table"].role == "table" and tuple(expected["l1.mlp.table"].shape) == (50, 2)
    assert tuple(expected["l1.mlp.e2.up"].shape) == (24, 48) and tuple(expected["l1.mlp.e2.down"].shape) == (48, 24)
    assert "l1.mlp.e3.up" not in expected and "l0.mlp.table" not in expected
    # the blend weight is read only by the layers that blend; the norm of a missing feed-forward is read past
    assert expected["l0.mix.vmix"].optional and expected["l1.mix.vmix"].optional and not expected["l2.mix.vmix"].optional
    assert expected["l0.norm2"].optional and not expected["l1.norm2"].optional and tuple(expected["final.norm"].shape) == (48,)


@pytest.mark.parametrize("change, words", [
    (lambda r: r["layers"][0].update(type="recurrent"), "no mixer"),
    (lambda r: r["layers"][1]["mlp"].update(kind="dense"), "no feed-forward"),
    (lambda r: r["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda r: r["norm"].update(groups=5), "does not divide"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=16), "cannot share values"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=4), "top=4"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "lacks"),
    (lambda r: r.pop("vocab"), "lacks"),
])
def test_what_the_design_does_not_have_is_refused_in_words(change, words):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError, match=words):
        config_from_dict(raw)


def test_random_tables_name_distinct_experts_and_models_round_trip(tmp_path):
    config = config_from_dict(RAW)
    expected = expected_tensors(config.model_spec())
    table = random_tensor("l1.mlp.table", expected["l1.mlp.table"], 7, torch.int32)
    assert table.dtype == torch.int32 and tuple(table.shape) == (50, 2)
    assert int(table.min()) >= 0 and int(table.max()) <= 2 and bool((table[:, 0] != table[:, 1]).all())
    assert len({tuple(row) for row in table.tolist()}) > 1
    assert torch.equal(table, random_tensor("l1.mlp.table", expected["l1.mlp.table"], 7, torch.int32))
    folder = write_random_model(tmp_path / "m", config, seed=3, dtype=torch.float32)
    source = open_checkpoint(folder, expected)
    assert source("l0.norm2") is None and tuple(source("l2.mix.vmix").shape) == ()
    checkpoint = Checkpoint(folder)
    weights = {name: checkpoint.read(name) for name in checkpoint.names()}
    assert bool((weights["l1.mix.r2"] > 0).all())
    logits, layers = plain.forward(config.to_hf_dict(), weights, [1, 2, 3, 4, 5, 6, 7], return_layers=True)
    assert tuple(logits.shape) == (7, 50) and tuple(layers.shape) == (3, 7, 48) and bool(torch.isfinite(logits).all())
    # a tensor the design does not have is an error, not something read past
    from qwen_triton_b200.weights import write_safetensors
    weights["l0.mix.o.b"] = torch.zeros(48)
    write_safetensors(folder / "model.safetensors", weights)
    with pytest.raises(WeightsError, match="unexpected"):
        open_checkpoint(folder, expected)


def test_plain_mechanisms_on_hand_made_numbers():
    x = torch.tensor([[3.0, 4.0, 0.0, 5.0]])
    normed = plain.group_rms_norm(x, torch.tensor([1.0, 1.0, 2.0, 2.0]), 2, 0.0)
    assert torch.allclose(normed, torch.tensor([[3.0, 4.0, 0.0, 10.0]]) / (12.5 ** 0.5))
    assert torch.allclose(plain.unit_rms(torch.tensor([1.0, -1.0, 1.0, -1.0]), 0.0), torch.tensor([1.0, -1.0, 1.0, -1.0]))
    penalty = plain.distance_penalty(torch.tensor([2.0]), torch.tensor([0.5]), 3)
    assert torch.allclose(penalty[0, 2], torch.tensor([2.0 * torch.log(torch.tensor(2.0)), 2.0 * torch.log(torch.tensor(1.5)), 0.0]))
    seen = plain.visible(5, 2)
    assert seen[4].tolist() == [False, False, False, True, True] and seen[0].tolist() == [True, False, False, False, False]
    assert plain.visible(3, None)[2].tolist() == [True, True, True]
