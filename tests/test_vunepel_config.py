"""The Vunepel design without a GPU: configuration, spec, tensor names, what may be absent, refusals, and hand-made
numbers for the plain mechanisms that the GPU tests use as their oracle."""
import json
import math

import pytest
import torch

import plain_vunepel as plain
from qwen_triton_b200 import config_from_dict, load_config, load_preset, write_random_model
from qwen_triton_b200.config import ConfigError, VunepelConfig
from qwen_triton_b200.engine.model import expected_tensors


def raw_config():
    return json.loads(json.dumps(load_preset("vunepel-tiny-a").to_hf_dict()))


def test_presets_parse_and_round_trip():
    for name in ("vunepel-tiny-a", "vunepel-tiny-b"):
        config = load_preset(name)
        assert isinstance(config, VunepelConfig)
        assert config_from_dict(config.to_hf_dict()) == config
        spec = config.model_spec()
        assert [layer.block.kind for layer in spec.layers] == ["parallel"] * len(config.layers)
        assert spec.final_norm.kind == "dynamic_tanh"


def test_spec_names_the_parts_and_the_shared_cache():
    config = load_preset("vunepel-tiny-a")
    spec = config.model_spec()
    assert [layer.mixer.kind for layer in spec.layers] == ["gated_delta_rule", "attention", "gated_delta_rule", "attention"]
    assert [layer.feed_forward.kind if layer.feed_forward else None for layer in spec.layers] == ["gated_mlp", "routed_experts", None, "routed_experts"]
    assert [call.cache_of for call in spec.schedule] == [None, None, None, 1]
    reader = spec.layers[3].mixer
    assert reader["own_kv"] is False and reader["chunk"] == 33 and reader["maps"] == 2
    assert spec.layers[1].mixer["position"].kind == "rope" and spec.layers[1].mixer["position"]["rotary_dim"] == 8


def test_tensor_names_and_shapes():
    names = expected_tensors(load_preset("vunepel-tiny-a").model_spec())
    assert tuple(names["embed"].shape) == (193, 128) and tuple(names["head"].shape) == (193, 128)
    assert tuple(names["final.norm.alpha"].shape) == () and tuple(names["l0.norm1.b"].shape) == (128,)
    assert tuple(names["l0.mix.q"].shape) == (16, 128) and tuple(names["l0.mix.v.conv"].shape) == (64, 3)
    assert tuple(names["l0.mix.a1"].shape) == (8, 128) and tuple(names["l0.mix.a2"].shape) == (32, 8)
    assert tuple(names["l0.mix.g2"].shape) == (64, 12) and tuple(names["l0.mix.A_log"].shape) == (2,)
    assert tuple(names["l1.mix.q"].shape) == (2 * 2 * 16, 128) and tuple(names["l1.mix.k"].shape) == (1 * 2 * 16, 128)
    assert tuple(names["l1.mix.v"].shape) == (48, 128) and tuple(names["l1.mix.lq2"].shape) == (16,)
    assert tuple(names["l1.mlp.e3.down"].shape) == (128, 64) and tuple(names["l1.mlp.shared.sg"].shape) == (1, 128)
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and "l3.mix.k.norm" not in names and "l3.mix.q.norm" in names
    assert not any(name.startswith("l2.mlp") for name in names) and "l3.mlp.shared.gate" not in names
    assert not any(name.endswith(".weight") for name in names)


def test_narrow_projections_are_sized_by_the_stored_tensors(tmp_path):
    config = load_preset("vunepel-tiny-a")
    write_random_model(tmp_path, config, seed=1, dtype=torch.float32)
    bare = raw_config()
    for layer in bare["layers"]:
        layer["mixer"].pop("ranks", None)
    with pytest.raises(ConfigError, match="narrow projections"):
        config_from_dict(bare).model_spec()
    (tmp_path / "config.json").write_text(json.dumps(bare))
    assert load_config(tmp_path) == config


def test_what_may_be_absent():
    raw = raw_config()
    del raw["layers"][1]["mixer"]["rot"], raw["layers"][1]["mixer"]["mask"], raw["layers"][3]["mixer"]["rot"]
    raw["layers"][1]["mlp"].pop("shared")
    config = config_from_dict(raw)
    assert config.layers[1].rot_dims == 0 and config.layers[1].chunk is None and config.layers[1].mlp.shared_ff == 0
    spec = config.model_spec()
    assert spec.layers[1].mixer["position"].kind == "none" and spec.layers[1].mixer["chunk"] is None
    assert "l1.mlp.shared.sg" not in expected_tensors(spec)


@pytest.mark.parametrize("change, message", [
    (lambda raw: raw["layers"][0].update(type="convolution"), "no mixer"),
    (lambda raw: raw["layers"][0]["mlp"].update(kind="glu"), "no feed-forward"),
    (lambda raw: raw["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda raw: raw["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda raw: raw["layers"][3]["mixer"].update(heads=4), "differ"),
    (lambda raw: raw["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda raw: raw["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda raw: raw["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda raw: raw["norm"].pop("eps"), "norm.eps"),
])
def test_refusals(change, message):
    raw = raw_config()
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


# ----------------------------------------------------------------------------- the plain mechanisms, by hand
def test_plain_dynamic_tanh_and_capped_gate():
    x = torch.tensor([[0.0, 1.0, -2.0]], dtype=torch.float64)
    y = plain.dynamic_tanh(x, torch.tensor([2.0, 2.0, 2.0]), torch.tensor([0.5, 0.0, 0.0]), 0.5)
    assert torch.allclose(y, torch.tensor([[0.5, 2 * math.tanh(0.5), 2 * math.tanh(-1.0)]], dtype=torch.float64))
    g, u = torch.tensor([5.0, -1.0]), torch.tensor([-9.0, 0.5])
    y = plain.clamped_gate(g.double(), u.double(), 2.0)
    assert math.isclose(float(y[0]), 2.0 / (1 + math.exp(-3.404)) * (-2.0 + 1.0))
    assert math.isclose(float(y[1]), -1.0 / (1 + math.exp(1.702)) * 1.5)


def test_plain_short_convolution_and_rotation():
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    taps = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)          # the last column is the current token's
    assert plain.short_conv(x, taps).flatten().tolist() == [1.0, 12.0, 124.0]
    v = torch.tensor([[[1.0, 0.0, 7.0]]], dtype=torch.float64)               # two dims rotate, the third passes
    turned = plain.rotate(v, torch.tensor([1]), 2, 10000.0)
    assert torch.allclose(turned, torch.tensor([[[math.cos(1.0), math.sin(1.0), 7.0]]], dtype=torch.float64))


def test_plain_delta_rule_reads_its_own_write():
    """One head, one channel pair: after a single token with beta = 1 and a unit key the read-out along the key is v."""
    tensors = {"m.q": torch.eye(2), "m.k": torch.eye(2), "m.v": torch.eye(2), "m.b": torch.full((1, 2), 50.0), "m.a1": torch.zeros(1, 2),
               "m.a2": torch.zeros(2, 1), "m.dt_bias": torch.zeros(2), "m.A_log": torch.zeros(1), "m.g1": torch.zeros(1, 2),
               "m.g2": torch.zeros(2, 1), "m.norm": torch.ones(2), "m.o": torch.eye(2),
               "m.q.conv": torch.ones(2, 1), "m.k.conv": torch.ones(2, 1), "m.v.conv": torch.ones(2, 1)}
    h = torch.tensor([[3.0, 0.0]], dtype=torch.float64)
    out = plain.channel_delta(h, tensors, "m", {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2}, 1e-12)
    # q = k = silu(3) e0 made unit (q also over sqrt 2), v = silu(h): o = (k . q) v, then unit rms, then the gate sigmoid(0)
    silu3 = 3.0 / (1 + math.exp(-3.0))
    o = torch.tensor([silu3, 0.0], dtype=torch.float64) / math.sqrt(2.0)
    want = o / torch.sqrt((o * o).mean()) * 0.5
    assert torch.allclose(out[0], want, atol=1e-5)


def test_plain_chunks_and_the_difference_of_maps():
    """With zero queries every visible key weighs the same: position 5 of chunks of 4 averages the values of 4 and 5."""
    dim, vdim = 2, 2
    tensors = {"m.q": torch.zeros(2 * dim, 3), "m.q.norm": torch.ones(dim), "m.o": torch.eye(vdim),
               "m.lq1": torch.zeros(dim), "m.lk1": torch.zeros(dim), "m.lq2": torch.zeros(dim), "m.lk2": torch.zeros(dim)}
    mixer = {"heads": 1, "kv_heads": 1, "dim": dim, "vdim": vdim, "scale": 1.0, "diff": 0.25, "mask": {"size": 4}}
    tokens = 7
    keys = torch.zeros(tokens, 1, 2, dim, dtype=torch.float64)
    values = torch.arange(tokens, dtype=torch.float64)[:, None, None] * torch.tensor([1.0, -1.0], dtype=torch.float64)
    out = plain.differential_attention(torch.zeros(tokens, 3, dtype=torch.float64), tensors, "m", mixer, 1e-12, (keys, values))
    # lambda = 1 - 1 + 0.25: o = 0.75 * mean; unit rms of (a, -a) is (1, -1); times 1 - diff
    assert torch.allclose(out[5], torch.tensor([0.75, -0.75], dtype=torch.float64))
    assert torch.allclose(out[4], torch.tensor([0.75, -0.75], dtype=torch.float64))       # alone in its chunk so far


def test_plain_router_weights():
    tensors = {"f.router": torch.tensor([[1.0], [0.0], [-1.0]])}
    for e in range(3):
        tensors[f"f.e{e}.gate"] = torch.full((1, 1), 10.0)
        tensors[f"f.e{e}.up"] = torch.zeros(1, 1)
        tensors[f"f.e{e}.down"] = torch.full((1, 1), float(e + 1))
    mlp = {"kind": "moe", "router": {"experts": 3, "top": 2, "scale": 3.0}, "expert": {"ff": 1, "limit": 1.0}, "shared": None}
    out = plain.routed_ff(torch.ones(1, 1, dtype=torch.float64), tensors, "f", mlp)
    s0, s1 = 1 / (1 + math.exp(-1.0)), 0.5
    y = 1.0 / (1 + math.exp(-1.702))                     # g capped at 1, u = 0: sigmoid(1.702) * 1
    want = 3.0 * (s0 * 1.0 + s1 * 2.0) / (s0 + s1) * y
    assert math.isclose(float(out), want, rel_tol=1e-9)
