"""Vunepel models drawn at random from what config.json allows (sizes, head counts, the order and number of layers,
chunks, rotations, convolutions, narrow projections, experts; widths, head sizes and expert sizes off 8 among them,
layers without a feed-forward, readers of another layer's keys and values), each run whole, token by token, in portions
and as an unequal batch in both types against the plain implementation."""
import random
import tempfile
from pathlib import Path

import pytest
import torch

import plain_vunepel as plain
from qwen_triton_b200 import Engine, StepEntry, config_from_dict, write_random_model
from qwen_triton_b200.weights import Checkpoint, write_safetensors
from test_gpu_vunepel import STORE, close

pytestmark = pytest.mark.gpu


def draw_feed_forward(rng):
    kind = rng.random()
    if kind < 0.15:
        return None
    if kind < 0.45:
        return {"kind": "dense", "ff": rng.choice([8, 20, 48, 96, 136, 256]), "limit": rng.choice([0.5, 1.0, 2.0, 7.0])}
    experts = rng.randint(1, 9)
    mlp = {"kind": "moe", "router": {"experts": experts, "top": rng.randint(1, min(experts, 4)), "scale": rng.choice([1.0, 1.5, 2.5])},
           "expert": {"ff": rng.choice([8, 20, 48, 96, 136]), "limit": rng.choice([0.5, 1.0, 2.0, 7.0])}}
    if rng.random() < 0.6:
        mlp["shared"] = {"ff": rng.choice([8, 24, 64, 100]), "limit": rng.choice([1.0, 3.0])}
    return mlp


def draw(seed: int) -> dict:
    rng = random.Random(1000 + seed)
    width = rng.choice([36, 40, 64, 72, 96, 100, 128, 200])
    layers, owners = [], []
    for index in range(rng.randint(1, 6)):
        if rng.random() < 0.5:
            kv_heads = rng.choice([1, 2, 3])
            dim = rng.choice([4, 8, 12, 16, 20, 32, 64, 72, 128])
            mixer = {"heads": kv_heads * rng.choice([1, 2, 4]), "kv_heads": kv_heads, "dim": dim,
                     "vdim": rng.choice([4, 8, 16, 24, 40, 64, 100, 128]), "conv": rng.choice([1, 2, 3, 4, 4, 5, 8]),
                     "ranks": {"decay": rng.choice([1, 3, 8, 24]), "gate": rng.choice([1, 4, 8, 17])}}
            layers.append({"type": "channel_delta", "mixer": mixer, "mlp": draw_feed_forward(rng)})
            continue
        if owners and rng.random() < 0.35:                   # reads the keys and values of an earlier layer
            source = rng.choice(owners)
            mixer = dict(layers[source]["mixer"])
            mixer["kv_from"] = source
            mixer.pop("mask", None)
        else:
            kv_heads = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 64, 128])
            mixer = {"heads": kv_heads * rng.choice([1, 2, 4, 5]), "kv_heads": kv_heads, "dim": dim,
                     "vdim": dim if rng.random() < 0.4 else rng.choice([8, 16, 40, 64, 130])}
            if rng.random() < 0.7:
                mixer["rot"] = {"dims": rng.choice([d for d in (2, 4, 8, 16, dim // 2, dim) if d <= dim and d % 2 == 0]),
                                "base": rng.choice([100.0, 10000.0, 500000.0])}
            owners.append(index)
        mixer["scale"] = round(rng.uniform(0.05, 0.5), 3)
        mixer["diff"] = rng.choice([0.0, 0.1, 0.3, 0.8])
        if rng.random() < 0.7:
            mixer["mask"] = {"size": rng.choice([1, 2, 7, 33, 64, 65, 100, 190])}
        layers.append({"type": "attention", "mixer": mixer, "mlp": draw_feed_forward(rng)})
    return {"architecture": "Vunepel", "vocab": rng.randint(30, 300), "width": width,
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "layers": layers}


@pytest.mark.parametrize("dtype", ("fp32", "bf16"))
@pytest.mark.parametrize("seed", range(12))
def test_a_model_drawn_at_random(seed, dtype):
    raw = draw(seed)
    config = config_from_dict(raw)
    with tempfile.TemporaryDirectory() as holder:
        folder = write_random_model(holder, config, seed=seed, dtype=STORE[dtype])
        checkpoint = Checkpoint(folder)
        tensors = {n: checkpoint.read(n) for n in checkpoint.names()}
        for n in list(tensors):                    # sharper attention than the draw gives
            if n.endswith((".mix.q.norm", ".mix.k.norm")):
                tensors[n] = (tensors[n].float() * 2.0).to(tensors[n].dtype)
        write_safetensors(Path(folder) / "model.safetensors", tensors)
        weights = {n: t.float() for n, t in tensors.items()}
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=2048, max_step_tokens=random.Random(seed).choice([96, 512, 4096]))
    generator = torch.Generator().manual_seed(seed)
    lengths = (200, 1, 70)
    requests = [torch.randint(0, config.vocab_size, (n + 8,), generator=generator).tolist() for n in lengths]
    wants = [plain.forward(raw, weights, r, torch.float64).float() for r in requests]
    what = f"seed {seed}: {raw}"
    # whole, then the same request with its last 40 tokens one by one, then in portions of 19
    slot = engine.new_sequence()
    close(engine.step([StepEntry(slot, requests[0], list(range(len(requests[0]))))]), wants[0], dtype, "whole, " + what, model_rows=True)
    engine.release(slot)
    slot = engine.new_sequence()
    head = len(requests[0]) - 40
    rows = [engine.step([StepEntry(slot, requests[0][:head], [head - 1])])]
    rows += [engine.step([StepEntry(slot, [t], [0])]) for t in requests[0][head:]]
    engine.release(slot)
    close(torch.cat(rows), wants[0][head - 1:], dtype, "token by token, " + what, model_rows=True)
    slot = engine.new_sequence()
    rows = []
    for begin in range(0, len(requests[0]), 19):
        piece = requests[0][begin:begin + 19]
        rows.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]))
    engine.release(slot)
    close(torch.cat(rows), wants[0], dtype, "in portions, " + what, model_rows=True)
    # an unequal batch, then eight tokens each
    slots = [engine.new_sequence() for _ in requests]
    rows = [[] for _ in requests]
    out = engine.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, requests, lengths)])
    for i in range(len(requests)):
        rows[i].append(out[i:i + 1])
    for t in range(8):
        out = engine.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
        for i in range(len(requests)):
            rows[i].append(out[i:i + 1])
    for i, n in enumerate(lengths):
        close(torch.cat(rows[i]), wants[i][n - 1:], dtype, f"batch row {i}, " + what, model_rows=True)
    for s in slots:
        engine.release(s)
    engine.cache.book.check()
    engine.check_kernels()
