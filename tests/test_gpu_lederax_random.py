"""Lederax models drawn at random from what config.json allows (sizes, head counts, layer lists, windows, groups,
experts; widths and expert sizes off 8 among them, layers without a feed-forward, value sharing that starts late or
never), each run whole, token by token and as an unequal batch in both types against the plain implementation."""
import random
import tempfile
from pathlib import Path

import pytest
import torch

import plain_lederax as plain
from qwen_triton_b200 import Engine, StepEntry, config_from_dict, write_random_model
from qwen_triton_b200.weights import Checkpoint, write_safetensors
from test_gpu_lederax import STORE, close

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([36, 40, 64, 72, 96, 100, 128, 200])
    # groups of at least four elements: a group of one is x / sqrt(x^2 + eps), a sign, and a model of signs carries
    # rounding from one type to the next as whole units (the kernel test covers such groups on given numbers)
    groups = rng.choice([g for g in (1, 2, 3, 4, 5, 8, 9, 10, 25) if width % g == 0 and width // g >= 4])
    shared_kv, shared_vdim = rng.choice([1, 2, 3]), rng.choice([8, 16, 24, 32, 64, 128])
    layers = []
    for _ in range(rng.randint(1, 5)):
        v_mix = rng.random() < 0.6
        kv_heads = shared_kv if v_mix else rng.choice([1, 2, 3])
        dim = rng.choice([8, 16, 24, 32, 64, 128])
        vdim = shared_vdim if v_mix else (dim if rng.random() < 0.5 else rng.choice([8, 16, 40, 64]))
        mixer = {"heads": kv_heads * rng.choice([1, 2, 4, 5]), "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                 "scale": round(rng.uniform(0.05, 0.5), 3), "v_mix": v_mix}
        if rng.random() < 0.7:
            mixer["mask"] = {"size": rng.choice([1, 2, 7, 33, 64, 65, 100, 190])}
        mlp = None
        if rng.random() < 0.8:
            experts = rng.randint(1, 9)
            mlp = {"kind": "moe", "router": {"experts": experts, "top": rng.randint(1, min(experts, 4))},
                   "expert": {"ff": rng.choice([8, 20, 48, 96, 136])}}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Lederax", "vocab": rng.randint(30, 300), "width": width,
            "embedding": {"scale": round(rng.uniform(0.5, 8.0), 2)},
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3]), "groups": groups}, "layers": layers}


@pytest.mark.parametrize("dtype", ("fp32", "bf16"))
@pytest.mark.parametrize("seed", range(10))
def test_a_model_drawn_at_random(seed, dtype):
    raw = draw(seed)
    config = config_from_dict(raw)
    with tempfile.TemporaryDirectory() as holder:
        folder = write_random_model(holder, config, seed=seed, dtype=STORE[dtype])
        checkpoint = Checkpoint(folder)
        tensors = {n: checkpoint.read(n) for n in checkpoint.names()}
        for n in list(tensors):                    # sharper attention than the draw gives: q and k twice as large
            if n.endswith((".mix.q", ".mix.k")):
                tensors[n] = (tensors[n].float() * 2.0).to(tensors[n].dtype)
        write_safetensors(Path(folder) / "model.safetensors", tensors)
        weights = {n: (t.float() if t.dtype.is_floating_point else t) for n, t in tensors.items()}
        engine = Engine.from_pretrained(folder, dtype=dtype, max_tokens=2048, chunk_tokens=random.Random(seed).choice([16, 64, 256]))
    generator = torch.Generator().manual_seed(seed)
    lengths = (230, 1, 70)
    requests = [torch.randint(0, config.vocab_size, (n + 8,), generator=generator).tolist() for n in lengths]
    wants = [plain.forward(raw, weights, r) for r in requests]
    what = f"seed {seed}: {raw}"
    # whole, then the same request with its last 40 tokens one by one
    slot = engine.new_sequence()
    close(engine.step([StepEntry(slot, requests[0], list(range(len(requests[0]))))]), wants[0], dtype, "whole, " + what)
    engine.release(slot)
    slot = engine.new_sequence()
    head = len(requests[0]) - 40
    rows = [engine.step([StepEntry(slot, requests[0][:head], [head - 1])])]
    rows += [engine.step([StepEntry(slot, [t], [0])]) for t in requests[0][head:]]
    engine.release(slot)
    close(torch.cat(rows), wants[0][head - 1:], dtype, "token by token, " + what)
    # an unequal batch, then eight tokens each
    slots = [engine.new_sequence() for _ in requests]
    out = engine.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, requests, lengths)])
    for i, n in enumerate(lengths):
        close(out[i:i + 1], wants[i][n - 1:n], dtype, f"batch prompt {i}, " + what)
    for t in range(8):
        out = engine.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
        for i, n in enumerate(lengths):
            close(out[i:i + 1], wants[i][n + t:n + t + 1], dtype, f"batch step {t} row {i}, " + what)
    for s in slots:
        engine.release(s)
    engine.cache.book.check()
    engine.check_kernels()
