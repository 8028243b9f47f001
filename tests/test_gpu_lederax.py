"""The Lederax design on the GPU against the plain implementation of ``plain_lederax.py``: each mechanism's kernel
alone at sizes of its own, then whole models (the two presets and a third made here, which differ in every size and
in which options are equal or 1) whole, token by token, in portions, in unequal batches with slots used again, in
long decoding across window and ring edges, and through the generation entry point.  Where random weights would hide
a fault the inputs are made so that it shows: keys just inside and just outside a window that carry the softmax, a
far key that carries it, page tables in scrambled order with garbage in unused room."""
import functools
import math
import tempfile
from pathlib import Path

import pytest
import torch

import plain_lederax as plain
from qwen_triton_b200 import Engine, QwenB200ForCausalLM, StepEntry, config_from_dict, load_preset, write_random_model
from qwen_triton_b200.ops import kernels
from qwen_triton_b200.ops.kernels import GemmOut
from qwen_triton_b200.weights import Checkpoint, write_safetensors

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ("fp32", "bf16")
STORE = {"fp32": torch.float32, "bf16": torch.bfloat16}
TOL = {"fp32": dict(atol=2e-4, rtol=2e-4), "bf16": dict(atol=4e-2, rtol=4e-2)}
_KEEP = []

# a third configuration: one kv head per query head, norm groups of one element pair, a window longer than the
# prompts, a layer pair that shares values across different windows, top equal to the number of experts
ODD = {
    "architecture": "Lederax", "vocab": 61, "width": 72, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-4, "groups": 36},
    "layers": [
        {"type": "attention", "mlp": {"kind": "moe", "router": {"experts": 2, "top": 2}, "expert": {"ff": 20}},
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 12, "scale": 0.3, "mask": {"size": 4000}, "v_mix": True}},
        {"type": "attention", "mlp": {"kind": "moe", "router": {"experts": 6, "top": 1}, "expert": {"ff": 33}},
         "mixer": {"heads": 9, "kv_heads": 3, "dim": 8, "vdim": 12, "scale": 0.5, "mask": {"size": 3}, "v_mix": True}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 40, "vdim": 200, "scale": 0.1, "v_mix": False}},
    ],
}


def close(actual, expected, dtype, what=""):
    actual, expected = actual.float().cpu(), expected.float().cpu()
    assert actual.shape == expected.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    tol = TOL[dtype]
    bad = (actual - expected).abs() > tol["atol"] + tol["rtol"] * expected.abs()
    if bad.any():
        rows = bad.reshape(bad.shape[0], -1).any(dim=1).nonzero().flatten().tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} values differ, first wrong row {rows[0]} of {bad.shape[0]} "
                             f"(wrong rows {rows[:12]}), max abs error {float((actual - expected).abs().max()):.3e}")


# ----------------------------------------------------------------------------- models and their oracle
def config_of(name):
    return config_from_dict(ODD) if name == "odd" else load_preset(name)


@functools.lru_cache(maxsize=None)
def model(name: str, dtype: str, peaky: bool = False):
    """(folder, raw config, float weights for the oracle).  ``peaky``: q and k weights four times as large and the
    distance penalty's r1 a fifth, so that few keys, far ones among them, carry each softmax."""
    config = config_of(name)
    holder = tempfile.TemporaryDirectory(prefix=f"qt_{name}_{dtype}_")
    _KEEP.append(holder)
    folder = write_random_model(holder.name, config, seed=11 + len(name), dtype=STORE[dtype])
    if peaky:
        checkpoint = Checkpoint(folder)
        tensors = {n: checkpoint.read(n) for n in checkpoint.names()}
        for n in list(tensors):
            if n.endswith((".mix.q", ".mix.k")):
                tensors[n] = (tensors[n].float() * 4.0).to(tensors[n].dtype)
            if n.endswith(".mix.r1"):
                tensors[n] = (tensors[n].float() * 0.2).to(tensors[n].dtype)
        write_safetensors(Path(folder) / "model.safetensors", tensors)
    checkpoint = Checkpoint(folder)
    weights = {n: (checkpoint.read(n).float() if checkpoint.read(n).dtype.is_floating_point else checkpoint.read(n))
               for n in checkpoint.names()}
    return folder, config.to_hf_dict(), weights


@functools.lru_cache(maxsize=None)
def oracle(name: str, dtype: str, peaky: bool, tokens: tuple) -> torch.Tensor:
    _, raw, weights = model(name, dtype, peaky)
    return plain.forward(raw, weights, list(tokens))


def tokens_of(name: str, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(5000 + seed)
    return torch.randint(0, config_of(name).vocab_size, (length,), generator=generator).tolist()


def engine_of(name, dtype, peaky=False, **kwargs) -> Engine:
    kwargs.setdefault("max_tokens", 4096)
    return Engine.from_pretrained(model(name, dtype, peaky)[0], dtype=dtype, **kwargs)


MODELS = ("lederax-tiny-a", "lederax-tiny-b", "odd")
CASES = [(m, d) for m in MODELS for d in DTYPES]


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("width, groups", [(96, 3), (130, 5), (2048, 2), (72, 36), (64, 1), (7, 7)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_in_groups(width, groups, out_dtype):
    torch.manual_seed(width)
    rows = 9
    stream = torch.randn(rows, width, device=DEV) * 3
    delta = torch.randn(3, rows, width, device=DEV)
    weight = torch.rand(width, device=DEV) + 0.5
    want_stream = stream + delta.sum(0)
    want = plain.group_rms_norm(want_stream.cpu(), weight.cpu(), groups, 1e-5)
    got_stream = stream.clone()
    out = torch.empty(rows, width, device=DEV, dtype=out_dtype)
    kernels.add_rmsnorm(got_stream, GemmOut(delta), weight, 1e-5, out, None, groups)
    assert torch.allclose(got_stream.cpu(), want_stream.cpu(), atol=1e-6)
    close(out, want, "fp32" if out_dtype == torch.float32 else "bf16", "all rows")
    # listed rows only: the stream stays as it is
    picked = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    again = stream.clone()
    out = torch.empty(3, width, device=DEV, dtype=out_dtype)
    kernels.add_rmsnorm(again, GemmOut(delta), weight, 1e-5, out, picked, groups)
    assert torch.equal(again, stream)
    close(out, want[picked.cpu().long()], "fp32" if out_dtype == torch.float32 else "bf16", "listed rows")


def test_embedding_is_scaled_in_float():
    table = torch.randn(11, 20, device=DEV).to(torch.bfloat16)
    ids = torch.tensor([3, 10, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 20, device=DEV)
    kernels.embedding(out, table, ids, 12.5)
    assert torch.equal(out.cpu(), plain.embed(ids.cpu().long(), table.float().cpu(), 12.5))


def paged(values: torch.Tensor, page_tokens: int, order: list[int], dtype):
    """Lay ``values`` [S, heads, d] of one sequence into pages in the given page order; unused room holds large
    numbers, so that a key read from there shows.  Returns the cache [pages, heads, page_tokens, d]."""
    length, heads, d = values.shape
    cache = torch.full((max(order) + 1, heads, page_tokens, d), 77.0, dtype=dtype, device=DEV)
    for pos in range(length):
        cache[order[pos // page_tokens], :, pos % page_tokens] = values[pos].to(dtype)
    return cache


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, d, dv, window", [(4, 2, 16, 32, 21), (3, 3, 40, 8, None), (8, 1, 64, 64, 64), (2, 1, 24, 130, 1),
                                                             (6, 2, 32, 32, 50), (2, 1, 128, 128, None), (34, 2, 48, 48, 129)])
def test_attention_with_distance_penalty_and_window_edges(dtype, heads, kv_heads, d, dv, window):
    """Prompt portions and one-token steps over a scrambled paged cache.  The keys just inside and just outside the
    window of the last queries, and one far key, are made to match their queries (score far above the rest): a window
    off by one, a dropped far key or a penalty with the wrong head's factors changes the result by much."""
    torch.manual_seed(heads * 100 + d)
    store = STORE[dtype]
    length, page = 200, 64
    q_all = torch.randn(length, heads, d)
    k = torch.randn(length, kv_heads, d)
    v = torch.randn(length, kv_heads, dv)
    per = heads // kv_heads
    for query in (length - 1, length - 2, 150, 70):
        edges = [query - 100] if window is None else [query - window + 1, query - window]
        for edge in edges + [3]:
            if 0 <= edge <= query:
                k[edge] = q_all[query].view(kv_heads, per, d)[:, 0] * 3.0
    q_all, k, v = (t.to(store).float() for t in (q_all, k, v))
    r1 = torch.rand(heads) * 2
    r2 = torch.rand(heads) * 0.5 + 0.01
    scale = 0.4

    def expected(rows):
        scores = torch.einsum("ihd,jhd->hij", q_all, k.repeat_interleave(per, 1)) * scale - plain.distance_penalty(r1, r2, length)
        scores = scores.masked_fill(~plain.visible(length, window), -math.inf)
        return torch.einsum("hij,jhd->ihd", torch.softmax(scores, -1), v.repeat_interleave(per, 1))[rows]

    order = [5, 2, 7, 0]
    kc, vc = paged(k, page, order, store), paged(v, page, order, store)
    table = torch.tensor([order], dtype=torch.int32, device=DEV)
    penalty = (r1.to(DEV), r2.to(DEV))
    # a portion: the last 130 tokens as queries over the whole cache
    first = length - 130
    q = q_all[first:].to(store).to(DEV).contiguous()
    out = torch.empty(130, heads, dv, dtype=store, device=DEV)
    kernels.attention_prefill(q, kc, vc, out, table, torch.tensor([0, 130], dtype=torch.int32, device=DEV),
                              torch.tensor([first], dtype=torch.int32, device=DEV), 130, kv_heads, page, 0, window, scale, penalty=penalty)
    close(out, expected(slice(first, length)), dtype, "portion")
    # one token, keys cut into 1 and 3 ranges
    for splits in (1, 3):
        q = q_all[length - 1:].to(store).to(DEV).contiguous()
        out = torch.empty(1, heads, dv, dtype=store, device=DEV)
        acc = torch.empty(heads * splits * dv, device=DEV)
        ml = torch.empty(heads * splits * 2, device=DEV)
        kernels.attention_decode(q, kc, vc, out, table, torch.tensor([length], dtype=torch.int32, device=DEV), kv_heads, page, 0,
                                 window, scale, splits, acc, ml, penalty=penalty)
        close(out, expected(slice(length - 1, length)), dtype, f"one token, {splits} ranges")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, dv", [(12, 20), (10, 6), (128, 256), (260, 8)])
def test_values_are_normed_blended_and_cached(dtype, d, dv):
    """The kernel behind the projection: bias on split sums, q out, k and v into a ring of pages; values divided by
    their root mean square, kept by a source layer and blended by a later one."""
    torch.manual_seed(3)
    store = STORE[dtype]
    tokens, nq, nkv, page, ring = 37, 4, 2, 64, 128
    width = (nq + nkv) * d + nkv * dv
    sums = torch.randn(2, tokens, width, device=DEV)
    bias = torch.randn(width, device=DEV)
    total = (sums.sum(0) + bias).cpu()
    pos = torch.arange(100, 100 + tokens, dtype=torch.int32, device=DEV)          # crosses the ring's end at 128
    seq = torch.zeros(tokens, dtype=torch.int32, device=DEV)
    table = torch.tensor([[4, 1]], dtype=torch.int32, device=DEV)
    eps = 1e-3
    want_q = total[:, :nq * d].view(tokens, nq, d)
    want_k = total[:, nq * d:(nq + nkv) * d].view(tokens, nkv, d)
    want_v = plain.unit_rms(total[:, (nq + nkv) * d:].view(tokens, nkv, dv), eps)

    def run(blend_from, weight, keep_to):
        q = torch.empty(tokens, nq, d, dtype=store, device=DEV)
        kc = torch.zeros(5, nkv, page, d, dtype=store, device=DEV)
        vc = torch.zeros(5, nkv, page, dv, dtype=store, device=DEV)
        kernels.qkv_treat_write(GemmOut(sums), bias, q, kc, vc, seq, pos, table, nq, nkv, d, dv, page, ring, v_norm_eps=eps,
                                blend_from=blend_from, blend_weight=weight, keep_to=keep_to)
        where = [(int(table[0, (p % ring) // page]), (p % ring) % page) for p in pos.tolist()]
        return q, torch.stack([kc[pg, :, at] for pg, at in where]), torch.stack([vc[pg, :, at] for pg, at in where])

    kept = torch.empty(tokens, nkv, dv, device=DEV)
    q, k, v = run(None, None, kept)
    close(q, want_q, dtype, "q"); close(k, want_k, dtype, "k"); close(v, want_v, dtype, "v of the source layer")
    close(kept, want_v, "fp32", "kept values are float")
    other = torch.randn(tokens, nkv, dv, device=DEV)
    lam = torch.tensor([0.3], device=DEV)
    _, _, v = run(other, lam, None)
    close(v, 0.7 * want_v + 0.3 * other.cpu(), dtype, "blended v")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, experts, top, width, ff", [(5, 3, 1, 40, 24), (33, 4, 4, 64, 72), (300, 12, 2, 128, 96), (700, 5, 3, 72, 200),
                                                               (1500, 6, 2, 512, 320), (2048, 4, 2, 256, 4360)])
def test_experts_chosen_by_the_token_table(dtype, tokens, experts, top, width, ff):
    torch.manual_seed(tokens)
    store = STORE[dtype]
    vocab = 50
    up = (torch.randn(experts, ff, width) * width ** -0.5).to(store)          # results of the order of 1
    down = (torch.randn(experts, width, ff) * 2.0 * ff ** -0.5).to(store)
    table = torch.stack([torch.randperm(experts)[:top] for _ in range(vocab)]).to(torch.int32)
    ids = torch.randint(0, vocab, (tokens,), dtype=torch.int32)
    x = torch.randn(tokens, width).to(store)
    weights = {"m.table": table}
    for e in range(experts):
        weights[f"m.e{e}.up"], weights[f"m.e{e}.down"] = up[e].float(), down[e].float()
    want = plain.routed_experts(x.float(), ids.long(), weights, "m", {"router": {"top": top}})
    from qwen_triton_b200.parts.base import Runtime, Workspace
    from qwen_triton_b200.parts.feed_forward import TableExperts
    runtime = Runtime(device=torch.device(DEV), dtype=store, max_step_tokens=2048, max_positions=64, workspace=Workspace(torch.device(DEV)))
    part = TableExperts({"hidden_size": width, "expert_size": ff, "experts": experts, "top": top, "vocab_size": vocab,
                         "activation": "gelu", "expert": "e{}", "weight_suffix": ""}, "m", runtime)
    runtime.workspace.allocate()
    part.load(lambda name: weights[name])

    class Ctx:
        token_ids = ids.to(DEV)
    close(part.forward(x.to(DEV), Ctx).value(), want, dtype, "experts")
    kernels.check_status(DEV)


# ----------------------------------------------------------------------------- whole models
def run_whole(engine, tokens):
    slot = engine.new_sequence()
    try:
        return engine.step([StepEntry(slot, list(tokens), list(range(len(tokens))))])
    finally:
        engine.release(slot)


@pytest.mark.parametrize("name, dtype", CASES)
def test_each_request_alone_and_whole(name, dtype):
    engine = engine_of(name, dtype)
    for i, length in enumerate((1, 2, 33, 170, 400)):
        tokens = tokens_of(name, length, i)
        close(run_whole(engine, tokens), oracle(name, dtype, False, tuple(tokens)), dtype, f"{length} tokens")
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
def test_prompt_then_token_by_token_across_window_and_page_edges(name, dtype):
    """Peaky weights; decoding starts before and runs past every edge there is: the windows (24, 70, 130, 300, 3),
    the pages (64) and, with chunks of 16 tokens, the rings of the windowed groups."""
    engine = engine_of(name, dtype, peaky=True, chunk_tokens=16)
    tokens = tokens_of(name, 340, 77)
    want = oracle(name, dtype, True, tuple(tokens))
    for head in (20, 290):
        slot = engine.new_sequence()
        rows = [engine.step([StepEntry(slot, tokens[:head], [0, head - 1])])]
        last = min(len(tokens), head + 60)
        for at in range(head, last):
            rows.append(engine.step([StepEntry(slot, [tokens[at]], [0])]))
        engine.release(slot)
        close(torch.cat(rows), want[[0] + list(range(head - 1, last))], dtype, f"prompt of {head}, then one by one")
    assert engine.graph_replays > 0
    engine.check_kernels()


@pytest.mark.parametrize("name, dtype", CASES)
@pytest.mark.parametrize("portion", [2, 3, 17, 64, 100])
def test_portions_of_a_prompt(name, dtype, portion):
    engine = engine_of(name, dtype, peaky=True, chunk_tokens=32)
    tokens = tokens_of(name, 230, 5)
    want = oracle(name, dtype, True, tuple(tokens))
    slot = engine.new_sequence()
    rows = []
    for begin in range(0, len(tokens), portion):
        piece = tokens[begin:begin + portion]
        rows.append(engine.step([StepEntry(slot, piece, list(range(len(piece))))]))
    engine.release(slot)
    close(torch.cat(rows), want, dtype, f"portions of {portion}")


@pytest.mark.parametrize("name, dtype", CASES)
def test_unequal_batches_with_slots_and_pages_used_again(name, dtype):
    """Batches of unequal requests, one after another on one engine whose cache holds little more than a batch, each
    request decoded on for a few tokens; the shorter ones end earlier.  Every row equals the request run alone."""
    engine = engine_of(name, dtype, peaky=True, max_tokens=1024)
    for batch in range(3):
        lengths = [(7, 150, 1, 64, 65), (300, 2, 129), (31, 31, 200, 3)][batch]
        requests = [tokens_of(name, n + 6, 100 * batch + i) for i, n in enumerate(lengths)]
        slots = [engine.new_sequence() for _ in requests]
        out = engine.step([StepEntry(s, r[:n], [0, n - 1] if n > 1 else [0]) for s, r, n in zip(slots, requests, lengths)])
        at = 0
        for r, n in zip(requests, lengths):
            want = oracle(name, dtype, True, tuple(r))
            picked = [0, n - 1] if n > 1 else [0]
            close(out[at:at + len(picked)], want[picked], dtype, f"batch {batch}: prompt of {n}")
            at += len(picked)
        live = list(range(len(requests)))
        for step in range(6):
            if step == 3:                         # the first request ends early; the others go on
                engine.release(slots[live.pop(0)])
            out = engine.step([StepEntry(slots[i], [requests[i][lengths[i] + step]], [0]) for i in live])
            for row, i in enumerate(live):
                want = oracle(name, dtype, True, tuple(requests[i]))
                close(out[row:row + 1], want[lengths[i] + step:lengths[i] + step + 1], dtype, f"batch {batch}: request {i}, step {step}")
        for i in live:
            engine.release(slots[i])
        engine.cache.book.check()
    engine.check_kernels()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_of_several_rows(dtype):
    name = "lederax-tiny-a"
    engine = engine_of(name, dtype, peaky=True, chunk_tokens=16)
    lengths = (1, 30, 90)
    steps = 150
    requests = [tokens_of(name, n + steps, 900 + i) for i, n in enumerate(lengths)]
    slots = [engine.new_sequence() for _ in requests]
    engine.step([StepEntry(s, r[:n], []) for s, r, n in zip(slots, requests, lengths)])
    rows = [[] for _ in requests]
    for t in range(steps):
        out = engine.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, requests, lengths)])
        for i in range(len(requests)):
            rows[i].append(out[i:i + 1])
    for i, (r, n) in enumerate(zip(requests, lengths)):
        close(torch.cat(rows[i]), oracle(name, dtype, True, tuple(r))[n:], dtype, f"row {i}")
    engine.check_kernels()


@pytest.mark.parametrize("name", MODELS)
def test_greedy_generation_through_the_entry_point(name):
    folder, raw, weights = model(name, "fp32")
    lm = QwenB200ForCausalLM.from_pretrained_hf(folder, dtype="fp32", max_tokens=2048)
    prompts = [tokens_of(name, n, 40 + n) for n in (5, 1, 47)]
    results = lm.generate(prompts, max_new_tokens=12, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert result.tokens == plain.greedy_generate(raw, weights, prompt, 12)
    # the same in bfloat16 runs and stays within the vocabulary
    lm16 = QwenB200ForCausalLM.from_pretrained_hf(model(name, "bf16")[0], dtype="bf16", max_tokens=2048)
    for result in lm16.generate(prompts, max_new_tokens=12, ignore_eos=True, temperature=0.7, seed=3):
        assert len(result.tokens) == 12 and all(0 <= t < config_of(name).vocab_size for t in result.tokens)


def test_random_weights_on_the_device_equal_the_written_folder():
    config = load_preset("lederax-tiny-b")
    tokens = tokens_of("lederax-tiny-b", 50, 1)
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, config, seed=9, dtype=torch.float32)
        a = run_whole(Engine.from_pretrained(folder, dtype="fp32", max_tokens=256), tokens)
    b = run_whole(Engine.from_config(config, seed=9, dtype="fp32", max_tokens=256), tokens)
    assert torch.equal(a, b)


# ----------------------------------------------------------------------------- as a user runs it
def test_command_line_with_a_preset_and_random_weights():
    """``scripts.smoke`` as a child process: weights drawn on the device from --seed, prompts of random ids; the same
    draw on the host gives the oracle its model."""
    import ast
    import re
    import subprocess
    import sys
    from qwen_triton_b200.engine.model import expected_tensors
    from qwen_triton_b200.weights import random_tensor
    name, seed, lengths = "lederax-tiny-b", 4, (9, 30)
    config = load_preset(name)
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, "-m", "qwen_triton_b200.scripts.smoke", "--preset", name, "--random-weights", "--seed", str(seed),
                           "--dtype", "fp32", "--random-prompts", ",".join(map(str, lengths)), "--max-new-tokens", "5", "--ignore-eos",
                           "--max-tokens", "512"], cwd=root, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = [ast.literal_eval(m.group(1)) for m in re.finditer(r"generated=(\[.*?\]) finish=length", proc.stdout)]
    weights = {n: random_tensor(n, spec, seed, torch.float32 if spec.role != "table" else torch.int32)
               for n, spec in expected_tensors(config.model_spec()).items() if not spec.optional}
    generator = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, config.vocab_size, (n,), generator=generator).tolist() for n in lengths]
    assert got == [plain.greedy_generate(config.to_hf_dict(), weights, p, 5) for p in prompts]


@pytest.mark.parametrize("dtype, name", [("float32", "fp32"), ("bfloat16", "bf16")])
def test_trace_replay_of_a_folder(tmp_path, dtype, name):
    """``bin/trace_run`` as a child process on a model folder of the design: a batch of unequal prompts, then their
    next tokens one by one, one request ending early; under a --max-tokens of exactly what is live at most."""
    import json
    import subprocess
    import sys
    import numpy as np
    model_name = "lederax-tiny-a"
    folder = model(model_name, name)[0]
    lengths = {"a": 70, "b": 3, "c": 129}
    requests = {key: tokens_of(model_name, n + 4, 60 + n) for key, n in lengths.items()}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": r[:lengths[k]], "want": [lengths[k] - 1]} for k, r in requests.items()], "end": []}]
    for t in range(4):
        live = [k for k in requests if not (k == "b" and t >= 2)]
        steps.append({"step": t + 1, "entries": [{"id": k, "tokens": [requests[k][lengths[k] + t]], "want": [0] if t != 1 else []} for k in live],
                      "end": (["b"] if t == 1 else []) + (live if t == 3 else [])})
    most = 128 + 64 + 192                      # each request rounded up to whole pages of 64
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(tmp_path),
                           "--max-tokens", str(most)], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {i}" for i in range(5)]
    vocab = config_of(model_name).vocab_size
    for step in steps:
        wanted = [(e["id"], w) for e in step["entries"] for w in e["want"]]
        path = tmp_path / f"{step['step']}.f32"
        if not wanted:
            assert not path.exists()
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab).copy())
        for row, (key, _) in enumerate(wanted):
            at = lengths[key] - 1 + step["step"]
            close(got[row:row + 1], oracle(model_name, name, False, tuple(requests[key]))[at:at + 1], name, f"step {step['step']} request {key}")


def test_trace_replay_of_many_short_requests_at_once(tmp_path):
    """Forty requests of one to five tokens live together: 120 tokens in all, which --max-tokens states exactly, though
    every request holds a page of its own."""
    import json
    import subprocess
    import sys
    import numpy as np
    model_name = "lederax-tiny-b"
    folder = model(model_name, "fp32")[0]
    requests = {f"q{i}": tokens_of(model_name, 1 + i % 5, 300 + i) for i in range(40)}
    steps = [{"step": 0, "entries": [{"id": k, "tokens": r, "want": [len(r) - 1]} for k, r in requests.items()], "end": list(requests)}]
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path),
                           "--max-tokens", str(sum(len(r) for r in requests.values()))], input=json.dumps(steps[0]) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = torch.from_numpy(np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(40, config_of(model_name).vocab_size).copy())
    for row, r in enumerate(requests.values()):
        close(got[row:row + 1], oracle(model_name, "fp32", False, tuple(r))[-1:], "fp32", f"request {row}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompt_in_passes_and_decoding_across_position_1024(dtype):
    """A prompt of 1,300 tokens run in passes of 512 tokens (and chunks of 256 for the windowed groups), then a second
    sequence decoded from 1,000 to 1,060 tokens: the one-token step's page-table width and context bucket change at
    1,024, and the full-attention layer's keys are cut into more ranges."""
    name = "lederax-tiny-b"
    engine = engine_of(name, dtype, peaky=True, max_step_tokens=512)
    tokens = tokens_of(name, 1300, 21)
    want = oracle(name, dtype, True, tuple(tokens))
    picked = [0, 255, 256, 511, 512, 1023, 1024, 1299]
    slot = engine.new_sequence()
    close(engine.step([StepEntry(slot, tokens, picked)]), want[picked], dtype, "a prompt in passes")
    engine.release(slot)
    slot = engine.new_sequence()
    rows = [engine.step([StepEntry(slot, tokens[:1000], [999])])]
    rows += [engine.step([StepEntry(slot, [t], [0])]) for t in tokens[1000:1060]]
    engine.release(slot)
    close(torch.cat(rows), want[999:1060], dtype, "decoding across 1,024")
    engine.check_kernels()
