"""Plain, slow implementation of the Lederax design: the tests' oracle.

Whole sequences only, no cache, one function per mechanism, plain tensor operations in the
element type of the weights it is given (float32 or float64).  It shares no code with the
``qwen_triton_b200`` package: it reads the raw config.json mapping itself and takes weights as a
``name -> tensor`` mapping under the design's own tensor names.

The design in short.  Token embedding times a constant.  Pre-norm layers: x += mixer(norm(x)),
then, where the layer has one, x += feed_forward(norm(x)).  The norm is an RMS norm over equal
consecutive groups of the vector, then a weight over the whole.  The mixer is softmax attention with
grouped key/value heads, biased q/k/v projections, no rotation, a logarithmic distance penalty on
the scores, a sliding window, values divided by their root mean square per head and, in marked
layers after the first marked one, blended with the first marked layer's values of the same token.
The feed-forward is a set of small two-matrix experts with the exact GELU, of which a token uses the
few that a table names for its token id, equally weighted.  Final norm, output projection.
"""
from __future__ import annotations

import math
from typing import Mapping, Sequence

import torch


def group_rms_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Split the last dim into ``groups`` equal consecutive parts, divide each by sqrt(mean(part^2) + eps),
    multiply the whole by ``weight``."""
    *lead, width = x.shape
    parts = x.reshape(*lead, groups, width // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(*lead, width) * weight


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dim, no weight."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def embed(ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    return table[ids] * scale


def distance_penalty(r1: torch.Tensor, r2: torch.Tensor, length: int) -> torch.Tensor:
    """[heads, length, length]: r1_h * ln(1 + r2_h * (i - j)) for query i and key j (only j <= i is used)."""
    i = torch.arange(length, dtype=r1.dtype)[:, None]
    j = torch.arange(length, dtype=r1.dtype)[None, :]
    distance = (i - j).clamp(min=0)
    return r1[:, None, None] * torch.log(1.0 + r2[:, None, None] * distance)


def visible(length: int, window: int | None) -> torch.Tensor:
    """[length, length] bool: key j is seen from query i iff 0 <= i - j and, with a window, i - j < window."""
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    mask = j <= i
    if window is not None:
        mask &= (i - j) < window
    return mask


def attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mixer: Mapping, eps: float,
              v_first: torch.Tensor | None, blend: bool):
    """One attention mixer on the normed rows ``h`` [S, width].  Returns (output [S, width], values [S, G, vdim]).

    ``blend``: this layer blends its values with ``v_first`` (it is a marked layer and not the first one)."""
    S = h.shape[0]
    H, G, d, dv = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    q = (h @ w[f"{prefix}.q"].T + w[f"{prefix}.q.b"]).view(S, H, d)
    k = (h @ w[f"{prefix}.k"].T + w[f"{prefix}.k.b"]).view(S, G, d)
    v = (h @ w[f"{prefix}.v"].T + w[f"{prefix}.v.b"]).view(S, G, dv)
    v = unit_rms(v, eps)
    if blend:
        lam = w[f"{prefix}.vmix"]
        v = (1.0 - lam) * v + lam * v_first
    per = H // G
    k_of = k.repeat_interleave(per, dim=1)                                   # query head h reads kv head h // per
    v_of = v.repeat_interleave(per, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k_of) * float(mixer["scale"])
    scores = scores - distance_penalty(w[f"{prefix}.r1"], w[f"{prefix}.r2"], S)
    mask = mixer.get("mask") or {}
    window = int(mask["size"]) if mask.get("size") is not None else None
    scores = scores.masked_fill(~visible(S, window), -math.inf)
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", weights, v_of).reshape(S, H * dv)
    return out @ w[f"{prefix}.o"].T, v


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def routed_experts(h: torch.Tensor, ids: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str, mlp: Mapping) -> torch.Tensor:
    """Each token runs the ``top`` experts that the table's row of its token id names; their outputs are averaged."""
    top = int(mlp["router"]["top"])
    table = w[f"{prefix}.table"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for slot in range(top):
            e = int(table[int(ids[t]), slot])
            mid = gelu_erf(w[f"{prefix}.e{e}.up"] @ h[t])
            out[t] += (w[f"{prefix}.e{e}.down"] @ mid) / top
    return out


def forward(raw: Mapping, weights: Mapping[str, torch.Tensor], tokens: Sequence[int], return_layers: bool = False):
    """Logits [S, vocab] of one whole sequence; with ``return_layers`` also the stream after every layer."""
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    eps, groups = float(raw["norm"]["eps"]), int(raw["norm"]["groups"])
    x = embed(ids, weights["embed"], float(raw["embedding"]["scale"]))
    v_first = None
    after = []
    for index, layer in enumerate(raw["layers"]):
        if layer["type"] != "attention":
            raise ValueError(f"layer {index}: the design has no mixer {layer['type']!r}")
        p = f"l{index}"
        marked = bool(layer["mixer"].get("v_mix", False))
        h = group_rms_norm(x, weights[f"{p}.norm1"], groups, eps)
        y, v = attention(h, weights, f"{p}.mix", layer["mixer"], eps, v_first, marked and v_first is not None)
        if marked and v_first is None:
            v_first = v
        x = x + y
        if layer.get("mlp") is not None:
            h = group_rms_norm(x, weights[f"{p}.norm2"], groups, eps)
            x = x + routed_experts(h, ids, weights, f"{p}.mlp", layer["mlp"])
        after.append(x)
    x = group_rms_norm(x, weights["final.norm"], groups, eps)
    logits = x @ weights["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy_generate(raw: Mapping, weights: Mapping[str, torch.Tensor], prompt: Sequence[int], new_tokens: int) -> list[int]:
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(forward(raw, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
