"""A plain, slow statement of the Vunepel design, one function per mechanism, in whatever float type it is given.

It shares nothing with the library: tensors come in a dict by checkpoint name, the configuration as the dict that
config.json holds.  Everything runs token-parallel where the design allows it and token by token where it does not
(the delta rule), on whole sequences; there is no cache.

Notation: x [T, W] residual stream of one sequence, h = norm(x); W_* weights [out, in]; p positions 0..T-1.
"""
from __future__ import annotations

import math

import torch


def dynamic_tanh(x, weight, bias, alpha):
    """y = tanh(alpha x) * w + b; no statistics of x are taken."""
    return torch.tanh(alpha * x) * weight + bias


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def clamped_gate(g, u, limit):
    """The feed-forward's activation: g capped from above, u from both sides; g sigmoid(1.702 g) (u + 1)."""
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, min=-limit, max=limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def gated_ff(h, w_gate, w_up, w_down, limit):
    return clamped_gate(h @ w_gate.T, h @ w_up.T, limit) @ w_down.T


def routed_ff(h, tensors, prefix, mlp):
    """Sigmoid router, the ``top`` largest scores, their scores over their sum times router.scale; a shared expert
    behind a sigmoid gate of one number per token."""
    router = mlp["router"]
    scores = torch.sigmoid(h @ tensors[f"{prefix}.router"].to(h.dtype).T)
    top = torch.topk(scores, int(router["top"]), dim=-1)
    weights = top.values / (top.values.sum(dim=-1, keepdim=True) + 1e-20) * float(router["scale"])
    out = torch.zeros_like(h)
    limit = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        for j in range(top.indices.shape[1]):
            e = int(top.indices[t, j])
            y = gated_ff(h[t:t + 1], tensors[f"{prefix}.e{e}.gate"].to(h.dtype), tensors[f"{prefix}.e{e}.up"].to(h.dtype),
                         tensors[f"{prefix}.e{e}.down"].to(h.dtype), limit)
            out[t] += weights[t, j] * y[0]
    if mlp.get("shared") is not None:
        y = gated_ff(h, tensors[f"{prefix}.shared.gate"].to(h.dtype), tensors[f"{prefix}.shared.up"].to(h.dtype),
                     tensors[f"{prefix}.shared.down"].to(h.dtype), float(mlp["shared"]["limit"]))
        out = out + torch.sigmoid(h @ tensors[f"{prefix}.shared.sg"].to(h.dtype).T) * y
    return out


def feed_forward(h, tensors, prefix, mlp):
    if mlp is None:
        return torch.zeros_like(h)
    if mlp["kind"] == "dense":
        return gated_ff(h, tensors[f"{prefix}.gate"].to(h.dtype), tensors[f"{prefix}.up"].to(h.dtype),
                        tensors[f"{prefix}.down"].to(h.dtype), float(mlp["limit"]))
    return routed_ff(h, tensors, prefix, mlp)


def short_conv(x, taps):
    """Causal convolution per channel: y[t, c] = sum_d taps[c, K - 1 - d] x[t - d, c], zeros before the start."""
    count = taps.shape[1]
    out = torch.zeros_like(x)
    for d in range(min(count, x.shape[0])):
        out[d:] += x[:x.shape[0] - d] * taps[:, count - 1 - d]
    return out


def softplus(x):
    return torch.clamp(x, min=0) + torch.log1p(torch.exp(-x.abs()))


def channel_delta(h, tensors, prefix, mixer, eps):
    """Gated delta rule with one decay per head and key channel; returns the mixer's output [T, W]."""
    heads, kv_heads, dim, vdim = (int(mixer[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
    group = heads // kv_heads
    get = lambda name: tensors[f"{prefix}.{name}"].to(h.dtype)
    tokens = h.shape[0]
    silu = torch.nn.functional.silu
    def conv(name, x):                       # a model whose convolutions have one tap may leave the tensors out
        taps = tensors.get(f"{prefix}.{name}.conv")
        return short_conv(x, taps.to(h.dtype)) if taps is not None else x

    q = silu(conv("q", h @ get("q").T)).view(tokens, kv_heads, dim)
    k = silu(conv("k", h @ get("k").T)).view(tokens, kv_heads, dim)
    v = silu(conv("v", h @ get("v").T)).view(tokens, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ get("b").T)                                            # [T, heads]
    rate = torch.exp(get("A_log")).view(1, heads, 1)
    decay = torch.exp(-rate * softplus((h @ get("a1").T) @ get("a2").T + get("dt_bias")).view(tokens, heads, dim))
    state = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = torch.zeros(tokens, heads, vdim, dtype=h.dtype)
    for t in range(tokens):
        for head in range(heads):
            s = state[head] * decay[t, head][:, None]
            kt, qt = k[t, head // group], q[t, head // group]
            u = beta[t, head] * (v[t, head] - s.T @ kt)
            s = s + kt[:, None] * u[None, :]
            state[head] = s
            out[t, head] = s.T @ qt
    out = rms_unit(out, eps) * get("norm")
    out = out * torch.sigmoid((h @ get("g1").T) @ get("g2").T).view(tokens, heads, vdim)
    return out.reshape(tokens, heads * vdim) @ get("o").T


def rotate(x, positions, dims, base):
    """Rotary positions on the first ``dims`` of the last axis, element i paired with i + dims / 2."""
    half = dims // 2
    freq = base ** (-2.0 * torch.arange(half, dtype=x.dtype) / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]                          # [T, half]
    cos, sin = torch.cos(angle), torch.sin(angle)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = cos.view(shape), sin.view(shape)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., dims:]), dim=-1)


def attention_keys_values(h, tensors, prefix, mixer, eps):
    """What a layer with projections of its own caches: keys [T, G, 2, dim] after norm and rotation, values [T, G, vdim]."""
    kv_heads, dim, vdim = (int(mixer[k]) for k in ("kv_heads", "dim", "vdim"))
    tokens = h.shape[0]
    k = (h @ tensors[f"{prefix}.k"].to(h.dtype).T).view(tokens, kv_heads, 2, dim)
    k = rms_unit(k, eps) * tensors[f"{prefix}.k.norm"].to(h.dtype)
    rot = mixer.get("rot")
    if rot:
        k = rotate(k, torch.arange(tokens), int(rot["dims"]), float(rot["base"]))
    v = (h @ tensors[f"{prefix}.v"].to(h.dtype).T).view(tokens, kv_heads, vdim)
    return k, v


def differential_attention(h, tensors, prefix, mixer, eps, keys_values):
    """Two softmax maps per head over the same values, o = a1 - lambda a2, unit root mean square, (1 - diff)."""
    heads, kv_heads, dim, vdim = (int(mixer[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
    group = heads // kv_heads
    tokens = h.shape[0]
    get = lambda name: tensors[f"{prefix}.{name}"].to(h.dtype)
    q = (h @ get("q").T).view(tokens, heads, 2, dim)
    q = rms_unit(q, eps) * get("q.norm")
    rot = mixer.get("rot")
    if rot:
        q = rotate(q, torch.arange(tokens), int(rot["dims"]), float(rot["base"]))
    k, v = keys_values
    diff = float(mixer["diff"])
    lam = torch.exp((get("lq1") * get("lk1")).sum()) - torch.exp((get("lq2") * get("lk2")).sum()) + diff
    place = torch.arange(tokens)
    visible = place[None, :] <= place[:, None]
    mask = mixer.get("mask")
    if mask:
        size = int(mask["size"])
        visible = visible & ((place[None, :] // size) == (place[:, None] // size))
    out = torch.zeros(tokens, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        g = head // group
        maps = []
        for m in range(2):
            score = (q[:, head, m] @ k[:, g, m].T) * float(mixer["scale"])
            score = score.masked_fill(~visible, -math.inf)
            maps.append(torch.softmax(score, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, head] = rms_unit(o, eps) * (1.0 - diff)
    return out.reshape(tokens, heads * vdim) @ get("o").T


def forward(config: dict, tensors: dict, token_ids, dtype=torch.float64, keep_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, with ``keep_layers``, the stream after every layer)."""
    eps = float(config["norm"]["eps"])
    get = lambda name: tensors[name].to(dtype)
    x = get("embed")[torch.as_tensor(token_ids, dtype=torch.long)]
    cached = {}
    streams = []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}"
        h = dynamic_tanh(x, get(f"{prefix}.norm1"), get(f"{prefix}.norm1.b"), get(f"{prefix}.norm1.alpha"))
        mixer = layer["mixer"]
        if layer["type"] == "channel_delta":
            mixed = channel_delta(h, tensors, f"{prefix}.mix", mixer, eps)
        elif layer["type"] == "attention":
            source = mixer.get("kv_from")
            if source is None:
                cached[index] = attention_keys_values(h, tensors, f"{prefix}.mix", mixer, eps)
                source = index
            mixed = differential_attention(h, tensors, f"{prefix}.mix", mixer, eps, cached[int(source)])
        else:
            raise ValueError(f"no mixer {layer['type']!r}")
        x = x + (mixed + feed_forward(h, tensors, f"{prefix}.mlp", layer.get("mlp")))
        streams.append(x)
    h = dynamic_tanh(x, get("final.norm"), get("final.norm.b"), get("final.norm.alpha"))
    logits = h @ get("head").T
    return (logits, torch.stack(streams)) if keep_layers else logits
