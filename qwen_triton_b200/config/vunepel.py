"""Typed configuration of the Vunepel design, read from config.json.

The file names its design under ``architecture`` and gives ``vocab``, ``width``, ``norm.eps`` and a list ``layers``.
An entry has ``type`` (its mixer: ``attention`` or ``channel_delta``), the mixer's sizes and constants under ``mixer``
and its feed-forward under ``mlp`` (null for none).  Layers need not be alike.

``attention``: ``heads``, ``kv_heads``, ``dim`` (of a query or key per score map), ``vdim``, ``scale``, ``diff``,
``rot.dims`` / ``rot.base`` (absent: no rotation), ``mask.size`` (absent: every earlier token is seen) and
``kv_from`` (the layer whose cached keys and values this one reads instead of projecting its own).
``channel_delta``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps).  Its two narrow projections' column
counts are no key of the file: they are the shapes of the stored tensors (``with_tensor_shapes``); a configuration that
is to draw random weights names them under ``mixer.ranks`` = {"decay": n, "gate": n}.
``mlp``: ``kind`` "dense" with ``ff`` and ``limit``, or "moe" with ``router.experts``, ``router.top``,
``router.scale``, ``expert.ff``, ``expert.limit`` and optionally ``shared.ff``, ``shared.limit``.

What the design fixes, and ``model_spec`` therefore states as parameters of the parts: one Dynamic Tanh norm per layer
whose output both the mixer and the feed-forward read, their results added to the stream together; differential
attention (two score maps per head over the same values, q/k RMS norm per head and map before a rotate-half rotation
of the first ``rot.dims`` dimensions, softmax within chunks of ``mask.size`` positions, o = a1 - lambda a2 brought to
unit root mean square, times 1 - diff); the gated delta rule with a decay per key channel; feed-forwards with the
capped gate g sigmoid(1.702 g) (u + 1); experts chosen by a sigmoid router; no biases; tensor names ``embed``,
``head``, ``final.norm`` and ``l<i>.{norm1,mix.*,mlp.*}`` without a ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Any, Mapping

from .qwen3 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MAX_POSITIONS = 1 << 20          # the design names no longest sequence; the rotation table is made for the cache's length


@dataclass(frozen=True)
class VunepelFeedForward:
    kind: str                       # "dense" or "moe"
    ff: int                         # width of the middle (of every expert for "moe")
    limit: float
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    shared_ff: int = 0              # 0: no shared expert
    shared_limit: float = 0.0


@dataclass(frozen=True)
class VunepelLayer:
    type: str                       # "attention" or "channel_delta"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    mlp: VunepelFeedForward | None
    # attention
    scale: float = 0.0
    diff: float = 0.0
    rot_dims: int = 0               # 0: no rotation
    rot_base: float = 10000.0
    chunk: int | None = None        # mask.size
    kv_from: int | None = None
    # channel_delta
    conv: int = 1
    decay_rank: int = 0             # 0: not known yet (see with_tensor_shapes)
    gate_rank: int = 0


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or mapping.get(key) is None:
        raise ConfigError(f"config.json lacks {where}.{key}" if where else f"config.json lacks the key {key!r}")
    return mapping[key]


def _feed_forward(mlp, where: str) -> VunepelFeedForward | None:
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind == "dense":
        return VunepelFeedForward("dense", int(_need(mlp, "ff", where)), float(_need(mlp, "limit", where)))
    if kind != "moe":
        raise ConfigError(f"{where}: the Vunepel design has no feed-forward {kind!r}")
    router = _need(mlp, "router", where)
    expert = _need(mlp, "expert", where)
    shared = mlp.get("shared")
    return VunepelFeedForward(
        "moe", int(_need(expert, "ff", f"{where}.expert")), float(_need(expert, "limit", f"{where}.expert")),
        experts=int(_need(router, "experts", f"{where}.router")), top=int(_need(router, "top", f"{where}.router")),
        route_scale=float(router.get("scale", 1.0)),
        shared_ff=int(_need(shared, "ff", f"{where}.shared")) if shared is not None else 0,
        shared_limit=float(_need(shared, "limit", f"{where}.shared")) if shared is not None else 0.0)


@dataclass(frozen=True)
class VunepelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[VunepelLayer, ...]
    architecture: str = "Vunepel"
    raw: Mapping[str, Any] = field(default_factory=dict, repr=False, compare=False)

    family = "vunepel"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "VunepelConfig":
        if not isinstance(raw, Mapping):
            raise TypeError(f"unsupported config type: {type(raw)!r}")
        entries = _need(raw, "layers", "")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            kind = _need(entry, "type", where)
            mixer = _need(entry, "mixer", where)
            heads = int(_need(mixer, "heads", f"{where}.mixer"))
            dim = int(_need(mixer, "dim", f"{where}.mixer"))
            common = dict(type=kind, heads=heads, kv_heads=int(mixer.get("kv_heads") or heads), dim=dim,
                          vdim=int(mixer.get("vdim") or dim), mlp=_feed_forward(entry.get("mlp"), f"{where}.mlp"))
            if kind == "attention":
                rot = mixer.get("rot") or {}
                mask = mixer.get("mask") or {}
                layers.append(VunepelLayer(
                    **common, scale=float(_need(mixer, "scale", f"{where}.mixer")), diff=float(_need(mixer, "diff", f"{where}.mixer")),
                    rot_dims=int(rot.get("dims") or 0), rot_base=float(rot.get("base", 10000.0)),
                    chunk=int(mask["size"]) if mask.get("size") is not None else None,
                    kv_from=int(mixer["kv_from"]) if mixer.get("kv_from") is not None else None))
            elif kind == "channel_delta":
                ranks = mixer.get("ranks") or {}
                layers.append(VunepelLayer(**common, conv=int(mixer.get("conv") or 1), decay_rank=int(ranks.get("decay") or 0),
                                           gate_rank=int(ranks.get("gate") or 0)))
            else:
                raise ConfigError(f"{where}: the Vunepel design has no mixer {kind!r}")
        config = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                     norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm")), layers=tuple(layers),
                     architecture=str(raw.get("architecture", "Vunepel")), raw=dict(raw))
        config.validate()
        return config

    def with_tensor_shapes(self, shapes: Mapping[str, tuple[int, ...]]) -> "VunepelConfig":
        """The sizes that only the stored tensors give: the column counts of the recurrent layers' narrow projections
        (``l<i>.mix.a1`` is [decay columns, width], ``l<i>.mix.g1`` [gate columns, width])."""
        layers = []
        for index, layer in enumerate(self.layers):
            if layer.type == "channel_delta":
                found = {}
                for key, name in (("decay_rank", f"l{index}.mix.a1"), ("gate_rank", f"l{index}.mix.g1")):
                    shape = shapes.get(name)
                    if shape is not None and len(shape) == 2:
                        found[key] = int(shape[0])
                layer = replace(layer, **found)
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def validate(self) -> None:
        problems: list[str] = []
        if self.vocab <= 0 or self.width <= 0:
            problems.append("vocab and width must be positive")
        if self.norm_eps <= 0.0:
            problems.append("norm.eps must be positive")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if min(layer.heads, layer.kv_heads, layer.dim, layer.vdim) <= 0:
                problems.append(f"{where}: heads, kv_heads, dim and vdim must be positive")
                continue
            if layer.heads % layer.kv_heads:
                problems.append(f"{where}: heads={layer.heads} is not a multiple of kv_heads={layer.kv_heads}")
            if layer.type == "attention":
                if layer.rot_dims % 2 or layer.rot_dims > layer.dim or layer.rot_dims < 0:
                    problems.append(f"{where}: rot.dims={layer.rot_dims} must be even and at most dim={layer.dim}")
                if layer.chunk is not None and layer.chunk <= 0:
                    problems.append(f"{where}: mask.size={layer.chunk} must be positive")
                if layer.kv_from is not None:
                    source = self.layers[layer.kv_from] if 0 <= layer.kv_from < index else None
                    if source is None or source.type != "attention" or source.kv_from is not None:
                        problems.append(f"{where}: kv_from={layer.kv_from} must name an earlier attention layer with keys and values of its own")
                    elif (source.heads, source.kv_heads, source.dim, source.vdim, source.rot_dims, source.rot_base) != \
                            (layer.heads, layer.kv_heads, layer.dim, layer.vdim, layer.rot_dims, layer.rot_base):
                        problems.append(f"{where}: head counts, sizes and rotation differ from those of layer {layer.kv_from}, whose keys it reads")
            elif not 1 <= layer.conv <= 16:
                problems.append(f"{where}: conv={layer.conv} taps (1..16)")
            mlp = layer.mlp
            if mlp is not None:
                if mlp.ff <= 0 or mlp.limit <= 0:
                    problems.append(f"{where}.mlp: ff={mlp.ff}, limit={mlp.limit}")
                if mlp.kind == "moe" and not 0 < mlp.top <= mlp.experts:
                    problems.append(f"{where}.mlp: top={mlp.top} of experts={mlp.experts}")
        if problems:
            raise ConfigError("invalid Vunepel configuration: " + "; ".join(problems))

    # ------------------------------------------------------------------ export
    def to_hf_dict(self) -> dict[str, Any]:
        """The config.json that parses back into this configuration."""
        layers = []
        for layer in self.layers:
            mixer: dict[str, Any] = {"dim": layer.dim, "heads": layer.heads, "kv_heads": layer.kv_heads, "vdim": layer.vdim}
            if layer.type == "attention":
                mixer.update(diff=layer.diff, scale=layer.scale)
                if layer.rot_dims:
                    mixer["rot"] = {"base": layer.rot_base, "dims": layer.rot_dims}
                if layer.chunk is not None:
                    mixer["mask"] = {"size": layer.chunk}
                if layer.kv_from is not None:
                    mixer["kv_from"] = layer.kv_from
            else:
                mixer["conv"] = layer.conv
                if layer.decay_rank or layer.gate_rank:
                    mixer["ranks"] = {"decay": layer.decay_rank, "gate": layer.gate_rank}
            mlp = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                mlp = {"ff": layer.mlp.ff, "kind": "dense", "limit": layer.mlp.limit}
            elif layer.mlp is not None:
                mlp = {"expert": {"ff": layer.mlp.ff, "limit": layer.mlp.limit}, "kind": "moe",
                       "router": {"experts": layer.mlp.experts, "scale": layer.mlp.route_scale, "top": layer.mlp.top}}
                if layer.mlp.shared_ff:
                    mlp["shared"] = {"ff": layer.mlp.shared_ff, "limit": layer.mlp.shared_limit}
            layers.append({"mixer": mixer, "mlp": mlp, "type": layer.type})
        return {"architecture": self.architecture, "layers": layers, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def model_spec(self) -> ModelSpec:
        norm_params = {"size": self.width, "suffix": "", "bias_suffix": ".b", "alpha_suffix": ".alpha"}
        norm = PartSpec("dynamic_tanh", norm_params)
        block = PartSpec("parallel", {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1"})
        init_std = 0.06
        layers, schedule = [], []
        for index, layer in enumerate(self.layers):
            if layer.type == "attention":
                position = PartSpec("rope", {"theta": layer.rot_base, "rotary_dim": layer.rot_dims, "head_dim": layer.dim, "angles": "float64"}) \
                    if layer.rot_dims else PartSpec("none")
                mixer = PartSpec("attention", {
                    "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                    "v_head_dim": layer.vdim, "scale": layer.scale, "maps": 2, "diff": layer.diff, "head_norm_eps": self.norm_eps,
                    "chunk": layer.chunk, "own_kv": layer.kv_from is None, "qk_norm": True, "qk_norm_eps": self.norm_eps,
                    "position": position, "float_out": True, "init_std": init_std,
                    "q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "weight_suffix": "", "norm_suffix": ""})
            else:
                if not (layer.decay_rank and layer.gate_rank):
                    raise ConfigError(f"layers[{index}]: the column counts of the narrow projections are unknown: they are the shapes "
                                      f"of l{index}.mix.a1 and l{index}.mix.g1 in a model folder, or mixer.ranks in the configuration")
                mixer = PartSpec("gated_delta_rule", {
                    "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                    "v_head_dim": layer.vdim, "conv": layer.conv, "eps": self.norm_eps, "decay_rank": layer.decay_rank,
                    "gate_rank": layer.gate_rank, "float_out": True, "init_std": init_std,
                    "beta": "b", "decay_in": "a1", "decay_out": "a2", "decay_bias": "dt_bias", "decay_rate": "A_log",
                    "gate_in": "g1", "gate_out": "g2", "norm": "norm", "weight_suffix": "", "conv_suffix": ".conv"})
            feed_forward = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                feed_forward = PartSpec("gated_mlp", {
                    "hidden_size": self.width, "intermediate_size": layer.mlp.ff, "activation": "capped_sigmoid", "limit": layer.mlp.limit,
                    "gate": "gate", "up": "up", "down": "down", "weight_suffix": "", "float_out": True, "init_std": init_std})
            elif layer.mlp is not None:
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": self.width, "expert_size": layer.mlp.ff, "experts": layer.mlp.experts, "top": layer.mlp.top,
                    "route_scale": layer.mlp.route_scale, "activation": "capped_sigmoid", "limit": layer.mlp.limit,
                    "shared": {"intermediate_size": layer.mlp.shared_ff, "limit": layer.mlp.shared_limit} if layer.mlp.shared_ff else None,
                    "router": "router", "expert": "e{}", "gate": "gate", "up": "up", "down": "down", "shared_name": "shared",
                    "shared_gate": "sg", "weight_suffix": "", "init_std": init_std})
            layers.append(LayerSpec(prefix=f"l{index}", block=block, mixer=mixer, feed_forward=feed_forward, norm=norm))
            schedule.append(LayerCall(layer=index, cache_of=layer.kv_from))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("token_embedding", {"name": "embed", "init_std": 0.5}),
            layers=tuple(layers), schedule=tuple(schedule),
            final_norm=PartSpec("dynamic_tanh", {**norm_params, "name": "final.norm"}),
            head=PartSpec("linear_head", {"name": "head", "tied_to": None, "init_std": 0.25}),
            max_positions=MAX_POSITIONS, eos_token_ids=(),
        )
        spec.validate()
        return spec
