"""Typed configuration of the Lederax design, read from config.json.

The file names its design under ``architecture`` and gives every size and constant that can differ between
models: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and ``norm.groups``, and a list ``layers`` whose
entries each give ``type`` (the mixer; the design has ``attention``), the mixer's sizes and constants under
``mixer`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``v_mix``) and the feed-forward
under ``mlp`` (``kind`` "moe" with ``router.experts``, ``router.top`` and ``expert.ff``; null for a layer without
one).  Layers need not be alike.

What the design fixes, and ``model_spec`` therefore states as parameters of the parts: projections q, k, v carry a
bias and o does not; no rotation; every value head is divided by its root mean square (the norm's eps); scores lose
r1 ln(1 + r2 distance) per head; the layers marked ``v_mix`` share the first marked layer's values (it is the
"source", the later ones "blend"); experts are up -> exact GELU -> down without biases, chosen by a table over
token ids, averaged; the norm is an RMS norm in groups; tensor names are ``embed``, ``head``, ``final.norm`` and
``l<i>.{norm1,norm2,mix.*,mlp.*}`` without a ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .qwen3 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MAX_POSITIONS = 1 << 24          # the design has no position table and no longest sequence; the cache sets the limit


@dataclass(frozen=True)
class LederaxExperts:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class LederaxLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None              # a query sees itself and the window - 1 tokens before it; None: all before it
    v_mix: bool
    mlp: LederaxExperts | None


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or mapping.get(key) is None:
        raise ConfigError(f"config.json lacks {where}.{key}" if where else f"config.json lacks the key {key!r}")
    return mapping[key]


@dataclass(frozen=True)
class LederaxConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: tuple[LederaxLayer, ...]
    architecture: str = "Lederax"
    raw: Mapping[str, Any] = field(default_factory=dict, repr=False, compare=False)

    family = "lederax"

    # names the rest of the library asks a configuration for
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
    def from_hf_config(cls, raw: Mapping[str, Any]) -> "LederaxConfig":
        if not isinstance(raw, Mapping):
            raise TypeError(f"unsupported config type: {type(raw)!r}")
        layers = []
        entries = _need(raw, "layers", "")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            kind = _need(entry, "type", where)
            if kind != "attention":
                raise ConfigError(f"{where}: the Lederax design has no mixer {kind!r}")
            mixer = _need(entry, "mixer", where)
            mask = mixer.get("mask") or {}
            window = mask.get("size")
            mlp = entry.get("mlp")
            experts = None
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"{where}.mlp: the Lederax design has no feed-forward {mlp.get('kind')!r}")
                router = _need(mlp, "router", f"{where}.mlp")
                experts = LederaxExperts(experts=int(_need(router, "experts", f"{where}.mlp.router")),
                                         top=int(_need(router, "top", f"{where}.mlp.router")),
                                         ff=int(_need(_need(mlp, "expert", f"{where}.mlp"), "ff", f"{where}.mlp.expert")))
            heads = int(_need(mixer, "heads", f"{where}.mixer"))
            dim = int(_need(mixer, "dim", f"{where}.mixer"))
            layers.append(LederaxLayer(
                heads=heads, kv_heads=int(mixer.get("kv_heads") or heads), dim=dim, vdim=int(mixer.get("vdim") or dim),
                scale=float(_need(mixer, "scale", f"{where}.mixer")), window=int(window) if window is not None else None,
                v_mix=bool(mixer.get("v_mix", False)), mlp=experts))
        norm = _need(raw, "norm", "")
        config = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                     embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                     norm_eps=float(_need(norm, "eps", "norm")), norm_groups=int(norm.get("groups", 1)),
                     layers=tuple(layers), architecture=str(raw.get("architecture", "Lederax")), raw=dict(raw))
        config.validate()
        return config

    def validate(self) -> None:
        problems: list[str] = []
        if self.vocab <= 0 or self.width <= 0:
            problems.append("vocab and width must be positive")
        if self.norm_eps <= 0.0:
            problems.append("norm.eps must be positive")
        if self.norm_groups <= 0 or (self.width > 0 and self.width % self.norm_groups):
            problems.append(f"norm.groups={self.norm_groups} does not divide width={self.width}")
        shared = None
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if min(layer.heads, layer.kv_heads, layer.dim, layer.vdim) <= 0:
                problems.append(f"{where}: heads, kv_heads, dim and vdim must be positive")
            elif layer.heads % layer.kv_heads:
                problems.append(f"{where}: heads={layer.heads} is not a multiple of kv_heads={layer.kv_heads}")
            if layer.window is not None and layer.window <= 0:
                problems.append(f"{where}: mask.size={layer.window} must be positive")
            if layer.v_mix:
                if shared is None:
                    shared = (layer.kv_heads, layer.vdim)
                elif shared != (layer.kv_heads, layer.vdim):
                    problems.append(f"{where}: a v_mix layer with kv_heads x vdim = {layer.kv_heads} x {layer.vdim} cannot "
                                    f"share values of {shared[0]} x {shared[1]}")
            if layer.mlp is not None and not (0 < layer.mlp.top <= layer.mlp.experts and layer.mlp.ff > 0):
                problems.append(f"{where}.mlp: top={layer.mlp.top}, experts={layer.mlp.experts}, ff={layer.mlp.ff}")
        if problems:
            raise ConfigError("invalid Lederax configuration: " + "; ".join(problems))

    # ------------------------------------------------------------------ export
    def to_hf_dict(self) -> dict[str, Any]:
        """The config.json that parses back into this configuration."""
        layers = []
        for layer in self.layers:
            mixer: dict[str, Any] = {"dim": layer.dim, "heads": layer.heads, "kv_heads": layer.kv_heads, "scale": layer.scale,
                                     "v_mix": layer.v_mix, "vdim": layer.vdim}
            if layer.window is not None:
                mixer["mask"] = {"size": layer.window}
            mlp = None
            if layer.mlp is not None:
                mlp = {"expert": {"ff": layer.mlp.ff}, "kind": "moe",
                       "router": {"experts": layer.mlp.experts, "top": layer.mlp.top}}
            layers.append({"mixer": mixer, "mlp": mlp, "type": "attention"})
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": layers,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "vocab": self.vocab, "width": self.width}

    def model_spec(self) -> ModelSpec:
        norm_params = {"size": self.width, "eps": self.norm_eps, "groups": self.norm_groups, "suffix": ""}
        norm = PartSpec("rmsnorm", norm_params)
        block = PartSpec("pre_norm", {"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1", "feed_forward_norm": "norm2"})
        first_marked = next((i for i, layer in enumerate(self.layers) if layer.v_mix), None)
        layers = []
        for index, layer in enumerate(self.layers):
            blend = None if not layer.v_mix else ("source" if index == first_marked else "blend")
            mixer = PartSpec("attention", {
                "hidden_size": self.width, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads,
                "head_dim": layer.dim, "v_head_dim": layer.vdim, "scale": layer.scale, "window": layer.window,
                "bias": True, "o_bias": False, "position": PartSpec("none"),
                "v_norm": True, "v_norm_eps": self.norm_eps, "v_blend": blend, "v_blend_key": "first",
                "v_blend_weight_stored": True, "distance_penalty": "log",
                "q": "q", "k": "k", "v": "v", "o": "o", "r1": "r1", "r2": "r2", "v_blend_weight": "vmix",
                "weight_suffix": "", "bias_suffix": ".b",
            })
            feed_forward = None
            if layer.mlp is not None:
                feed_forward = PartSpec("table_experts", {
                    "hidden_size": self.width, "expert_size": layer.mlp.ff, "experts": layer.mlp.experts,
                    "top": layer.mlp.top, "vocab_size": self.vocab, "activation": "gelu",
                    "table": "table", "expert": "e{}", "up": "up", "down": "down", "weight_suffix": "",
                })
            layers.append(LayerSpec(prefix=f"l{index}", block=block, mixer=mixer, feed_forward=feed_forward, norm=norm))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("token_embedding", {"name": "embed", "scale": self.embedding_scale, "init_std": 0.08}),
            layers=tuple(layers), schedule=tuple(LayerCall(layer=i) for i in range(len(layers))),
            final_norm=PartSpec("rmsnorm", {**norm_params, "name": "final.norm"}),
            head=PartSpec("linear_head", {"name": "head", "tied_to": None}),
            max_positions=MAX_POSITIONS, eos_token_ids=(),
        )
        spec.validate()
        return spec
