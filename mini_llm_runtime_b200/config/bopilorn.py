"""Typed configuration of the ``Bopilorn`` architecture, read from the keys of its config.json, and
its layout as parts.

A Bopilorn model is a stack of layers given one by one in config.json's ``layers`` list: every entry
names its mixer (``type``: ``attention``), the mixer's sizes and constants (``mixer``) and its
feed-forward (``mlp``: ``{"kind": "moe", "expert": {"ff": n}, "router": {...}}`` or null).  The token
embedding is multiplied by ``embedding.scale``; the residual stream is 32-bit; every sublayer sits
between two layer norms that have a weight and no bias; a final norm of the same kind and a head
matrix of its own give the logits.

The mixer is grouped-query softmax attention over all earlier keys.  Queries and keys are
RMS-normalised over their whole projection (all heads at once, one weight per entry) and turned by
their positions over the first ``rot.dims`` entries of each head, pairs (2i, 2i + 1), with the
frequencies optionally rescaled (``rot.scaling``); values are brought to unit root mean square per
head, turned by their own positions over all their entries before they are cached, and each head's
output is turned back by the query's position.  The score scale is a constant of the layer.

The feed-forward is a routed set of small gated experts: softmax router in 32-bit, a per-expert
correction that enters the choice only, a choice restricted to the best groups of neighbouring
experts, weights that are the chosen experts' own softmax scores (not renormalised).

No size or constant of a model stands in code: all of them come from config.json, tensor shapes are
derived from them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

# what the design fixes for its one mixer kind
MIXER_KINDS = {
    "attention": {"rope_layout": "interleaved", "qk_norm": "projection", "value_norm": True, "value_rotation": True},
}
UNLIMITED_POSITIONS = 1 << 30     # the design sets no position limit


def _positive(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) <= 0:
        raise ValueError(f"Bopilorn config: {what} must be a positive integer, got {value!r}")
    return int(value)


def _number(value, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ValueError(f"Bopilorn config: {what} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class BopilornLayer:
    """One entry of ``layers``: the mixer's kind with its arguments, and the feed-forward's (empty:
    none), both as sorted tuples of items (hashable)."""

    type: str
    mixer: tuple
    mlp: tuple = ()

    @property
    def mixer_args(self) -> dict[str, Any]:
        return dict(self.mixer)

    @property
    def mlp_args(self) -> dict[str, Any]:
        return dict(self.mlp)


def _mixer_from_dict(where: str, mixer: Mapping[str, Any]) -> dict[str, Any]:
    args: dict[str, Any] = {name: _positive(mixer.get(name), f"{where}.{name}") for name in ("heads", "dim", "vdim")}
    args["kv_heads"] = _positive(mixer.get("kv_heads", args["heads"]), f"{where}.kv_heads")
    if args["heads"] % args["kv_heads"]:
        raise ValueError(f"Bopilorn config: {where}.heads must be a multiple of kv_heads")
    if args["vdim"] % 2:
        raise ValueError(f"Bopilorn config: {where}.vdim must be even (values are turned in pairs)")
    if "scale" not in mixer:
        raise KeyError(f"Bopilorn config: {where} lacks 'scale'")
    args["scale"] = _number(mixer["scale"], f"{where}.scale")
    rot = mixer.get("rot")
    if not isinstance(rot, Mapping) or "base" not in rot:
        raise KeyError(f"Bopilorn config: {where} lacks the object 'rot' with 'base'")
    args["rope_base"] = _number(rot["base"], f"{where}.rot.base")
    args["rope_dims"] = _positive(rot.get("dims", args["dim"]), f"{where}.rot.dims")
    if args["rope_dims"] % 2 or args["rope_dims"] > args["dim"]:
        raise ValueError(f"Bopilorn config: {where}.rot.dims must be even and at most dim")
    scaling = rot.get("scaling")
    args["rope_scaling"] = ()
    if scaling is not None:
        if not isinstance(scaling, Mapping) or any(name not in scaling for name in ("factor", "original", "fast", "slow")):
            raise KeyError(f"Bopilorn config: {where}.rot.scaling needs 'factor', 'original', 'fast' and 'slow'")
        args["rope_scaling"] = tuple((name, _number(scaling[name], f"{where}.rot.scaling.{name}"))
                                     for name in ("factor", "original", "fast", "slow"))
    return args


def _mlp_from_dict(where: str, mlp: Mapping[str, Any]) -> dict[str, Any]:
    if mlp.get("kind") != "moe":
        raise ValueError(f"Bopilorn config: {where} has feed-forward kind {mlp.get('kind')!r}; known: moe")
    expert, router = mlp.get("expert"), mlp.get("router")
    if not isinstance(expert, Mapping) or not isinstance(router, Mapping):
        raise KeyError(f"Bopilorn config: {where} needs the objects 'expert' and 'router'")
    args = {"ff": _positive(expert.get("ff"), f"{where}.expert.ff"),
            "experts": _positive(router.get("experts"), f"{where}.router.experts"),
            "top": _positive(router.get("top"), f"{where}.router.top")}
    groups = router.get("groups")
    args["groups"], args["keep"], args["groups_given"] = 1, 1, groups is not None
    if groups is not None:
        if not isinstance(groups, Mapping):
            raise KeyError(f"Bopilorn config: {where}.router.groups must be an object with 'count' and 'keep'")
        args["groups"] = _positive(groups.get("count"), f"{where}.router.groups.count")
        args["keep"] = _positive(groups.get("keep"), f"{where}.router.groups.keep")
    if args["experts"] % args["groups"] or args["keep"] > args["groups"]:
        raise ValueError(f"Bopilorn config: {where}.router needs experts divisible by groups.count and keep <= count")
    if args["top"] > args["keep"] * (args["experts"] // args["groups"]):
        raise ValueError(f"Bopilorn config: {where}.router.top exceeds the experts of the kept groups")
    return args


def _layer_from_dict(index: int, data: Mapping[str, Any]) -> BopilornLayer:
    kind = data.get("type")
    if kind not in MIXER_KINDS:
        raise ValueError(f"Bopilorn config: layer {index} has type {kind!r}; known: {', '.join(MIXER_KINDS)}")
    mixer = data.get("mixer")
    if not isinstance(mixer, Mapping):
        raise KeyError(f"Bopilorn config: layer {index} lacks the object 'mixer'")
    args = _mixer_from_dict(f"layer {index} mixer", mixer)
    mlp = data.get("mlp")
    mlp_args = {} if mlp is None else _mlp_from_dict(f"layer {index} mlp", mlp)
    return BopilornLayer(kind, tuple(sorted(args.items())), tuple(sorted(mlp_args.items())))


def _layer_to_dict(layer: BopilornLayer) -> dict[str, Any]:
    args = layer.mixer_args
    rot: dict[str, Any] = {"base": args["rope_base"], "dims": args["rope_dims"]}
    if args["rope_scaling"]:
        rot["scaling"] = dict(args["rope_scaling"])
    mixer = {"heads": args["heads"], "kv_heads": args["kv_heads"], "dim": args["dim"], "vdim": args["vdim"],
             "scale": args["scale"], "rot": rot}
    mlp = None
    if layer.mlp:
        m = layer.mlp_args
        router: dict[str, Any] = {"experts": m["experts"], "top": m["top"]}
        if m["groups_given"]:
            router["groups"] = {"count": m["groups"], "keep": m["keep"]}
        mlp = {"kind": "moe", "expert": {"ff": m["ff"]}, "router": router}
    return {"type": layer.type, "mixer": mixer, "mlp": mlp}


@dataclass(frozen=True)
class BopilornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[BopilornLayer, ...]
    max_positions: int = UNLIMITED_POSITIONS

    architecture = "Bopilorn"

    def __post_init__(self) -> None:
        for name in ("vocab", "width", "max_positions"):
            if getattr(self, name) <= 0:
                raise ValueError(f"Bopilorn config: {name} must be > 0")
        if self.norm_eps <= 0:
            raise ValueError("Bopilorn config: norm.eps must be > 0")
        if not self.layers:
            raise ValueError("Bopilorn config: 'layers' must list at least one layer")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "BopilornConfig":
        missing = [name for name in ("vocab", "width", "norm", "layers", "embedding") if name not in data]
        if missing:
            raise KeyError(f"config.json lacks these keys: {', '.join(missing)}")
        norm, embedding = data["norm"], data["embedding"]
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise KeyError("config.json: 'norm' must be an object with the key 'eps'")
        if not isinstance(embedding, Mapping) or "scale" not in embedding:
            raise KeyError("config.json: 'embedding' must be an object with the key 'scale'")
        layers = data["layers"]
        if not isinstance(layers, (list, tuple)):
            raise ValueError("config.json: 'layers' must be a list")
        return cls(vocab=_positive(data["vocab"], "vocab"), width=_positive(data["width"], "width"),
                   norm_eps=_number(norm["eps"], "norm.eps"),
                   embedding_scale=_number(embedding["scale"], "embedding.scale"),
                   layers=tuple(_layer_from_dict(i, layer) for i, layer in enumerate(layers)),
                   max_positions=int(data.get("max_positions", UNLIMITED_POSITIONS)))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
               "layers": [_layer_to_dict(layer) for layer in self.layers]}
        if self.max_positions != UNLIMITED_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


def bopilorn_model_spec(config: BopilornConfig) -> ModelSpec:
    """Bopilorn as parts.  Tensor names: ``embed``, ``l<i>.norm1|norm2|norm1b|norm2b``,
    ``l<i>.mix.{q,k,v,o,q.norm,k.norm}``, ``l<i>.mlp.{router,correction}``,
    ``l<i>.mlp.e<j>.{gate,up,down}``, ``final.norm``, ``head``."""
    width, eps = config.width, config.norm_eps
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        kind = MIXER_KINDS[layer.type]
        args = {**layer.mixer_args, "hidden_size": width, "eps": eps, **kind}

        def norm(name):
            return PartSpec("layer_norm", {"size": width, "eps": eps, "tensor": prefix + name, "bias": False})

        feed_forward = feed_forward_norm = None
        extras = [("mixer_post_norm", "norm", norm("norm1b"))]
        if layer.mlp:
            m = layer.mlp_args
            feed_forward = PartSpec("routed_experts", {
                "hidden_size": width, "intermediate_size": m["ff"], "experts": m["experts"], "top": m["top"],
                "groups": m["groups"], "keep": m["keep"], "activation": "silu", "scoring": "softmax",
                "renormalise": False}, prefix + "mlp.")
            feed_forward_norm = norm("norm2")
            extras.append(("feed_forward_post_norm", "norm", norm("norm2b")))
        layers.append(LayerSpec(block="sandwich_norm", mixer=PartSpec("rotated_value_attention", args, prefix + "mix."),
                                feed_forward=feed_forward, mixer_norm=norm("norm1"),
                                feed_forward_norm=feed_forward_norm, extra_parts=tuple(extras)))
    return ModelSpec(
        architecture=config.architecture, vocab_size=config.vocab, hidden_size=width,
        max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "embed",
                                               "rows": "float32", "scale": config.embedding_scale}),
        layers=tuple(layers),
        run_order=tuple(RunStep(layer=index, cache=index) for index in range(len(config.layers))),
        final_norm=PartSpec("layer_norm", {"size": width, "eps": eps, "tensor": "final.norm", "bias": False}),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "head"}),
    )
