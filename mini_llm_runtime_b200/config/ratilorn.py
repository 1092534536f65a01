"""Typed configuration of the ``Ratilorn`` architecture, read from the keys of its config.json, and
its layout as parts.

A Ratilorn model is a stack of layers given one by one in config.json's ``layers`` list: every entry
names its mixer (``type``: ``attention`` or ``parallel``), the mixer's sizes and constants (``mixer``)
and its feed-forward (``mlp``: ``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n},
"router": {...}, "shared": {"ff": n}}`` or null).  The token embedding gets a learned position vector;
the residual stream is 32-bit; the norms sit on the sublayers' outputs only (x <- x + norm(sublayer(x)),
the sublayers read x itself) and store their weights as offsets from one; the head is the embedding table and
the logits are multiplied by ``logit_scale``.

``attention``: grouped-query attention without a rotation whose q and k are divided by their root mean
square per head, whose weights are sigmoid(score - r1 ln(1 + r2 distance) + b) without normalisation
over the keys and are mixed across heads; layers with ``v_mix`` blend their values with those of the
first such layer.  ``parallel``: an ordinary softmax attention (q and k RMS-normalised per head with a
learned weight, no rotation) beside a selective state-space layer with a scalar decay per head, both
reading the same rows; the mean of their RMS-normalised outputs is the mixer's output.

The feed-forward is a gated layer (silu), dense or a routed set of small experts with a sigmoid
router, a correction that enters the choice only, groups ranked by the sum of their two best choice
scores, renormalised weights and a shared expert.

No size or constant of a model stands in code: all of them come from config.json, tensor shapes are
derived from them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("attention", "parallel")
# what the design fixes
GROUP_SCORE_TOP = 2            # a group of experts is ranked by the sum of this many of its best choice scores
RENORM_EPS = 1e-20             # added to the sum the chosen experts' scores are divided by


def _positive(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) <= 0:
        raise ValueError(f"Ratilorn config: {what} must be a positive integer, got {value!r}")
    return int(value)


def _number(value, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ValueError(f"Ratilorn config: {what} must be a number, got {value!r}")
    return float(value)


def _freeze(value):
    """Nested dicts as sorted tuples of items (hashable), and back with ``_thaw``."""
    if isinstance(value, Mapping):
        return tuple(sorted((key, _freeze(item)) for key, item in value.items()))
    return value


def _thaw(value):
    if isinstance(value, tuple) and all(isinstance(item, tuple) and len(item) == 2 and isinstance(item[0], str)
                                        for item in value):
        return {key: _thaw(item) for key, item in value}
    return value


@dataclass(frozen=True)
class RatilornLayer:
    """One entry of ``layers``: the mixer's kind with its arguments, and the feed-forward's (empty:
    none), both frozen into sorted tuples of items."""

    type: str
    mixer: tuple
    mlp: tuple = ()

    @property
    def mixer_args(self) -> dict[str, Any]:
        return _thaw(self.mixer)

    @property
    def mlp_args(self) -> dict[str, Any]:
        return _thaw(self.mlp) if self.mlp else {}


def _attention_from_dict(where: str, mixer: Mapping[str, Any], *, v_mix_allowed: bool) -> dict[str, Any]:
    args: dict[str, Any] = {name: _positive(mixer.get(name), f"{where}.{name}") for name in ("heads", "dim", "vdim")}
    args["kv_heads"] = _positive(mixer.get("kv_heads", args["heads"]), f"{where}.kv_heads")
    if args["heads"] % args["kv_heads"]:
        raise ValueError(f"Ratilorn config: {where}.heads must be a multiple of kv_heads")
    if "scale" not in mixer:
        raise KeyError(f"Ratilorn config: {where} lacks 'scale'")
    args["scale"] = _number(mixer["scale"], f"{where}.scale")
    if v_mix_allowed:
        args["v_mix"] = bool(mixer.get("v_mix", False))
    return args


def _state_space_from_dict(where: str, mixer: Mapping[str, Any]) -> dict[str, Any]:
    args = {name: _positive(mixer.get(name), f"{where}.{name}") for name in ("heads", "vdim", "state", "conv")}
    args["groups"] = _positive(mixer.get("groups", 1), f"{where}.groups")
    args["norm_groups"] = _positive(mixer.get("norm_groups", 1), f"{where}.norm_groups")
    if args["heads"] % args["groups"]:
        raise ValueError(f"Ratilorn config: {where}.heads must be a multiple of groups")
    if (args["heads"] * args["vdim"]) % args["norm_groups"]:
        raise ValueError(f"Ratilorn config: {where}.norm_groups must divide heads * vdim")
    if args["conv"] < 2:
        raise ValueError(f"Ratilorn config: {where}.conv must be at least 2 taps")
    return args


def _gated_from_dict(where: str, data) -> int:
    if not isinstance(data, Mapping):
        raise KeyError(f"Ratilorn config: {where} must be an object with 'ff'")
    return _positive(data.get("ff"), f"{where}.ff")


def _mlp_from_dict(where: str, mlp: Mapping[str, Any]) -> dict[str, Any]:
    kind = mlp.get("kind")
    if kind == "dense":
        return {"kind": "dense", "ff": _positive(mlp.get("ff"), f"{where}.ff")}
    if kind != "moe":
        raise ValueError(f"Ratilorn config: {where} has feed-forward kind {kind!r}; known: dense, moe")
    router = mlp.get("router")
    if not isinstance(router, Mapping):
        raise KeyError(f"Ratilorn config: {where} needs the object 'router'")
    args: dict[str, Any] = {"kind": "moe", "ff": _gated_from_dict(f"{where}.expert", mlp.get("expert")),
                            "experts": _positive(router.get("experts"), f"{where}.router.experts"),
                            "top": _positive(router.get("top"), f"{where}.router.top")}
    groups = router.get("groups")
    args["groups"], args["keep"], args["groups_given"] = 1, 1, groups is not None
    if groups is not None:
        if not isinstance(groups, Mapping):
            raise KeyError(f"Ratilorn config: {where}.router.groups must be an object with 'count' and 'keep'")
        args["groups"] = _positive(groups.get("count"), f"{where}.router.groups.count")
        args["keep"] = _positive(groups.get("keep"), f"{where}.router.groups.keep")
    if args["experts"] % args["groups"] or args["keep"] > args["groups"]:
        raise ValueError(f"Ratilorn config: {where}.router needs experts divisible by groups.count and keep <= count")
    if args["top"] > args["keep"] * (args["experts"] // args["groups"]):
        raise ValueError(f"Ratilorn config: {where}.router.top exceeds the experts of the kept groups")
    args["shared"] = 0 if mlp.get("shared") is None else _gated_from_dict(f"{where}.shared", mlp["shared"])
    return args


def _layer_from_dict(index: int, data: Mapping[str, Any]) -> RatilornLayer:
    kind = data.get("type")
    if kind not in MIXER_TYPES:
        raise ValueError(f"Ratilorn config: layer {index} has type {kind!r}; known: {', '.join(MIXER_TYPES)}")
    mixer = data.get("mixer")
    if not isinstance(mixer, Mapping):
        raise KeyError(f"Ratilorn config: layer {index} lacks the object 'mixer'")
    where = f"layer {index} mixer"
    if kind == "attention":
        args = _attention_from_dict(where, mixer, v_mix_allowed=True)
    else:
        if not isinstance(mixer.get("left"), Mapping) or not isinstance(mixer.get("right"), Mapping):
            raise KeyError(f"Ratilorn config: {where} needs the objects 'left' and 'right'")
        args = {"left": _attention_from_dict(where + ".left", mixer["left"], v_mix_allowed=False),
                "right": _state_space_from_dict(where + ".right", mixer["right"])}
    mlp = data.get("mlp")
    mlp_args = {} if mlp is None else _mlp_from_dict(f"layer {index} mlp", mlp)
    return RatilornLayer(kind, _freeze(args), _freeze(mlp_args))


def _attention_to_dict(args: Mapping[str, Any]) -> dict[str, Any]:
    out = {name: args[name] for name in ("heads", "kv_heads", "dim", "vdim", "scale")}
    if args.get("v_mix"):
        out["v_mix"] = True
    return out


def _layer_to_dict(layer: RatilornLayer) -> dict[str, Any]:
    args = layer.mixer_args
    if layer.type == "attention":
        mixer = _attention_to_dict(args)
    else:
        mixer = {"left": _attention_to_dict(args["left"]), "right": dict(args["right"])}
    mlp = None
    if layer.mlp:
        m = layer.mlp_args
        if m["kind"] == "dense":
            mlp = {"kind": "dense", "ff": m["ff"]}
        else:
            router: dict[str, Any] = {"experts": m["experts"], "top": m["top"]}
            if m["groups_given"]:
                router["groups"] = {"count": m["groups"], "keep": m["keep"]}
            mlp = {"kind": "moe", "expert": {"ff": m["ff"]}, "router": router}
            if m["shared"]:
                mlp["shared"] = {"ff": m["shared"]}
    return {"type": layer.type, "mixer": mixer, "mlp": mlp}


@dataclass(frozen=True)
class RatilornConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_scale: float
    layers: tuple[RatilornLayer, ...]

    architecture = "Ratilorn"

    def __post_init__(self) -> None:
        for name in ("vocab", "width", "max_positions"):
            if getattr(self, name) <= 0:
                raise ValueError(f"Ratilorn config: {name} must be > 0")
        if self.norm_eps <= 0:
            raise ValueError("Ratilorn config: norm.eps must be > 0")
        if not self.layers:
            raise ValueError("Ratilorn config: 'layers' must list at least one layer")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RatilornConfig":
        missing = [name for name in ("vocab", "width", "max_positions", "norm", "layers") if name not in data]
        if missing:
            raise KeyError(f"config.json lacks these keys: {', '.join(missing)}")
        norm = data["norm"]
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise KeyError("config.json: 'norm' must be an object with the key 'eps'")
        layers = data["layers"]
        if not isinstance(layers, (list, tuple)):
            raise ValueError("config.json: 'layers' must be a list")
        return cls(vocab=_positive(data["vocab"], "vocab"), width=_positive(data["width"], "width"),
                   max_positions=_positive(data["max_positions"], "max_positions"),
                   norm_eps=_number(norm["eps"], "norm.eps"),
                   logit_scale=_number(data.get("logit_scale", 1.0), "logit_scale"),
                   layers=tuple(_layer_from_dict(i, layer) for i, layer in enumerate(layers)))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "logit_scale": self.logit_scale, "layers": [_layer_to_dict(layer) for layer in self.layers]}


def _softmax_attention_spec(args, width, eps, prefix) -> PartSpec:
    return PartSpec("head_norm_attention", {
        "hidden_size": width, "eps": eps, "heads": args["heads"], "kv_heads": args["kv_heads"], "dim": args["dim"],
        "vdim": args["vdim"], "scale": args["scale"], "bias": True, "qk_norm_weight": True, "weights": "softmax"}, prefix)


def ratilorn_model_spec(config: RatilornConfig) -> ModelSpec:
    """Ratilorn as parts.  Tensor names: ``embed``, ``pos``, ``l<i>.norm1|norm2``, ``l<i>.mix.*`` (an
    attention layer), ``l<i>.mix.left.*`` / ``l<i>.mix.right.*`` (a parallel layer),
    ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router,correction}``, ``l<i>.mlp.e<j>.{gate,up,down}`` and
    ``l<i>.mlp.shared.{gate,up,down}``, ``final.norm``."""
    width, eps = config.width, config.norm_eps
    layers = []
    value_source_seen = False
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        args = layer.mixer_args

        def norm(name):
            return PartSpec("stream_rms_norm", {"size": width, "eps": eps, "tensor": prefix + name, "one_plus": True})

        if layer.type == "attention":
            value_mix = None
            if args.get("v_mix"):
                value_mix = "blend" if value_source_seen else "source"
                value_source_seen = True
            mixer = PartSpec("head_norm_attention", {
                "hidden_size": width, "eps": eps, "heads": args["heads"], "kv_heads": args["kv_heads"],
                "dim": args["dim"], "vdim": args["vdim"], "scale": args["scale"], "bias": True,
                "qk_norm_weight": False, "weights": "sigmoid", "distance_bias": True, "score_bias": True,
                "head_mix": True, "value_mix": value_mix}, prefix + "mix.")
        else:
            left = _softmax_attention_spec(args["left"], width, eps, prefix + "mix.left.")
            right = PartSpec("state_space", {"hidden_size": width, "eps": eps, **args["right"]}, prefix + "mix.right.")
            mixer = PartSpec("parallel_mixers", {
                "hidden_size": width, "eps": eps,
                "branches": (("left", left, prefix + "mix.left.out"), ("right", right, prefix + "mix.right.out"))},
                prefix + "mix.")
        feed_forward = feed_forward_norm = None
        if layer.mlp:
            m = layer.mlp_args
            feed_forward_norm = norm("norm2")
            if m["kind"] == "dense":
                feed_forward = PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": m["ff"],
                                                      "activation": "silu", "names": ("gate", "up", "down")},
                                        prefix + "mlp.")
            else:
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": width, "intermediate_size": m["ff"], "experts": m["experts"], "top": m["top"],
                    "groups": m["groups"], "keep": m["keep"], "group_top": GROUP_SCORE_TOP, "activation": "silu",
                    "scoring": "sigmoid", "renormalise": True, "renorm_eps": RENORM_EPS, "shared": m["shared"]},
                    prefix + "mlp.")
        layers.append(LayerSpec(block="post_norm_residual", mixer=mixer, feed_forward=feed_forward,
                                mixer_norm=norm("norm1"), feed_forward_norm=feed_forward_norm))
    return ModelSpec(
        architecture=config.architecture, vocab_size=config.vocab, hidden_size=width,
        max_positions=config.max_positions,
        embedding=PartSpec("token_position_embedding",
                           {"vocab_size": config.vocab, "hidden_size": width, "max_positions": config.max_positions,
                            "token_tensor": "embed", "position_tensor": "pos"}),
        layers=tuple(layers),
        run_order=tuple(RunStep(layer=i, cache=i) for i in range(len(layers))),
        final_norm=PartSpec("stream_rms_norm", {"size": width, "eps": eps, "tensor": "final.norm", "one_plus": True}),
        head=PartSpec("tied_head", {"vocab_size": config.vocab, "hidden_size": width, "tied_to": "embed",
                                    "scale": config.logit_scale, "own_copy": False}),
    )
