"""Typed configuration of the ``Zazasun`` architecture, read from the keys of its config.json, and
its layout as parts.

A Zazasun model is a stack of layers given one by one in config.json's ``layers`` list: every entry
names its mixer (``type``: ``attention``, ``wkv`` or ``hgrn2``), the mixer's sizes and constants
(``mixer``) and its feed-forward (``mlp``: ``{"kind": "dense", "ff": n}`` or null).  The model adds a
learned position vector to the token embedding, keeps its residual stream in 32-bit floats, uses one
scalar-gain RMS norm per layer that mixer and feed-forward both read, blends the mixer's input with
the previous token's (a per-channel token shift carried across steps), and ends with a scalar-gain
norm and an untied head.  No size or constant of a model stands in code: all of them come from
config.json, tensor shapes are derived from them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("attention", "wkv", "hgrn2")


def _positive(value, what: str) -> int:
    number = int(value)
    if number <= 0 or number != value:
        raise ValueError(f"Zazasun config: {what} must be a positive integer, got {value!r}")
    return number


@dataclass(frozen=True)
class ZazasunLayer:
    """One entry of ``layers``: the mixer's kind with its arguments as a sorted tuple of items
    (hashable), and the feed-forward's inner width (0: none)."""

    type: str
    mixer: tuple
    ff: int = 0

    @property
    def mixer_args(self) -> dict[str, Any]:
        return dict(self.mixer)


def _layer_from_dict(index: int, data: Mapping[str, Any]) -> ZazasunLayer:
    kind = data.get("type")
    if kind not in MIXER_TYPES:
        raise ValueError(f"Zazasun config: layer {index} has type {kind!r}; known: {', '.join(MIXER_TYPES)}")
    mixer = data.get("mixer")
    if not isinstance(mixer, Mapping):
        raise KeyError(f"Zazasun config: layer {index} lacks the object 'mixer'")
    where = f"layer {index} mixer"
    args: dict[str, Any] = {"heads": _positive(mixer.get("heads"), f"{where}.heads"),
                            "dim": _positive(mixer.get("dim"), f"{where}.dim")}
    if kind in ("attention", "hgrn2"):
        args["vdim"] = _positive(mixer.get("vdim"), f"{where}.vdim")
    if kind == "attention":
        args["kv_heads"] = _positive(mixer.get("kv_heads", args["heads"]), f"{where}.kv_heads")
        if args["heads"] % args["kv_heads"]:
            raise ValueError(f"Zazasun config: {where}.heads must be a multiple of kv_heads")
        for name in ("diff", "scale"):
            if name not in mixer:
                raise KeyError(f"Zazasun config: {where} lacks {name!r}")
            args[name] = float(mixer[name])
        mask = mixer.get("mask")
        if mask is None:
            args["window"], args["keep_first"] = 0, 0          # every earlier key is visible
        else:
            args["window"] = _positive(mask.get("size"), f"{where}.mask.size")
            args["keep_first"] = int(mask.get("keep_first", 0))
            if args["keep_first"] < 0:
                raise ValueError(f"Zazasun config: {where}.mask.keep_first must not be negative")
    mlp = data.get("mlp")
    ff = 0
    if mlp is not None:
        if mlp.get("kind") != "dense":
            raise ValueError(f"Zazasun config: layer {index} has feed-forward kind {mlp.get('kind')!r}; known: dense")
        ff = _positive(mlp.get("ff"), f"layer {index} mlp.ff")
    return ZazasunLayer(kind, tuple(sorted(args.items())), ff)


def _layer_to_dict(layer: ZazasunLayer) -> dict[str, Any]:
    args = layer.mixer_args
    mixer: dict[str, Any] = {"heads": args["heads"], "dim": args["dim"]}
    if "vdim" in args:
        mixer["vdim"] = args["vdim"]
    if layer.type == "attention":
        mixer.update(kv_heads=args["kv_heads"], diff=args["diff"], scale=args["scale"])
        if args["window"]:
            mixer["mask"] = {"size": args["window"], "keep_first": args["keep_first"]}
    return {"type": layer.type, "mixer": mixer,
            "mlp": {"kind": "dense", "ff": layer.ff} if layer.ff else None}


@dataclass(frozen=True)
class ZazasunConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: tuple[ZazasunLayer, ...]

    architecture = "Zazasun"

    def __post_init__(self) -> None:
        for name in ("vocab", "width", "max_positions"):
            if getattr(self, name) <= 0:
                raise ValueError(f"Zazasun config: {name} must be > 0")
        if self.norm_eps <= 0:
            raise ValueError("Zazasun config: norm.eps must be > 0")
        if not self.layers:
            raise ValueError("Zazasun config: 'layers' must list at least one layer")

    # the names the command line and the generic tools read
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ZazasunConfig":
        missing = [name for name in ("vocab", "width", "max_positions", "norm", "layers") if name not in data]
        if missing:
            raise KeyError(f"config.json lacks these keys: {', '.join(missing)}")
        norm = data["norm"]
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise KeyError("config.json: 'norm' must be an object with the key 'eps'")
        layers = data["layers"]
        if not isinstance(layers, (list, tuple)):
            raise ValueError("config.json: 'layers' must be a list")
        return cls(vocab=int(data["vocab"]), width=int(data["width"]), max_positions=int(data["max_positions"]),
                   norm_eps=float(norm["eps"]),
                   layers=tuple(_layer_from_dict(i, layer) for i, layer in enumerate(layers)))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "layers": [_layer_to_dict(layer) for layer in self.layers]}


def zazasun_model_spec(config: ZazasunConfig) -> ModelSpec:
    """Zazasun as parts.  Tensor names: ``embed``, ``pos``, ``l<i>.norm1`` (a single number),
    ``l<i>.shift``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``."""
    width, eps = config.width, config.norm_eps
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        args = {**layer.mixer_args, "hidden_size": width, "eps": eps}
        kind = {"attention": "differential_attention", "wkv": "wkv", "hgrn2": "hgrn2"}[layer.type]
        feed_forward = None
        if layer.ff:
            feed_forward = PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": layer.ff,
                                                  "activation": "gelu_tanh",
                                                  "names": ("gate", "up", "down")}, prefix + "mlp.")
        layers.append(LayerSpec(
            block="parallel_shifted",
            mixer=PartSpec(kind, args, prefix + "mix."),
            feed_forward=feed_forward,
            mixer_norm=PartSpec("scalar_rms_norm", {"eps": eps, "tensor": prefix + "norm1"}),
            feed_forward_norm=None,
            extra_parts=(("shift", "shift", PartSpec("token_shift", {"hidden_size": width,
                                                                     "tensor": prefix + "shift"})),),
        ))
    return ModelSpec(
        architecture=config.architecture, vocab_size=config.vocab, hidden_size=width,
        max_positions=config.max_positions,
        embedding=PartSpec("token_position_embedding",
                           {"vocab_size": config.vocab, "hidden_size": width, "max_positions": config.max_positions,
                            "token_tensor": "embed", "position_tensor": "pos"}),
        layers=tuple(layers),
        run_order=tuple(RunStep(layer=i, cache=i) for i in range(len(layers))),
        final_norm=PartSpec("scalar_rms_norm", {"eps": eps, "tensor": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "head"}),
    )
