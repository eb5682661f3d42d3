"""Typed configuration of the ``Rozesun`` architecture, read from the keys of its config.json, and
its layout as parts.

A Rozesun model is a stack of layers given one by one in config.json's ``layers`` list: every entry
names its mixer (``type``: ``latent_attention`` or ``latent_attention_2``), the mixer's sizes and
constants (``mixer``) and its feed-forward (``mlp``: ``{"kind": "dense", "ff": n, "limit": c}`` or
null).  ``loop`` = {start, stop, times} makes the layers start .. stop-1 run ``times`` times in a row
with the same weights (each pass with a cache of its own), a learned vector (row t of ``loop.step``)
being added to the stream before pass t.  The residual stream is 32-bit; every sublayer sits between
two layer norms (weight and bias); the head is the embedding table, its logits multiplied by
``logit_scale``.  Both mixers are attention over low-rank latents; they differ in what the design
fixes for each kind:

    latent_attention     rotate-half pairs, all earlier keys visible, plain softmax, a gate per channel
    latent_attention_2   interleaved pairs, a sliding window (``mask.size``), a per-head sink in the
                         softmax, a gate per head

No size or constant of a model stands in code: all of them come from config.json, tensor shapes are
derived from them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

# what each mixer kind fixes: pair layout of the rotation, windowed or not, sink, gate granularity
MIXER_KINDS = {
    "latent_attention": {"rope_layout": "half", "windowed": False, "sink": False, "gate": "channel"},
    "latent_attention_2": {"rope_layout": "interleaved", "windowed": True, "sink": True, "gate": "head"},
}
GATE_SLOPE = 1.702          # the feed-forward's g * sigmoid(1.702 g)
UNLIMITED_POSITIONS = 1 << 30     # the design sets no position limit


def _positive(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) <= 0:
        raise ValueError(f"Rozesun config: {what} must be a positive integer, got {value!r}")
    return int(value)


@dataclass(frozen=True)
class RozesunLayer:
    """One entry of ``layers``: the mixer's kind with its arguments as a sorted tuple of items
    (hashable), the feed-forward's inner width (0: none) and clamp."""

    type: str
    mixer: tuple
    ff: int = 0
    limit: float = 0.0

    @property
    def mixer_args(self) -> dict[str, Any]:
        return dict(self.mixer)


def _layer_from_dict(index: int, data: Mapping[str, Any]) -> RozesunLayer:
    kind = data.get("type")
    if kind not in MIXER_KINDS:
        raise ValueError(f"Rozesun config: layer {index} has type {kind!r}; known: {', '.join(MIXER_KINDS)}")
    mixer = data.get("mixer")
    if not isinstance(mixer, Mapping):
        raise KeyError(f"Rozesun config: layer {index} lacks the object 'mixer'")
    where = f"layer {index} mixer"
    args: dict[str, Any] = {name: _positive(mixer.get(name), f"{where}.{name}")
                            for name in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
    if "scale" not in mixer:
        raise KeyError(f"Rozesun config: {where} lacks 'scale'")
    args["scale"] = float(mixer["scale"])
    rot = mixer.get("rot")
    if not isinstance(rot, Mapping) or "base" not in rot:
        raise KeyError(f"Rozesun config: {where} lacks the object 'rot' with 'base'")
    args["rope_base"] = float(rot["base"])
    args["rope_dims"] = _positive(rot.get("dims", args["rot_dim"]), f"{where}.rot.dims")
    if args["rope_dims"] % 2 or args["rope_dims"] > args["rot_dim"]:
        raise ValueError(f"Rozesun config: {where}.rot.dims must be even and at most rot_dim")
    args["window"] = 0
    if MIXER_KINDS[kind]["windowed"]:
        mask = mixer.get("mask")
        if not isinstance(mask, Mapping):
            raise KeyError(f"Rozesun config: {where} lacks the object 'mask'")
        args["window"] = _positive(mask.get("size"), f"{where}.mask.size")
    mlp = data.get("mlp")
    ff, limit = 0, 0.0
    if mlp is not None:
        if mlp.get("kind") != "dense":
            raise ValueError(f"Rozesun config: layer {index} has feed-forward kind {mlp.get('kind')!r}; known: dense")
        ff = _positive(mlp.get("ff"), f"layer {index} mlp.ff")
        if "limit" not in mlp or not float(mlp["limit"]) > 0:
            raise ValueError(f"Rozesun config: layer {index} mlp.limit must be a positive number")
        limit = float(mlp["limit"])
    return RozesunLayer(kind, tuple(sorted(args.items())), ff, limit)


def _layer_to_dict(layer: RozesunLayer) -> dict[str, Any]:
    args = layer.mixer_args
    mixer: dict[str, Any] = {name: args[name] for name in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
    mixer["scale"] = args["scale"]
    mixer["rot"] = {"base": args["rope_base"], "dims": args["rope_dims"]}
    if args["window"]:
        mixer["mask"] = {"size": args["window"]}
    return {"type": layer.type, "mixer": mixer,
            "mlp": {"kind": "dense", "ff": layer.ff, "limit": layer.limit} if layer.ff else None}


@dataclass(frozen=True)
class RozesunConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: tuple[RozesunLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0        # start == stop: no layer runs more than once
    loop_times: int = 1
    loop_given: bool = False  # config.json has a 'loop' object (then the checkpoint holds its vectors)
    max_positions: int = UNLIMITED_POSITIONS

    architecture = "Rozesun"

    def __post_init__(self) -> None:
        for name in ("vocab", "width", "max_positions"):
            if getattr(self, name) <= 0:
                raise ValueError(f"Rozesun config: {name} must be > 0")
        if self.norm_eps <= 0:
            raise ValueError("Rozesun config: norm.eps must be > 0")
        if not self.layers:
            raise ValueError("Rozesun config: 'layers' must list at least one layer")
        if not 0 <= self.loop_start <= self.loop_stop <= len(self.layers) or self.loop_times < 0:
            raise ValueError("Rozesun config: 'loop' needs 0 <= start <= stop <= number of layers and times >= 0")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def loops(self) -> bool:
        return self.loop_stop > self.loop_start

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "RozesunConfig":
        missing = [name for name in ("vocab", "width", "norm", "layers", "logit_scale") if name not in data]
        if missing:
            raise KeyError(f"config.json lacks these keys: {', '.join(missing)}")
        norm = data["norm"]
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise KeyError("config.json: 'norm' must be an object with the key 'eps'")
        layers = data["layers"]
        if not isinstance(layers, (list, tuple)):
            raise ValueError("config.json: 'layers' must be a list")
        loop = data.get("loop")
        start = stop = 0
        times = 1
        if loop is not None:
            if not isinstance(loop, Mapping) or any(name not in loop for name in ("start", "stop", "times")):
                raise KeyError("config.json: 'loop' must be an object with 'start', 'stop' and 'times'")
            start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        return cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(norm["eps"]),
                   logit_scale=float(data["logit_scale"]),
                   layers=tuple(_layer_from_dict(i, layer) for i, layer in enumerate(layers)),
                   loop_start=start, loop_stop=stop, loop_times=times, loop_given=loop is not None,
                   max_positions=int(data.get("max_positions", UNLIMITED_POSITIONS)))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
               "layers": [_layer_to_dict(layer) for layer in self.layers]}
        if self.loop_given or self.loops:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.max_positions != UNLIMITED_POSITIONS:
            out["max_positions"] = self.max_positions
        return out


def rozesun_run_order(config: RozesunConfig) -> tuple[RunStep, ...]:
    """Layers before the loop once, the looped run ``times`` times (each pass's first layer asks for
    the pass's vector), the rest once; every run step has a cache entry of its own."""
    order: list[tuple[int, int | None]] = [(i, None) for i in range(config.loop_start)]
    if config.loops:
        for number in range(config.loop_times):
            order += [(i, number if i == config.loop_start else None)
                      for i in range(config.loop_start, config.loop_stop)]
    order += [(i, None) for i in range(config.loop_stop, len(config.layers))]
    return tuple(RunStep(layer=layer, cache=entry, offset_row=row) for entry, (layer, row) in enumerate(order))


def rozesun_model_spec(config: RozesunConfig) -> ModelSpec:
    """Rozesun as parts.  Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1|norm2|norm1b|norm2b`` (+ ``.b``),
    ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm`` (+ ``.b``)."""
    width, eps = config.width, config.norm_eps
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        kind = MIXER_KINDS[layer.type]
        args = {**layer.mixer_args, "hidden_size": width, "eps": eps, "rope_layout": kind["rope_layout"],
                "sink": kind["sink"], "gate": kind["gate"]}

        def norm(name):
            return PartSpec("layer_norm", {"size": width, "eps": eps, "tensor": prefix + name})

        feed_forward = feed_forward_norm = None
        extras = [("mixer_post_norm", "norm", norm("norm1b"))]
        if layer.ff:
            feed_forward = PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": layer.ff,
                                                  "activation": "clamped_swish", "limit": layer.limit,
                                                  "slope": GATE_SLOPE, "names": ("gate", "up", "down")}, prefix + "mlp.")
            feed_forward_norm = norm("norm2")
            extras.append(("feed_forward_post_norm", "norm", norm("norm2b")))
        layers.append(LayerSpec(block="sandwich_norm", mixer=PartSpec("latent_attention", args, prefix + "mix."),
                                feed_forward=feed_forward, mixer_norm=norm("norm1"),
                                feed_forward_norm=feed_forward_norm, extra_parts=tuple(extras)))
    offsets = None
    if config.loops or config.loop_given:
        offsets = PartSpec("learned_offsets", {"rows": config.loop_times, "size": width, "tensor": "loop.step"})
    return ModelSpec(
        architecture=config.architecture, vocab_size=config.vocab, hidden_size=width,
        max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "embed",
                                               "rows": "float32"}),
        layers=tuple(layers), run_order=rozesun_run_order(config),
        final_norm=PartSpec("layer_norm", {"size": width, "eps": eps, "tensor": "final.norm"}),
        head=PartSpec("tied_head", {"vocab_size": config.vocab, "hidden_size": width, "scale": config.logit_scale,
                                    "own_copy": False}),
        offsets=offsets,
    )
