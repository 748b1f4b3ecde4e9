"""The typed configuration of the Tisalorn design, read from config.json's own keys.

A Tisalorn config.json names the design under `architecture` and gives: `vocab`, `width`, `embedding.scale`,
`norm.eps`, `layers` (a list; every entry has `type`, one of parallel / lightning / delta, the mixer's sizes under
`mixer`, and the feed-forward under `mlp`, or null for none) and optionally `loop` (`start`, `stop`, `times`: the
layers start .. stop - 1 run `times` times in a row). Nothing here is a size of a particular model."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .registry import ConfigError

MIXER_TYPES = ("parallel", "lightning", "delta")
DEFAULT_MAX_POSITION = 32768
"""The design has no longest sequence; this bounds the rotary table and the cache unless `max_position` is given."""


def _need(where: str, mapping: Any, keys) -> None:
    if not isinstance(mapping, Mapping):
        raise ConfigError(f"{where} must be an object")
    missing = [k for k in keys if k not in mapping]
    if missing:
        raise ConfigError(f"{where} has no {', '.join(missing)}")


def _positive(where: str, mapping: Mapping, keys) -> None:
    for key in keys:
        if not isinstance(mapping[key], int) or isinstance(mapping[key], bool) or mapping[key] <= 0:
            raise ConfigError(f"{where}.{key} must be a positive integer, not {mapping[key]!r}")


def _decays(where: str, mixer: Mapping) -> None:
    decay = mixer["decay"]
    if not isinstance(decay, (list, tuple)) or len(decay) != mixer["heads"]:
        raise ConfigError(f"{where}.decay must list one decay per head ({mixer['heads']})")
    if any(not 0.0 <= float(d) <= 1.0 for d in decay):
        raise ConfigError(f"{where}.decay: every decay lies in [0, 1]")


def _check_layer(index: int, layer: Any) -> None:
    where = f"layers[{index}]"
    _need(where, layer, ("type", "mixer"))
    kind, mixer = layer["type"], layer["mixer"]
    if kind not in MIXER_TYPES:
        raise ConfigError(f"{where}.type {kind!r} is not supported (supported: {', '.join(MIXER_TYPES)})")
    if kind == "parallel":
        _need(f"{where}.mixer", mixer, ("left", "right"))
        left, right = mixer["left"], mixer["right"]
        _need(f"{where}.mixer.left", left, ("heads", "kv_heads", "dim", "vdim", "rot", "scale"))
        _positive(f"{where}.mixer.left", left, ("heads", "kv_heads", "dim", "vdim"))
        _need(f"{where}.mixer.left.rot", left["rot"], ("base", "dims"))
        if left["heads"] % left["kv_heads"]:
            raise ConfigError(f"{where}.mixer.left: {left['heads']} heads are not a multiple of {left['kv_heads']} "
                              f"kv_heads")
        if left["vdim"] != left["dim"]:
            raise ConfigError(f"{where}.mixer.left: the values are the keys, so vdim ({left['vdim']}) must equal dim "
                              f"({left['dim']})")
        dims = left["rot"]["dims"]
        if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > left["dim"]:
            raise ConfigError(f"{where}.mixer.left.rot.dims must be even and at most dim, not {dims!r}")
        if dims and not float(left["rot"]["base"]) > 0:
            raise ConfigError(f"{where}.mixer.left.rot.base must be positive")
        _need(f"{where}.mixer.right", right, ("heads", "dim", "vdim", "decay"))
        _positive(f"{where}.mixer.right", right, ("heads", "dim", "vdim"))
        _decays(f"{where}.mixer.right", right)
    elif kind == "lightning":
        _need(f"{where}.mixer", mixer, ("heads", "dim", "vdim", "decay"))
        _positive(f"{where}.mixer", mixer, ("heads", "dim", "vdim"))
        _decays(f"{where}.mixer", mixer)
    else:
        _need(f"{where}.mixer", mixer, ("heads", "kv_heads", "dim", "vdim", "conv"))
        _positive(f"{where}.mixer", mixer, ("heads", "kv_heads", "dim", "vdim", "conv"))
        if mixer["heads"] % mixer["kv_heads"]:
            raise ConfigError(f"{where}.mixer: {mixer['heads']} heads are not a multiple of {mixer['kv_heads']} "
                              f"kv_heads")
    mlp = layer.get("mlp")
    if mlp is not None:
        _need(f"{where}.mlp", mlp, ("kind", "ff", "limit"))
        if mlp["kind"] != "dense":
            raise ConfigError(f"{where}.mlp.kind {mlp['kind']!r} is not supported (supported: dense)")
        _positive(f"{where}.mlp", mlp, ("ff",))
        if not float(mlp["limit"]) > 0:
            raise ConfigError(f"{where}.mlp.limit must be positive")


@dataclass(frozen=True)
class TisalornConfig:
    model_type = "Tisalorn"

    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple = field(default_factory=tuple)
    """The layer entries as config.json gives them (checked)."""
    loop: Mapping | None = None
    max_position: int = DEFAULT_MAX_POSITION
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)

    def __post_init__(self) -> None:
        for name in ("vocab", "width", "max_position"):
            if int(getattr(self, name)) <= 0:
                raise ConfigError(f"{name} must be positive, not {getattr(self, name)}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, not {self.norm_eps}")
        if not self.layers:
            raise ConfigError("layers is empty")
        for index, layer in enumerate(self.layers):
            _check_layer(index, layer)
        if self.loop is not None:
            _need("loop", self.loop, ("start", "stop", "times"))
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start < stop <= len(self.layers)):
                raise ConfigError(f"loop: start {start!r} and stop {stop!r} must bound a stretch of the "
                                  f"{len(self.layers)} layers")
            if not isinstance(times, int) or times < 1:
                raise ConfigError(f"loop.times must be a positive integer, not {times!r}")

    @classmethod
    def from_hf(cls, config: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "TisalornConfig":
        if config.get("architecture") != "Tisalorn":
            raise ConfigError(f"architecture {config.get('architecture')!r} is not 'Tisalorn'")
        _need("config.json", config, ("vocab", "width", "embedding", "norm", "layers"))
        _need("embedding", config["embedding"], ("scale",))
        _need("norm", config["norm"], ("eps",))
        if not isinstance(config["layers"], (list, tuple)):
            raise ConfigError("layers must be a list")
        eos = config.get("eos_token_id")
        eos = [] if eos is None else ([int(t) for t in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        return cls(
            vocab=int(config["vocab"]), width=int(config["width"]),
            embedding_scale=float(config["embedding"]["scale"]), norm_eps=float(config["norm"]["eps"]),
            layers=tuple(copy.deepcopy(layer) for layer in config["layers"]),
            loop=copy.deepcopy(config["loop"]) if config.get("loop") is not None else None,
            max_position=int(config.get("max_position", DEFAULT_MAX_POSITION)),
            eos_token_ids=tuple(eos),
        )

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        out: dict[str, Any] = {
            "architecture": "Tisalorn", "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
        if self.loop is not None:
            out["loop"] = copy.deepcopy(dict(self.loop))
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
