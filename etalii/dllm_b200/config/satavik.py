"""The typed configuration of the Satavik design, read from config.json's own keys.

A Satavik config.json names the design under `architecture` and gives `vocab`, `width`, `embedding.scale`, `norm.eps`
and `layers`: a list whose entries have `type` ("attention"), the mixer's sizes and constants under `mixer` (`heads`,
`kv_heads`, `dim`, `vdim`, `scale`, `softcap`, `diff`, `mask.size`, `rot.base`, `rot.dims`, and optionally `kv_from`:
the layer whose keys and values this one reads instead of projecting its own) and the feed-forward under `mlp` (kind
"moe": `expert.ff`, `expert.limit`, `router.experts`, `router.top`, optionally `shared.ff` and `shared.limit`; or null
for a layer without one). Nothing here is a size of a particular model."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping

from .registry import ConfigError

MIXER_TYPES = ("attention",)
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


def _check_mixer(where: str, mixer: Any) -> None:
    _need(where, mixer, ("heads", "kv_heads", "dim", "vdim", "scale", "diff"))
    _positive(where, mixer, ("heads", "kv_heads", "dim", "vdim"))
    if mixer["heads"] % mixer["kv_heads"]:
        raise ConfigError(f"{where}: {mixer['heads']} heads are not a multiple of {mixer['kv_heads']} kv_heads")
    if not float(mixer["scale"]) > 0:
        raise ConfigError(f"{where}.scale must be positive")
    if mixer.get("softcap") is not None and not float(mixer["softcap"]) > 0:
        raise ConfigError(f"{where}.softcap must be positive")
    rot = mixer.get("rot")
    if rot is not None:
        _need(f"{where}.rot", rot, ("base", "dims"))
        dims = rot["dims"]
        if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > mixer["dim"]:
            raise ConfigError(f"{where}.rot.dims must be even and at most dim, not {dims!r}")
        if dims and not float(rot["base"]) > 0:
            raise ConfigError(f"{where}.rot.base must be positive")
    mask = mixer.get("mask")
    if mask is not None:
        _need(f"{where}.mask", mask, ("size",))
        _positive(f"{where}.mask", mask, ("size",))


def _check_mlp(where: str, mlp: Any) -> None:
    _need(where, mlp, ("kind", "expert", "router"))
    if mlp["kind"] != "moe":
        raise ConfigError(f"{where}.kind {mlp['kind']!r} is not supported (supported: moe)")
    _need(f"{where}.expert", mlp["expert"], ("ff", "limit"))
    _positive(f"{where}.expert", mlp["expert"], ("ff",))
    _need(f"{where}.router", mlp["router"], ("experts", "top"))
    _positive(f"{where}.router", mlp["router"], ("experts", "top"))
    if mlp["router"]["top"] > mlp["router"]["experts"]:
        raise ConfigError(f"{where}.router: top {mlp['router']['top']} of {mlp['router']['experts']} experts")
    if not float(mlp["expert"]["limit"]) > 0:
        raise ConfigError(f"{where}.expert.limit must be positive")
    shared = mlp.get("shared")
    if shared is not None:
        _need(f"{where}.shared", shared, ("ff", "limit"))
        _positive(f"{where}.shared", shared, ("ff",))
        if not float(shared["limit"]) > 0:
            raise ConfigError(f"{where}.shared.limit must be positive")


def _check_layers(layers) -> None:
    for index, layer in enumerate(layers):
        where = f"layers[{index}]"
        _need(where, layer, ("type", "mixer"))
        if layer["type"] not in MIXER_TYPES:
            raise ConfigError(f"{where}.type {layer['type']!r} is not supported (supported: {', '.join(MIXER_TYPES)})")
        _check_mixer(f"{where}.mixer", layer["mixer"])
        if layer.get("mlp") is not None:
            _check_mlp(f"{where}.mlp", layer["mlp"])
    for index, layer in enumerate(layers):
        source = layer["mixer"].get("kv_from")
        if source is None:
            continue
        where = f"layers[{index}].mixer.kv_from"
        if not isinstance(source, int) or isinstance(source, bool) or not 0 <= source < index:
            raise ConfigError(f"{where} must name an earlier layer, not {source!r}")
        other, own = layers[source]["mixer"], layer["mixer"]
        if other.get("kv_from") is not None:
            raise ConfigError(f"{where}: layer {source} has no keys and values of its own")
        for key in ("kv_heads", "dim", "vdim", "rot"):
            if other.get(key) != own.get(key):
                raise ConfigError(f"{where}: layer {source}'s {key} ({other.get(key)!r}) differs from this layer's "
                                  f"({own.get(key)!r})")


@dataclass(frozen=True)
class SatavikConfig:
    model_type = "Satavik"

    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple = field(default_factory=tuple)
    """The layer entries as config.json gives them (checked)."""
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
        _check_layers(self.layers)

    @classmethod
    def from_hf(cls, config: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "SatavikConfig":
        if config.get("architecture") != "Satavik":
            raise ConfigError(f"architecture {config.get('architecture')!r} is not 'Satavik'")
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
            max_position=int(config.get("max_position", DEFAULT_MAX_POSITION)),
            eos_token_ids=tuple(eos),
        )

    def to_hf(self) -> dict:
        """The config.json that reads back as this configuration."""
        out: dict[str, Any] = {
            "architecture": "Satavik", "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
