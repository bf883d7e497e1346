"""Typed configuration of Marutar, read from its own config.json keys.

A Marutar checkpoint lists its layers one by one: ``layers`` is a list of
``{"type": "mingru" | "attention", "mixer": {...sizes...}, "mlp": null | {"kind": "dense", "ff": n}}``;
beside it stand ``vocab``, ``width``, ``max_positions`` (rows of the table of position vectors) and
``norm.eps``.  Every size and constant is free; what the design does not have is refused.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config.model_config import as_float, as_int
from ..errors import ConfigError

MIXERS = ("mingru", "attention")


def _mixer_sizes(index: int, kind: str, mixer) -> dict:
    if not isinstance(mixer, dict):
        raise ConfigError(f"layers[{index}].mixer must be an object")
    where = f"layers[{index}].mixer"
    if kind == "mingru":
        return {"width": as_int(f"{where}.width", mixer.get("width"))}
    heads, kv_heads = as_int(f"{where}.heads", mixer.get("heads")), as_int(f"{where}.kv_heads", mixer.get("kv_heads", mixer.get("heads")))
    if heads % kv_heads != 0:
        raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    dim = as_int(f"{where}.dim", mixer.get("dim"))
    sizes = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": as_int(f"{where}.vdim", mixer.get("vdim", dim)),
             "scale": as_float(f"{where}.scale", mixer.get("scale", dim ** -0.5))}
    mask = mixer.get("mask")
    if mask is not None:
        if not isinstance(mask, dict):
            raise ConfigError(f"{where}.mask must be an object or null")
        sizes["mask"] = {"size": as_int(f"{where}.mask.size", mask.get("size"))}
    return sizes


@dataclass(frozen=True)
class MarutarConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: tuple          # one dictionary per layer: {"type", "mixer", "mlp"}, checked
    architecture: str = "Marutar"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: dict) -> "MarutarConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        missing = [key for key in ("vocab", "width", "max_positions", "norm", "layers") if key not in data]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        if not isinstance(data["norm"], dict) or "eps" not in data["norm"]:
            raise ConfigError("config.json: norm must be an object with eps")
        if not isinstance(data["layers"], list) or not data["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for index, layer in enumerate(data["layers"]):
            if not isinstance(layer, dict):
                raise ConfigError(f"layers[{index}] must be an object")
            kind = layer.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"layers[{index}].type must be one of {MIXERS}, got {kind!r}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"layers[{index}].mlp must be null or a dense feed-forward, got {mlp!r}")
                mlp = {"kind": "dense", "ff": as_int(f"layers[{index}].mlp.ff", mlp.get("ff"))}
            layers.append({"type": kind, "mixer": _mixer_sizes(index, kind, layer.get("mixer")), "mlp": mlp})
        return cls(vocab=as_int("vocab", data["vocab"]), width=as_int("width", data["width"]), max_positions=as_int("max_positions", data["max_positions"]),
                   norm_eps=as_float("norm.eps", data["norm"]["eps"]), layers=tuple(layers), architecture=str(data.get("architecture", "Marutar")))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
                "norm": {"eps": self.norm_eps}, "layers": [dict(layer) for layer in self.layers]}
