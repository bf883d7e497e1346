"""Typed configuration of Zirutar, read from its own config.json keys.

``layers`` lists the layers one by one: ``{"type": "attention" | "latent_attention" | "channel_delta", "mixer": {...sizes...},
"mlp": null | {"kind": "dense", "ff": n, "limit": x}}``.  Beside it: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``logit_scale``, optionally ``loop`` = {start, stop, times} (layers start .. stop - 1 run ``times`` times in a row) and
``token_side`` = {dim} (every layer adds a gated slice of a second token table).  Every size and constant is free; what the
design does not have is refused.  The low ranks of the delta rule's decay and gate are read from the tensors' shapes.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..config.model_config import as_float, as_int
from ..errors import ConfigError

MIXERS = ("attention", "latent_attention", "channel_delta")


def _heads(where: str, mixer: dict) -> tuple[int, int]:
    heads = as_int(f"{where}.heads", mixer.get("heads"))
    kv_heads = as_int(f"{where}.kv_heads", mixer.get("kv_heads", heads))
    if heads % kv_heads != 0:
        raise ConfigError(f"{where}: heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return heads, kv_heads


def _mixer_sizes(index: int, kind: str, mixer) -> dict:
    where = f"layers[{index}].mixer"
    if not isinstance(mixer, dict):
        raise ConfigError(f"{where} must be an object")
    dim = as_int(f"{where}.dim", mixer.get("dim"))
    vdim = as_int(f"{where}.vdim", mixer.get("vdim", dim))
    if kind == "attention":
        heads, kv_heads = _heads(where, mixer)
        if vdim != dim:
            raise ConfigError(f"{where}: the values are the keys, so vdim ({vdim}) must equal dim ({dim})")
        sizes = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": as_float(f"{where}.scale", mixer.get("scale", dim ** -0.5))}
        mask = mixer.get("mask")
        if mask is not None:
            if not isinstance(mask, dict):
                raise ConfigError(f"{where}.mask must be an object or null")
            sizes["mask"] = {"size": as_int(f"{where}.mask.size", mask.get("size")), "keep_first": as_int(f"{where}.mask.keep_first", mask.get("keep_first", 0), minimum=0)}
        return sizes
    if kind == "latent_attention":
        heads = as_int(f"{where}.heads", mixer.get("heads"))
        rot_dim = as_int(f"{where}.rot_dim", mixer.get("rot_dim"))
        rot = mixer.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"{where}.rot must be an object with base and dims")
        dims = as_int(f"{where}.rot.dims", rot.get("dims", rot_dim))
        if dims > rot_dim or dims % 2 or rot_dim % 2:
            raise ConfigError(f"{where}: rot.dims ({dims}) must be even and at most rot_dim ({rot_dim}), which must be even")
        return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": as_int(f"{where}.kv_rank", mixer.get("kv_rank")),
                "scale": as_float(f"{where}.scale", mixer.get("scale", (dim + rot_dim) ** -0.5)), "rot": {"base": as_float(f"{where}.rot.base", rot.get("base")), "dims": dims}}
    heads, kv_heads = _heads(where, mixer)
    sizes = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": as_int(f"{where}.conv", mixer.get("conv"))}
    for key in ("decay_rank", "gate_rank"):   # not part of a checkpoint's config.json: filled in from the tensors' shapes when a folder is read
        if key in mixer:
            sizes[key] = as_int(f"{where}.{key}", mixer[key])
    return sizes


@dataclass(frozen=True)
class ZirutarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple                # one dictionary per layer: {"type", "mixer", "mlp"}, checked
    loop: dict | None = None     # {"start", "stop", "times"}
    token_side: dict | None = None   # {"dim"}
    architecture: str = "Zirutar"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, data: dict) -> "ZirutarConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        missing = [key for key in ("vocab", "width", "norm", "layers") if key not in data]
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
                mlp = {"kind": "dense", "ff": as_int(f"layers[{index}].mlp.ff", mlp.get("ff")), "limit": as_float(f"layers[{index}].mlp.limit", mlp.get("limit"))}
            layers.append({"type": kind, "mixer": _mixer_sizes(index, kind, layer.get("mixer")), "mlp": mlp})
        loop = data.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: loop must be an object or absent")
            loop = {"start": as_int("loop.start", loop.get("start"), minimum=0), "stop": as_int("loop.stop", loop.get("stop")), "times": as_int("loop.times", loop.get("times"))}
            if not loop["start"] < loop["stop"] <= len(layers):
                raise ConfigError(f"loop: start ({loop['start']}) < stop ({loop['stop']}) <= layers ({len(layers)}) does not hold")
        side = data.get("token_side")
        if side is not None:
            if not isinstance(side, dict):
                raise ConfigError("config.json: token_side must be an object or absent")
            side = {"dim": as_int("token_side.dim", side.get("dim"))}
        embedding = data.get("embedding") or {}
        return cls(vocab=as_int("vocab", data["vocab"]), width=as_int("width", data["width"]), norm_eps=as_float("norm.eps", data["norm"]["eps"]),
                   embedding_scale=as_float("embedding.scale", embedding.get("scale", 1.0)), logit_scale=as_float("logit_scale", data.get("logit_scale", 1.0)),
                   layers=tuple(layers), loop=loop, token_side=side, architecture=str(data.get("architecture", "Zirutar")))

    def with_tensor_shapes(self, shapes: dict) -> "ZirutarConfig":
        """The sizes a checkpoint's config.json leaves to its tensors, read from ``shapes`` (name -> shape): the delta rule's low ranks."""
        layers = []
        for index, layer in enumerate(self.layers):
            mixer = dict(layer["mixer"])
            if layer["type"] == "channel_delta":
                for key, tensor in (("decay_rank", f"l{index}.mix.a1"), ("gate_rank", f"l{index}.mix.g1")):
                    if key not in mixer and tensor in shapes:
                        mixer[key] = int(shapes[tensor][0])
            layers.append({**layer, "mixer": mixer})
        return ZirutarConfig(self.vocab, self.width, self.norm_eps, self.embedding_scale, self.logit_scale, tuple(layers), self.loop, self.token_side, self.architecture)

    def to_dict(self) -> dict:
        data = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "layers": [dict(layer) for layer in self.layers]}
        if self.loop is not None:
            data["loop"] = dict(self.loop)
        if self.token_side is not None:
            data["token_side"] = dict(self.token_side)
        return data
