"""Marutar as data: its configuration turned into a ModelSpec.

A decoder whose layers are listed one by one.  The embedding adds a learned vector per position and is
normalised.  A layer is a pre-norm residual block around a mixer, a minGRU recurrence (state per request)
or attention with a distance bias, heads mixed before the softmax, a sliding window and an output gate
(paged keys and values), followed or not by a dense feed-forward with the square of relu.  A final norm and
an untied head.  Tensor names carry no ``.weight``: ``l<i>.norm1``, ``l<i>.mix.q``, ``l<i>.mlp.up`` and so on.
This file only names parts and sizes; every formula lives in the parts.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from .marutar_config import MarutarConfig

SLOPE_EXPONENT = 8.0   # head h of H is biased by slope 2^(-8 (h + 1) / H) per token of distance


def distance_slopes(heads: int) -> tuple:
    return tuple(2.0 ** (-SLOPE_EXPONENT * (head + 1) / heads) for head in range(heads))


def build_marutar_spec(config: MarutarConfig) -> ModelSpec:
    width = config.width
    norm = PartSpec("rmsnorm", {"size": width, "eps": config.norm_eps, "suffix": ""})
    layers = []
    for index, layer in enumerate(config.layers):
        sizes = layer["mixer"]
        if layer["type"] == "mingru":
            mixer = PartSpec("mingru", {"hidden_size": width, "width": sizes["width"]})
        else:
            mixer = PartSpec("mixed_heads_attention", {
                "hidden_size": width, "num_heads": sizes["heads"], "num_kv_heads": sizes["kv_heads"], "key_dim": sizes["dim"], "value_dim": sizes["vdim"],
                "window": (sizes.get("mask") or {}).get("size", 0), "scale": sizes["scale"], "distance_slopes": distance_slopes(sizes["heads"]),
                "mix_heads": True, "output_gate": True,
            })
        mlp = layer["mlp"]
        feed_forward = None if mlp is None else PartSpec("dense_mlp", {"hidden_size": width, "intermediate_size": mlp["ff"], "activation": "relu_squared"})
        layers.append(LayerSpec(f"l{index}", PartSpec("pre_norm_residual", {
            "mixer_norm": norm, "mixer_norm_name": "norm1", "mixer": mixer, "mixer_name": "mix",
            "feed_forward_norm": norm, "feed_forward_norm_name": "norm2", "feed_forward": feed_forward, "feed_forward_name": "mlp",
        })))
    spec = ModelSpec(
        architecture="Marutar", hidden_size=width, vocab_size=config.vocab, max_positions=config.max_positions,
        embedding=PartSpec("positioned_embedding", {
            "vocab_size": config.vocab, "hidden_size": width, "tensor": "embed",
            "positions": {"tensor": "pos", "max_positions": config.max_positions}, "norm": {"tensor": "embed.norm", "eps": config.norm_eps},
        }),
        layers=tuple(layers), order=tuple(OrderEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": config.norm_eps, "suffix": "", "name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "head", "tied_to": None}),
    )
    spec.validate()
    return spec


MARUTAR = Architecture(name="Marutar", config_class=MarutarConfig, build_spec=build_marutar_spec)
register_architecture(MARUTAR, replace=True)
