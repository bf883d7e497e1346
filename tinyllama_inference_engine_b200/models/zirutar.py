"""Zirutar as data: its configuration turned into a ModelSpec.

A decoder whose layers are listed one by one and of which a run may repeat with the same weights.  The embedding is a table row
times a constant.  A layer is a pre-norm residual block (RMS norms whose weights are stored around zero) around a mixer, followed
or not by a gated feed-forward with clamped halves, followed (if the model has a second token table) by a gated slice of that
table.  Three mixers: attention without positions, with normalised queries and keys, values that are the keys, a sliding window
that keeps the first tokens and one output gate per head; latent attention with a rotated key part and a sink in the softmax;
the gated delta rule with one decay per key channel.  Before every pass of the repeated run a learned vector joins the stream;
every pass has cache streams of its own.  The final norm, then the embedding table as the head, times a constant.
Tensor names: ``embed``, ``loop.step``, ``side.embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``.
This file only names parts and sizes; every formula lives in the parts.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..errors import ConfigError
from ..parts.spec import LayerSpec, ModelSpec, OrderEntry, PartSpec
from .zirutar_config import ZirutarConfig

GATE_SLOPE = 1.702        # the feed-forward's gate is g * sigmoid(1.702 g)
UP_SHIFT = 1.0            # ... times (u + 1)
UNIT_EPS = 1e-6           # inside the root of the delta rule's unit norms
MAX_POSITIONS = 1 << 17   # the design has no table of positions: this only bounds a request's block table


def _mixer(width: int, kind: str, sizes: dict, eps: float, where: str) -> PartSpec:
    if kind == "attention":
        mask = sizes.get("mask") or {}
        return PartSpec("normed_key_attention", {
            "hidden_size": width, "num_heads": sizes["heads"], "num_kv_heads": sizes["kv_heads"], "key_dim": sizes["dim"], "value_dim": sizes["vdim"],
            "scale": sizes["scale"], "eps": eps, "window": mask.get("size", 0), "keep_first": mask.get("keep_first", 0), "values": "keys", "head_gate": True,
        })
    if kind == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": sizes["heads"], "plain_dim": sizes["dim"], "rot_dim": sizes["rot_dim"], "value_dim": sizes["vdim"], "rank": sizes["kv_rank"],
            "scale": sizes["scale"], "eps": eps, "rot_dims": sizes["rot"]["dims"], "rot_base": sizes["rot"]["base"], "sink": True,
        })
    if "decay_rank" not in sizes or "gate_rank" not in sizes:
        raise ConfigError(f"{where}: the low ranks of the decay and the gate are not known (they are read from the shapes of a1 and g1)")
    return PartSpec("channel_delta_rule", {
        "hidden_size": width, "num_heads": sizes["heads"], "num_kv_heads": sizes["kv_heads"], "key_dim": sizes["dim"], "value_dim": sizes["vdim"], "taps": sizes["conv"],
        "decay_rank": sizes["decay_rank"], "gate_rank": sizes["gate_rank"], "eps": eps, "unit_eps": UNIT_EPS,
    })


def build_zirutar_spec(config: ZirutarConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = PartSpec("rmsnorm", {"size": width, "eps": eps, "suffix": "", "offset": 1.0})
    count = len(config.layers)
    layers = []
    for index, layer in enumerate(config.layers):
        mlp = layer["mlp"]
        feed_forward = None if mlp is None else PartSpec("gated_mlp", {
            "hidden_size": width, "intermediate_size": mlp["ff"], "activation": "clamped_sigmoid", "limit": mlp["limit"], "alpha": GATE_SLOPE, "shift": UP_SHIFT,
            "names": ("gate", "up", "down"),
        })
        side = None if config.token_side is None else PartSpec("gated_token_slice", {
            "hidden_size": width, "dim": config.token_side["dim"], "slice": index, "slices": count, "vocab_size": config.vocab, "table": "side.embed", "eps": eps,
        })
        layers.append(LayerSpec(f"l{index}", PartSpec("pre_norm_residual", {
            "mixer_norm": norm, "mixer_norm_name": "norm1", "mixer": _mixer(width, layer["type"], layer["mixer"], eps, f"layers[{index}].mixer"), "mixer_name": "mix",
            "feed_forward_norm": norm, "feed_forward_norm_name": "norm2", "feed_forward": feed_forward, "feed_forward_name": "mlp",
            "token_input": side, "token_input_name": "side",
        })))
    # the order of runs: every run of a layer has a cache stream of its own; a pass of the repeated run starts with its vector
    order, stream = [], 0
    loop = config.loop
    runs = [(i, None) for i in range(count)]
    if loop is not None:
        runs = [(i, None) for i in range(loop["start"])]
        for t in range(loop["times"]):
            runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
        runs += [(i, None) for i in range(loop["stop"], count)]
    for index, starts_pass in runs:
        if starts_pass is not None:
            layers.append(LayerSpec("loop", PartSpec("stream_vector", {"tensor": "loop.step", "rows": loop["times"], "size": width, "row": starts_pass})))
            order.append(OrderEntry(layer=len(layers) - 1, cache=stream))
            stream += 1
        order.append(OrderEntry(layer=index, cache=stream))
        stream += 1
    spec = ModelSpec(
        architecture="Zirutar", hidden_size=width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("positioned_embedding", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "embed", "scale": config.embedding_scale}),
        layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec("rmsnorm", {"size": width, "eps": eps, "suffix": "", "offset": 1.0, "name": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tensor": "embed", "tied_to": None, "scale": config.logit_scale}),
    )
    spec.validate()
    return spec


ZIRUTAR = Architecture(name="Zirutar", config_class=ZirutarConfig, build_spec=build_zirutar_spec)
register_architecture(ZIRUTAR, replace=True)
