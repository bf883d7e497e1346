"""How the parts of one layer are arranged."""
from __future__ import annotations

import torch

from .base import Block, CacheNeed, LayerCache, build_part, norm_then_part, part_class, register_part
from .spec import PartSpec, TensorSpec


class PreNormResidualBlock(Block):
    """x -> x + mixer(norm(x)) -> x + feed_forward(norm(x))  (src/model.cpp:112-207).

    params: ``mixer``, ``feed_forward``, ``mixer_norm``, ``feed_forward_norm``
    (PartSpecs) and the tensor-name suffix of each (``*_name``).  ``feed_forward`` may be
    None: the layer is then x -> x + mixer(norm(x)) alone.  Optional ``token_input`` (a PartSpec of that category, with
    ``token_input_name``): after the sublayers the part adds what it makes of the tokens themselves into the finished stream.
    The hidden state travels as (32-bit residual, output not yet added): each norm
    adds the pending output into the residual before normalising, which is the
    reference's separate add kernel (src/cuda/kernels.cu:208-215) fused into its
    norm (:67-84).
    """

    _SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))

    capturable = True

    @classmethod
    def _slots(cls, spec: PartSpec):
        """The block's (slot, category) pairs; a block whose ``feed_forward`` is None is its first sublayer alone."""
        slots = [pair for pair in cls._SLOTS if spec.get("feed_forward") is not None or not pair[0].startswith("feed_forward")]
        return slots + ([("token_input", "token_input")] if spec.get("token_input") is not None else [])

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        specs: list[TensorSpec] = []
        for slot, category in cls._slots(spec):
            child = spec[slot]
            specs += part_class(category, child).tensor_specs(child, f"{prefix}.{spec[slot + '_name']}")
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return part_class("mixer", spec["mixer"]).cache_need(spec["mixer"])

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.feed_forward = self.feed_forward_norm = self.token_input = None
        for slot, category in self._slots(spec):
            setattr(self, slot, build_part(category, spec[slot], f"{prefix}.{spec[slot + '_name']}", weights, runtime))

    accepts_next_norm = True

    @property
    def first_norm(self):
        return self.mixer_norm

    def forward(self, residual, pending, ctx, cache: LayerCache, next_norm=None):
        from .. import ops

        fused = residual.shape[0] <= ops.fused_rows_limit(self.runtime.dtype, residual.device)
        if self.token_input is not None:
            next_norm = None   # the stream still changes after the last sublayer: nobody prepares the next norm from it
        if self.feed_forward is None:
            pending = norm_then_part(self.mixer_norm, self.mixer, residual, pending, fused, next_norm, ctx, cache)
        else:
            pending = norm_then_part(self.mixer_norm, self.mixer, residual, pending, fused, self.feed_forward_norm, ctx, cache)
            pending = norm_then_part(self.feed_forward_norm, self.feed_forward, residual, pending, fused, next_norm, ctx)
        if self.token_input is not None:
            self.token_input.forward(residual, ctx, pending)   # completes the residual with what is pending, then adds its own
            pending = None
        return residual, pending


class StreamVectorBlock(Block):
    """x -> x + vector: a learned vector, one row of a table, joins every row of the stream (what a model adds before each pass
    of a run of layers that it repeats).  It keeps nothing between steps and is no layer of its own in a trace.

    params: ``tensor`` (the table's full name), ``rows``, ``size``, ``row`` (which row this block adds)."""

    capturable = True
    traced = False

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(spec["tensor"], (spec["rows"], spec["size"]), std=0.5)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.vector = weights.get(spec["tensor"], torch.float32)[int(spec["row"])].contiguous()

    def forward(self, residual, pending, ctx, cache: LayerCache):
        from .. import ops

        ops.add_row_vector(residual, pending, self.vector)
        return residual, None


register_part("block", "pre_norm_residual", PreNormResidualBlock)
register_part("block", "stream_vector", StreamVectorBlock)
