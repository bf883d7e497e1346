"""Recurrent mixers: a state of fixed size per request instead of a cache that grows."""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, LayerCache, Mixer, register_part
from .spec import PartSpec, TensorSpec


class MinGRU(Mixer):
    """A gated recurrence whose gates read only the current token, so a prompt portion is a scan and not a loop.

    With a = W_z h + b_z and u = W_x h + b_x, per channel: z = sigmoid(a); the candidate is u + 1/2 for u >= 0 and
    sigmoid(u) below; S_t = (1 - z_t) S_{t-1} + z_t cand_t from S = 0; the mixer's output is W_o (S_t * silu(W_g h_t)).

    params: ``hidden_size``, ``width`` (channels of the state).
    tensors: ``<prefix>.z``, ``<prefix>.x``, ``<prefix>.g`` [width, hidden], ``<prefix>.z.b``, ``<prefix>.x.b`` [width],
    ``<prefix>.o`` [hidden, width].  The three input products are stacked into one [3 width, hidden] at load time; biases,
    gates, candidate and state are 32-bit in both precisions, and the state lives in the request's slot of the cache
    manager's state group (zero when the request is admitted).
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, width = spec["hidden_size"], spec["width"]
        std = hidden ** -0.5
        return [
            TensorSpec(f"{prefix}.z", (width, hidden), std=std), TensorSpec(f"{prefix}.z.b", (width,), std=1.0),
            TensorSpec(f"{prefix}.x", (width, hidden), std=std), TensorSpec(f"{prefix}.x.b", (width,), std=0.5),
            TensorSpec(f"{prefix}.g", (width, hidden), std=std), TensorSpec(f"{prefix}.o", (hidden, width), std=width ** -0.5),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed("state", state_shape=(int(spec["width"]),))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden = int(spec["hidden_size"])
        self.width = int(spec["width"])
        dtype = runtime.dtype
        self.w_zxg = torch.cat([weights.get(f"{prefix}.{n}", dtype) for n in ("z", "x", "g")], dim=0).contiguous()
        self.bias_z = weights.get(f"{prefix}.z.b", torch.float32).contiguous()
        self.bias_x = weights.get(f"{prefix}.x.b", torch.float32).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        zxg = ws.get("recurrent_in", tokens, 3 * self.width, dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_zxg, zxg)
        else:
            ops.linear(x, self.w_zxg, zxg)
        gated = ws.get("recurrent_out", tokens, self.width, dtype)
        ops.mingru_scan(zxg, self.bias_z, self.bias_x, cache.state, ctx.seq_starts, ctx.state_slots, gated, ctx.max_q_len)
        if accumulate_into is not None:
            ops.linear_accumulate(gated, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(gated, self.w_o, out)
        return out


register_part("mixer", "mingru", MinGRU)
