"""Attention over the paged cache: grouped-query attention with a position encoding, and attention whose heads are biased by
distance, mixed before the softmax and gated after it."""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, LayerCache, Mixer, build_part, register_part
from .spec import PartSpec, TensorSpec


class Attention(Mixer):
    """q, k, v projections, position encoding, cache write, attention, output projection.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``position`` (a PartSpec), optional ``window`` (0 = every earlier token) and
    ``scale`` (default head_dim ** -0.5).
    tensors: ``<prefix>.{q,k,v}_proj.weight [heads * head_dim, hidden]``,
    ``<prefix>.o_proj.weight [hidden, num_heads * head_dim]``; no biases
    (src/model_config.cpp:81-95).

    The reference issues three projections (src/cuda/model.cu:412-421); here their
    weights are stacked once at load time and one product yields ``[q | k | v]``.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, d = spec["hidden_size"], spec["head_dim"]
        q, kv = spec["num_heads"] * d, spec["num_kv_heads"] * d
        return [
            TensorSpec(f"{prefix}.q_proj.weight", (q, hidden)),
            TensorSpec(f"{prefix}.k_proj.weight", (kv, hidden)),
            TensorSpec(f"{prefix}.v_proj.weight", (kv, hidden)),
            TensorSpec(f"{prefix}.o_proj.weight", (hidden, q)),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return CacheNeed("pages", kv_heads=spec["num_kv_heads"], head_dim=spec["head_dim"], window=int(spec.get("window", 0) or 0))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden = int(spec["hidden_size"])
        self.q_heads = int(spec["num_heads"])
        self.kv_heads = int(spec["num_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = int(spec.get("window", 0) or 0)
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        dtype = runtime.dtype
        self.w_qkv = torch.cat([weights.get(f"{prefix}.{n}_proj.weight", dtype) for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = weights.get(f"{prefix}.o_proj.weight", dtype).contiguous()
        self.position = build_part("position", spec["position"], prefix, weights, runtime)
        self.qkv_width = (self.q_heads + 2 * self.kv_heads) * self.head_dim

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        qkv = ws.get("qkv", tokens, self.qkv_width, dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_qkv, qkv)
        else:
            ops.linear(x, self.w_qkv, qkv)
        table = self.position.rotary_table()
        if table is None:
            self.position.apply(qkv, ctx, self.q_heads, self.kv_heads, self.head_dim)
            inv_freq, rotary_dim = None, 0
        else:
            inv_freq, rotary_dim = table
        mixed = ws.get("attention", tokens, self.q_heads * self.head_dim, dtype)
        ops.attention_step(qkv, ctx.positions, ctx.token_seq, cache.block_table, inv_freq, rotary_dim, cache.pages, mixed,
                           self.q_heads, self.kv_heads, self.head_dim, cache.page_size, self.window, self.scale,
                           write_cache=cache.writes, batch=ctx)
        if accumulate_into is not None:
            ops.linear_accumulate(mixed, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        return out


class MixedHeadsAttention(Mixer):
    """Grouped heads without a rotation: positions enter through a distance bias, the heads' scores are mixed by a learned matrix
    before the softmax, and the concatenated heads pass an output gate before the output projection.

    Score of query head g at position i for key j: (q_g . k_j) * scale - slope_g (i - j); head h sees sum_g M[h, g] score_g;
    key j is visible while 0 <= i - j (and i - j < window, if there is a window); an ordinary softmax over the visible keys;
    out = W_o (concat_h(softmax_h . v) * sigmoid(W_gate x)).

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads`` (query head h reads key/value head h // (heads / kv heads)),
    ``key_dim`` (queries and keys), ``value_dim``, ``scale``, ``window`` (0: every earlier token), ``distance_slopes``
    (one slope per head, or None for no bias), ``mix_heads`` (tensor ``<prefix>.talk`` [heads, heads], row h mixing into head h),
    ``output_gate`` (tensor ``<prefix>.g`` [heads * value_dim, hidden]).
    tensors: ``<prefix>.q`` [heads * key_dim, hidden], ``<prefix>.k`` [kv * key_dim, hidden], ``<prefix>.v`` [kv * value_dim, hidden],
    ``<prefix>.o`` [hidden, heads * value_dim]; no biases.  q, k, v and the gate are one stacked product.  Keys and values are
    two planes of a page (of different widths if ``key_dim != value_dim``); scores, mix, softmax and the gate are 32-bit.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec) -> tuple[int, int, int, int, int]:
        return int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["key_dim"]), int(spec["value_dim"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, kv, key_dim, value_dim = cls._sizes(spec)
        std = hidden ** -0.5
        specs = [TensorSpec(f"{prefix}.q", (heads * key_dim, hidden), std=std), TensorSpec(f"{prefix}.k", (kv * key_dim, hidden), std=std),
                 TensorSpec(f"{prefix}.v", (kv * value_dim, hidden), std=std)]
        if spec.get("mix_heads"):
            specs.append(TensorSpec(f"{prefix}.talk", (heads, heads), std=heads ** -0.5))
        if spec.get("output_gate"):
            specs.append(TensorSpec(f"{prefix}.g", (heads * value_dim, hidden), std=std))
        return specs + [TensorSpec(f"{prefix}.o", (hidden, heads * value_dim), std=(heads * value_dim) ** -0.5)]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, _, kv, key_dim, value_dim = cls._sizes(spec)
        return CacheNeed("pages", window=int(spec.get("window", 0) or 0), planes=((kv, key_dim), (kv, value_dim)))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.kv_heads, self.key_dim, self.value_dim = self._sizes(spec)
        self.window = int(spec.get("window", 0) or 0)
        self.scale = float(spec["scale"]) if spec.get("scale") is not None else self.key_dim ** -0.5
        dtype = runtime.dtype
        stacked = [weights.get(f"{prefix}.{n}", dtype) for n in ("q", "k", "v")]
        self.k_offset = self.heads * self.key_dim
        self.v_offset = self.k_offset + self.kv_heads * self.key_dim
        self.gate_offset = -1
        if spec.get("output_gate"):
            self.gate_offset = self.v_offset + self.kv_heads * self.value_dim
            stacked.append(weights.get(f"{prefix}.g", dtype))
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()
        slopes = spec.get("distance_slopes")
        self.slopes = None if slopes is None else torch.tensor([float(v) for v in slopes], dtype=torch.float32, device=runtime.device)
        self.mix = weights.get(f"{prefix}.talk", torch.float32).contiguous() if spec.get("mix_heads") else None
        self.folded_slopes = ops.fast.folded_slopes(self.slopes, self.mix) if self.slopes is not None and self.slopes.is_cuda else None

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("qkv_gate", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        if cache.writes:
            ops.store_kv_planes(rows, self.k_offset, self.v_offset, ctx.positions, ctx.token_seq, cache, self.kv_heads, self.key_dim, self.value_dim)
        mixed = ws.get("attention", tokens, self.heads * self.value_dim, dtype)
        ops.mixed_heads_attention(rows, self.gate_offset, ctx.positions, ctx.token_seq, cache, self.slopes, self.mix, mixed, self.heads, self.kv_heads,
                                  self.key_dim, self.value_dim, self.window, self.scale, batch=ctx, folded_slopes=self.folded_slopes)
        if accumulate_into is not None:
            ops.linear_accumulate(mixed, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(mixed, self.w_o, out)
        return out


register_part("mixer", "attention", Attention)
register_part("mixer", "mixed_heads_attention", MixedHeadsAttention)
