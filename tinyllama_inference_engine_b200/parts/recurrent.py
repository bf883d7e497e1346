"""Recurrent mixers: a state of fixed size per request instead of a cache that grows: a gated recurrence per channel, and
the gated delta rule over a matrix per head."""
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


class ChannelDeltaRule(Mixer):
    """The gated delta rule with one decay per head and key channel: a matrix of fast weights per head that every token first
    lets decay, then corrects towards its value along its key, then reads with its query.

    Per token: q = W_q x, k = W_k x (``kv_heads`` heads of ``dim``; head h reads q/k head h // (heads / kv_heads)), v = W_v x (``heads`` of
    ``vdim``); each passes a short causal convolution over time per channel (``<tensor>.conv`` [channels, taps], the last column the
    current token's, zeros before a request's start) and silu; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)),
    q times dim^-1/2.  beta = sigmoid(W_b x) per head; decay g = exp(-exp(A_log_h) softplus(W_a2 W_a1 x + dt_bias)) per head and key
    channel.  Per head, in this order: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Each head's o is divided by
    its root mean square (``eps``), times ``<prefix>.norm`` [vdim], times sigmoid(W_g2 W_g1 x); then W_o.

    The state (32-bit, zero for a new request) is the heads' matrices and the convolution's last taps - 1 inputs, one flat vector
    in the request's state slot.  Everything after the projections is 32-bit.  The eight input products are one stacked product;
    the two second halves of the low-rank pairs are products of their own.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``key_dim``, ``value_dim``, ``taps``, ``decay_rank``, ``gate_rank``, ``eps``,
    ``unit_eps`` (1e-6).
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return tuple(int(spec[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "key_dim", "value_dim", "taps", "decay_rank", "gate_rank"))

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, heads, kv, dim, vdim, taps, decay_rank, gate_rank = cls._sizes(spec)
        std = hidden ** -0.5
        return [
            TensorSpec(f"{prefix}.q", (kv * dim, hidden), std=std), TensorSpec(f"{prefix}.q.conv", (kv * dim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.k", (kv * dim, hidden), std=std), TensorSpec(f"{prefix}.k.conv", (kv * dim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.v", (heads * vdim, hidden), std=std), TensorSpec(f"{prefix}.v.conv", (heads * vdim, taps), std=taps ** -0.5),
            TensorSpec(f"{prefix}.b", (heads, hidden), std=std), TensorSpec(f"{prefix}.A_log", (heads,), std=0.5),
            TensorSpec(f"{prefix}.norm", (vdim,), init="norm", std=0.1),
            TensorSpec(f"{prefix}.a1", (decay_rank, hidden), std=std), TensorSpec(f"{prefix}.a2", (heads * dim, decay_rank), std=decay_rank ** -0.5),
            TensorSpec(f"{prefix}.dt_bias", (heads * dim,), std=1.0),
            TensorSpec(f"{prefix}.g1", (gate_rank, hidden), std=std), TensorSpec(f"{prefix}.g2", (heads * vdim, gate_rank), std=gate_rank ** -0.5),
            TensorSpec(f"{prefix}.o", (hidden, heads * vdim), std=(heads * vdim) ** -0.5),
        ]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, heads, kv, dim, vdim, taps, _, _ = cls._sizes(spec)
        words, _ = ops.delta_state_words(heads, dim, vdim, 2 * kv * dim + heads * vdim, taps)
        return CacheNeed("state", state_shape=(words,))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.decay_rank, self.gate_rank = self._sizes(spec)
        self.eps, self.unit_eps = float(spec["eps"]), float(spec.get("unit_eps", 1e-6))
        dtype = runtime.dtype
        self.channels = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        _, self.conv_offset = ops.delta_state_words(self.heads, self.dim, self.vdim, self.channels, self.taps)
        self.w_in = torch.cat([weights.get(f"{prefix}.{n}", dtype) for n in ("q", "k", "v", "b", "a1", "g1")], dim=0).contiguous()
        self.beta_offset = self.channels
        self.a1_offset = self.beta_offset + self.heads
        self.g1_offset = self.a1_offset + self.decay_rank
        self.w_a2 = weights.get(f"{prefix}.a2", dtype).contiguous()
        self.w_g2 = weights.get(f"{prefix}.g2", dtype).contiguous()
        self.conv = torch.cat([weights.get(f"{prefix}.{n}.conv", torch.float32) for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = weights.get(f"{prefix}.A_log", torch.float32).contiguous()
        self.dt_bias = weights.get(f"{prefix}.dt_bias", torch.float32).contiguous()
        self.out_weight = weights.get(f"{prefix}.norm", torch.float32).contiguous()
        self.w_o = weights.get(f"{prefix}.o", dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_o)

    def forward(self, x, ctx, cache: LayerCache, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        rows = ws.get("delta_in", tokens, self.w_in.shape[0], dtype)
        if isinstance(x, ops.LazyNorm):
            ops.norm_linear(x, self.w_in, rows)
        else:
            ops.linear(x, self.w_in, rows)
        decay_in = ws.get("delta_decay_in", tokens, self.heads * self.dim, dtype)
        gate = ws.get("delta_gate", tokens, self.heads * self.vdim, dtype)
        first, second = rows[:, self.a1_offset : self.g1_offset], rows[:, self.g1_offset :]   # the low-rank pairs' first halves, columns of the stacked product
        ops.linear(first, self.w_a2, decay_in)
        ops.linear(second, self.w_g2, gate)
        prep = ws.get("delta_prep", tokens, self.channels + self.heads + self.heads * self.dim, torch.float32)
        ops.delta_prepare(rows, self.beta_offset, decay_in, self.conv, self.a_log, self.dt_bias, cache.state, self.conv_offset, ctx, prep, self.heads,
                          self.kv_heads, self.dim, self.vdim, self.unit_eps, self.dim ** -0.5)
        read = ws.get("delta_read", tokens, self.heads * self.vdim, torch.float32)
        ops.delta_rule(prep, cache.state, ctx, read, self.heads, self.kv_heads, self.dim, self.vdim)
        gated = ws.get("recurrent_out", tokens, self.heads * self.vdim, dtype)
        ops.delta_gate_norm(read, gate, self.out_weight, gated, self.eps, self.heads, self.vdim)
        if accumulate_into is not None:
            ops.linear_accumulate(gated, self.w_o, accumulate_into, prepare)
            return None
        out = ws.get("mixer_out", tokens, self.hidden, dtype)
        ops.linear(gated, self.w_o, out)
        return out


register_part("mixer", "mingru", MinGRU)
register_part("mixer", "channel_delta_rule", ChannelDeltaRule)
