"""Feed-forwards: the gated one, and the plain one of two products with an activation between them."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import ConfigError
from .base import FeedForward, register_part
from .spec import PartSpec, TensorSpec


class GatedMLP(FeedForward):
    """down( act(gate(x)) * up(x) ) with act = SiLU (src/model.cpp:187-203, src/operators.cpp:148-164).

    params: ``hidden_size``, ``intermediate_size``, ``activation`` ("silu", or "clamped_sigmoid": with g = min(gate, limit) and
    u = clamp(up, -limit, limit) the product is g * sigmoid(alpha * g) * (u + shift); params ``limit``, ``alpha``, ``shift``),
    optional ``names`` = (gate, up, down) tensor suffixes in full.
    tensors: ``<prefix>.{gate,up}_proj.weight [inter, hidden]``,
    ``<prefix>.down_proj.weight [hidden, inter]``.  gate and up are stacked at load
    time into one ``[2 * inter, hidden]`` product; the activation and the product with
    ``up`` are computed in 32-bit.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _names(cls, spec: PartSpec, prefix: str) -> tuple[str, str, str]:
        gate, up, down = spec.get("names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
        return f"{prefix}.{gate}", f"{prefix}.{up}", f"{prefix}.{down}"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        gate, up, down = cls._names(spec, prefix)
        if spec.get("names"):
            return [TensorSpec(gate, (inter, hidden), std=hidden ** -0.5), TensorSpec(up, (inter, hidden), std=hidden ** -0.5), TensorSpec(down, (hidden, inter), std=inter ** -0.5)]
        return [TensorSpec(gate, (inter, hidden)), TensorSpec(up, (inter, hidden)), TensorSpec(down, (hidden, inter))]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.activation = spec.get("activation", "silu")
        if self.activation not in ("silu", "clamped_sigmoid"):
            raise ConfigError(f"gated_mlp has no activation {spec.get('activation')!r}")
        if self.activation == "clamped_sigmoid":
            self.limit, self.alpha, self.shift = float(spec["limit"]), float(spec["alpha"]), float(spec["shift"])
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        dtype = runtime.dtype
        gate, up, down = self._names(spec, prefix)
        self.w_gate_up = torch.cat([weights.get(gate, dtype), weights.get(up, dtype)], dim=0).contiguous()
        self.w_down = weights.get(down, dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_down)

    def forward(self, x, ctx, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        act = ws.get("activated", tokens, self.inter, dtype)
        if self.activation == "clamped_sigmoid" and tokens <= ops.fused_rows_limit(dtype, act.device):
            # few rows: the clamps, the gate and the shift are applied in the stacked product's epilogue
            clamp = (self.limit, self.alpha, self.shift)
            if isinstance(x, ops.LazyNorm):
                ops.norm_linear(x, self.w_gate_up, act, gated=True, clamp=clamp)
            else:
                ops.linear_gated(x, self.w_gate_up, act, clamp=clamp)
        elif self.activation == "clamped_sigmoid":
            # the stacked product, then the clamps, the gate and the shift in one row-wise kernel (32-bit inside)
            gate_up = ws.get("gate_up", tokens, 2 * self.inter, dtype)
            if isinstance(x, ops.LazyNorm):
                ops.norm_linear(x, self.w_gate_up, gate_up)
            else:
                ops.linear(x, self.w_gate_up, gate_up)
            ops.clamped_gate_mul(gate_up, act, self.limit, self.alpha, self.shift)
        elif tokens <= ops.fused_rows_limit(dtype, act.device):
            # few rows: the gate is applied in the first product's epilogue, the residual add in the second's
            if isinstance(x, ops.LazyNorm):
                ops.norm_linear(x, self.w_gate_up, act, gated=True)
            else:
                ops.linear_gated(x, self.w_gate_up, act)
        elif dtype == torch.bfloat16:
            ops.linear_gated(x.tensor() if isinstance(x, ops.LazyNorm) else x, self.w_gate_up, act)   # picks the fused kernel for its size
        else:
            if isinstance(x, ops.LazyNorm):
                x = x.tensor()
            gate_up = ws.get("gate_up", tokens, 2 * self.inter, dtype)
            ops.linear(x, self.w_gate_up, gate_up)
            ops.silu_mul(gate_up, act)
        if accumulate_into is not None:
            ops.linear_accumulate(act, self.w_down, accumulate_into, prepare)
            return None
        out = ws.get("ff_out", tokens, self.hidden, dtype)
        ops.linear(act, self.w_down, out)
        return out


class DenseMLP(FeedForward):
    """down( act(up(x)) ), no gate and no biases.

    params: ``hidden_size``, ``intermediate_size``, ``activation`` ("relu_squared", "gelu_tanh" or "silu"; ops.ACTIVATIONS),
    optional ``up_name`` / ``down_name`` (the tensors are ``<prefix>.<name>``: "up" and "down" unless given).
    The activation is computed in 32-bit on the first product's (rounded) output.  With few rows the norm in front and the
    activation behind are applied inside the first product and the residual add inside the second, as the gated feed-forward does.
    """

    capturable = True
    accepts_lazy_norm = True
    fuses_residual_add = True
    prepares_next_norm = True

    @classmethod
    def _names(cls, spec: PartSpec, prefix: str) -> tuple[str, str]:
        return f"{prefix}.{spec.get('up_name', 'up')}", f"{prefix}.{spec.get('down_name', 'down')}"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        up, down = cls._names(spec, prefix)
        return [TensorSpec(up, (inter, hidden), std=hidden ** -0.5), TensorSpec(down, (hidden, inter), std=inter ** -0.5)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.activation = spec.get("activation", "relu_squared")
        if self.activation not in ops.ACTIVATIONS:
            raise ConfigError(f"dense_mlp has no activation {self.activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        up, down = self._names(spec, prefix)
        self.w_up = weights.get(up, runtime.dtype).contiguous()
        self.w_down = weights.get(down, runtime.dtype).contiguous()

    def adds_to_residual(self, rows: int) -> bool:
        return ops.can_accumulate(rows, self.w_down)

    def forward(self, x, ctx, accumulate_into=None, prepare=None):
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, x.shape[0]
        act = ws.get("activated", tokens, self.inter, dtype)
        ops.linear_activated(x, self.w_up, act, self.activation)   # few rows: norm, product and activation are one kernel
        if accumulate_into is not None:
            ops.linear_accumulate(act, self.w_down, accumulate_into, prepare)
            return None
        out = ws.get("ff_out", tokens, self.hidden, dtype)
        ops.linear(act, self.w_down, out)
        return out


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "dense_mlp", DenseMLP)
