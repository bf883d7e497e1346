"""What a layer adds to the stream from the token itself."""
from __future__ import annotations

import torch

from .. import ops
from .base import TokenInput, register_part
from .spec import PartSpec, TensorSpec


class GatedTokenSlice(TokenInput):
    """x <- x + norm(W_proj (gelu_tanh(W_gate x) * e)), with e a slice of the token's row in a second embedding table.

    The table has one slice of ``dim`` columns per layer; the layer reads columns [``slice`` * dim, (``slice`` + 1) * dim).  The gate
    reads the finished stream (not a normalised copy); the branch is divided by its root mean square (``eps`` inside the root)
    and multiplied by a plain weight before it joins the stream.  Norm statistics and the sum are 32-bit.

    params: ``hidden_size``, ``dim``, ``slice``, ``slices`` (how many the table holds), ``vocab_size``, ``table`` (the table's full
    name), ``eps``.  tensors: ``<table>`` [vocab, slices * dim], ``<prefix>.gate`` [dim, hidden], ``<prefix>.proj`` [hidden, dim],
    ``<prefix>.norm`` [hidden]."""

    capturable = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden, dim = spec["hidden_size"], spec["dim"]
        return [TensorSpec(spec["table"], (spec["vocab_size"], spec["slices"] * dim), std=1.0),
                TensorSpec(f"{prefix}.gate", (dim, hidden), std=hidden ** -0.5), TensorSpec(f"{prefix}.proj", (hidden, dim), std=dim ** -0.5),
                TensorSpec(f"{prefix}.norm", (hidden,), init="norm", std=0.1)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden, self.dim, self.offset = int(spec["hidden_size"]), int(spec["dim"]), int(spec["slice"]) * int(spec["dim"])
        self.eps = float(spec["eps"])
        dtype = runtime.dtype
        self.table = weights.get(spec["table"], dtype).contiguous()
        self.w_gate = weights.get(f"{prefix}.gate", dtype).contiguous()
        self.w_proj = weights.get(f"{prefix}.proj", dtype).contiguous()
        self.weight = weights.get(f"{prefix}.norm", torch.float32).contiguous()

    def forward(self, residual, ctx, pending=None) -> None:
        ws, dtype, tokens = self.runtime.workspace, self.runtime.dtype, residual.shape[0]
        if isinstance(pending, ops.LazyNorm):
            pending = None
        if dtype == torch.float32:
            if pending is not None:
                ops.add_(residual, pending)
            x = residual
        else:
            x = ws.get("stream_rounded", tokens, self.hidden, dtype)
            ops.complete_and_round(residual, pending, x)
        z = ws.get("token_gate", tokens, self.dim, dtype)
        ops.linear(x, self.w_gate, z)
        gated = ws.get("token_gated", tokens, self.dim, dtype)
        ops.gather_gated(z, self.table, ctx.token_ids, gated, self.offset)
        y = ws.get("token_branch", tokens, self.hidden, dtype)
        ops.linear(gated, self.w_proj, y)
        ops.unit_norm_add(residual, y, self.weight, self.eps)


register_part("token_input", "gated_token_slice", GatedTokenSlice)
