"""A plain, slow Marutar: whole sequences, no cache, one function per mechanism, 32-bit throughout.

Marutar is a decoder whose layers are listed one by one in its configuration.  A layer is
``x += mixer(norm1(x))`` and, if it has a feed-forward, ``x += ff(norm2(x))``.  Mixers:

* ``mingru``: a gated recurrence per channel.  With a = W_z h + b_z and u = W_x h + b_x,
  z = sigmoid(a), c = u + 1/2 for u >= 0 and sigmoid(u) below, S_t = (1 - z_t) S_{t-1} + z_t c_t
  from S = 0, and the mixer's output is W_o (S_t * silu(W_g h_t)).
* ``attention``: grouped heads without rotation.  The raw score of head g for query i and key j is
  (q_i . k_j) * scale - slope_g (i - j) with slope_g = 2^(-8 (g + 1) / H); the heads' scores are then mixed
  by a learned H x H matrix before the mask (key j visible from i while 0 <= i - j < window) and the
  softmax; the concatenated heads are multiplied by sigmoid(W_g h) before the output projection.

The embedding adds a learned position vector and is normalised; the feed-forward is W_down relu(W_up h)^2.
Nothing here is shared with the engine: the tests compare the two.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def embed(tokens: list[int], t: dict, eps: float, first_position: int = 0) -> torch.Tensor:
    ids = torch.tensor(tokens, dtype=torch.long)
    places = torch.arange(first_position, first_position + len(tokens))
    return rms_norm(t["embed"][ids] + t["pos"][places], t["embed.norm"], eps)


def mingru_candidate(u: torch.Tensor) -> torch.Tensor:
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru_mixer(h: torch.Tensor, t: dict, prefix: str, state: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Token by token; returns the mixer's output and the state after the last token."""
    z = torch.sigmoid(h @ t[f"{prefix}.z"].T + t[f"{prefix}.z.b"])
    c = mingru_candidate(h @ t[f"{prefix}.x"].T + t[f"{prefix}.x.b"])
    g = h @ t[f"{prefix}.g"].T
    s = torch.zeros(z.shape[1]) if state is None else state.clone()
    rows = []
    for i in range(h.shape[0]):
        s = (1.0 - z[i]) * s + z[i] * c[i]
        rows.append(s * (g[i] * torch.sigmoid(g[i])))
    return torch.stack(rows) @ t[f"{prefix}.o"].T, s


def head_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])


def attention_mixer(h: torch.Tensor, t: dict, prefix: str, mixer: dict) -> torch.Tensor:
    heads, kv_heads, dim, vdim = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    window = (mixer.get("mask") or {}).get("size", 0)
    n = h.shape[0]
    q = (h @ t[f"{prefix}.q"].T).view(n, heads, dim)
    k = (h @ t[f"{prefix}.k"].T).view(n, kv_heads, dim)
    v = (h @ t[f"{prefix}.v"].T).view(n, kv_heads, vdim)
    group = heads // kv_heads
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    distance = (i - j).float()
    slopes = head_slopes(heads)
    raw = torch.stack([(q[:, g] @ k[:, g // group].T) * mixer["scale"] - slopes[g] * distance for g in range(heads)])   # [H, n, n]
    mixed = torch.einsum("hg,gij->hij", t[f"{prefix}.talk"], raw)
    visible = (i - j >= 0) & ((i - j < window) if window else True)
    mixed = mixed.masked_fill(~visible, -math.inf)
    p = torch.softmax(mixed, -1)
    out = torch.cat([p[g] @ v[:, g // group] for g in range(heads)], dim=-1)          # [n, H * vdim]
    out = out * torch.sigmoid(h @ t[f"{prefix}.g"].T)
    return out @ t[f"{prefix}.o"].T


def dense_ff(h: torch.Tensor, t: dict, prefix: str) -> torch.Tensor:
    return (torch.relu(h @ t[f"{prefix}.up"].T) ** 2) @ t[f"{prefix}.down"].T


def forward(config: dict, tensors: dict, tokens: list[int], trace: list | None = None) -> torch.Tensor:
    """Logits [len(tokens), vocab] of a whole sequence; ``trace`` receives the residual stream after every layer."""
    t = {name: value.float() for name, value in tensors.items()}
    eps = config["norm"]["eps"]
    x = embed(tokens, t, eps)
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}"
        h = rms_norm(x, t[f"{prefix}.norm1"], eps)
        if layer["type"] == "mingru":
            x = x + mingru_mixer(h, t, f"{prefix}.mix")[0]
        elif layer["type"] == "attention":
            x = x + attention_mixer(h, t, f"{prefix}.mix", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense_ff(rms_norm(x, t[f"{prefix}.norm2"], eps), t, f"{prefix}.mlp")
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T
