"""A plain, slow Zirutar: whole sequences, no cache, one function per mechanism, token-by-token recurrence, scores materialised.

It shares no code with the engine.  Everything is computed in the dtype of the tensors it is given (the tests use float32 or
float64).  ``weights`` maps tensor names to tensors; ``config`` is the dictionary of a config.json.
"""
from __future__ import annotations

import math

import torch


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def visible(i: int, j: int, window, keep_first: int) -> bool:
    """Whether query position i sees key position j under a sliding window that keeps the first tokens (``window`` None: no window)."""
    return j <= i and (window is None or i - j < window or j < keep_first)


def windowed_attention(h, w, p, sizes, eps):
    """Grouped attention without positions: q and k unit-rms per head, values are the un-normalised keys, a window that keeps
    the first tokens, one output gate per head."""
    T = h.shape[0]
    H, G, dim = sizes["heads"], sizes["kv_heads"], sizes["dim"]
    mask = sizes.get("mask") or {}
    window, keep = mask.get("size"), mask.get("keep_first", 0)
    q = (h @ w[p + ".q"].T).view(T, H, dim)
    k = (h @ w[p + ".k"].T).view(T, G, dim)
    v = k
    qn, kn = unit_rms(q, eps), unit_rms(k, eps)
    gate = torch.sigmoid(h @ w[p + ".g"].T)
    out = torch.zeros(T, H, dim, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        for i in range(T):
            keys = [j for j in range(i + 1) if visible(i, j, window, keep)]
            s = torch.stack([(qn[i, head] * kn[j, kv]).sum() * sizes["scale"] for j in keys])
            pr = torch.softmax(s, dim=0)
            out[i, head] = sum(pr[n] * v[j, kv] for n, j in enumerate(keys)) * gate[i, head]
    return out.reshape(T, H * dim) @ w[p + ".o"].T


def rotate_pairs(x, positions, base, dims):
    """Interleaved rotation of the first ``dims`` elements of the last axis: (x[2i], x[2i+1]) turn by positions * base^(-2i/dims)."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(x.dtype) * (base ** (-2.0 * i / dims))
        cos, sin = torch.cos(angle), torch.sin(angle)
        shape = [-1] + [1] * (x.dim() - 2)
        cos, sin = cos.view(shape), sin.view(shape)
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * cos - b * sin
        out[..., 2 * i + 1] = b * cos + a * sin
    return out


def latent_attention(h, w, p, sizes, eps):
    """Keys and values expanded from one cached latent per token, a rotated key part shared by the heads, a sink in the softmax."""
    T = h.shape[0]
    H, dim, rot, vdim, rank = sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"]
    positions = torch.arange(T)
    q = (h @ w[p + ".q"].T).view(T, H, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    down = h @ w[p + ".dkv"].T
    latent = unit_rms(down[:, :rank], eps) * w[p + ".dkv.norm"]
    k_rot = down[:, rank:]
    k_plain = (latent @ w[p + ".uk"].T).view(T, H, dim)
    v = (latent @ w[p + ".uv"].T).view(T, H, vdim)
    q_rot = rotate_pairs(q_rot, positions, sizes["rot"]["base"], sizes["rot"]["dims"])
    k_rot = rotate_pairs(k_rot, positions, sizes["rot"]["base"], sizes["rot"]["dims"])
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for head in range(H):
        sink = w[p + ".sink"][head]
        for i in range(T):
            s = ((k_plain[: i + 1, head] @ q_plain[i, head]) + (k_rot[: i + 1] @ q_rot[i, head])) * sizes["scale"]
            m = torch.maximum(s.max(), sink)
            e = torch.exp(s - m)
            out[i, head] = (e / (e.sum() + torch.exp(sink - m))) @ v[: i + 1, head]
    return out.reshape(T, H * vdim) @ w[p + ".o"].T


def short_convolution(x, taps):
    """Causal per-channel convolution; the last column of ``taps`` [channels, n] multiplies the current token, zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, x.shape[1], dtype=x.dtype), x], dim=0)
    return sum(padded[j : j + T] * taps[:, j] for j in range(n))


def silu(x):
    return x * torch.sigmoid(x)


def channel_delta(h, w, p, sizes, eps):
    """The gated delta rule with one decay per head and key channel, token by token."""
    T = h.shape[0]
    H, G, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    q = silu(short_convolution(h @ w[p + ".q"].T, w[p + ".q.conv"])).view(T, G, dim)
    k = silu(short_convolution(h @ w[p + ".k"].T, w[p + ".k.conv"])).view(T, G, dim)
    v = silu(short_convolution(h @ w[p + ".v"].T, w[p + ".v.conv"])).view(T, H, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + ".b"].T)
    step = torch.nn.functional.softplus((h @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".dt_bias"]).view(T, H, dim)
    decay = torch.exp(-torch.exp(w[p + ".A_log"]).view(1, H, 1) * step)
    gate = torch.sigmoid((h @ w[p + ".g1"].T) @ w[p + ".g2"].T).view(T, H, vdim)
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head].unsqueeze(1) * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    out = unit_rms(out, eps) * w[p + ".norm"] * gate
    return out.reshape(T, H * vdim) @ w[p + ".o"].T


MIXERS = {"attention": windowed_attention, "latent_attention": latent_attention, "channel_delta": channel_delta}


def clamped_feed_forward(h, w, p, mlp):
    limit = mlp["limit"]
    g = torch.clamp(h @ w[p + ".gate"].T, max=limit)
    u = torch.clamp(h @ w[p + ".up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + ".down"].T


def token_side_input(x, tokens, w, layer: int, dim: int, eps):
    """What a layer adds from the token itself: a slice of a second embedding, gated by the stream, projected and normalised."""
    p = f"l{layer}.side"
    e = w["side.embed"][tokens][:, layer * dim : (layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + ".gate"].T) * e) @ w[p + ".proj"].T
    return unit_rms(y, eps) * w[p + ".norm"]


def layer_runs(config):
    """[(layer index, pass number or None if the pass does not start here)] in the order the layers run."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], count)]


def forward(config, w, tokens, trace: list | None = None):
    """Logits [T, vocab] of one sequence; ``trace`` receives the stream after every run of a layer."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens] * config["embedding"]["scale"]
    side = config.get("token_side")
    for index, starts_pass in layer_runs(config):
        layer = config["layers"][index]
        p = f"l{index}"
        if starts_pass is not None:
            x = x + w["loop.step"][starts_pass]
        x = x + MIXERS[layer["type"]](offset_norm(x, w[p + ".norm1"], eps), w, p + ".mix", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + clamped_feed_forward(offset_norm(x, w[p + ".norm2"], eps), w, p + ".mlp", layer["mlp"])
        if side:
            x = x + token_side_input(x, tokens, w, index, side["dim"], eps)
        if trace is not None:
            trace.append(x.clone())
    return (offset_norm(x, w["final.norm"], eps) @ w["embed"].T) * config["logit_scale"]
