"""A plain, slow statement of the Latinex architecture in float64, one function per mechanism.

It takes a configuration as the dictionary of ``config.json`` and the weights as a dictionary name -> tensor,
and runs one whole sequence at a time, token after token where the mechanism is a recurrence.  Nothing here is
shared with the engine: no part, no kernel, no configuration class.

Notation: ``T`` tokens, ``W`` the model width.  Linear weights are ``[out, in]`` and applied as ``x @ M.T``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def dyt(x, alpha, w, b):
    """The model's norm: an element-wise squashing, no statistics: tanh(alpha x) w + b."""
    return torch.tanh(alpha * x) * w + b


def rotate_pairs(x, positions, base, dims):
    """x [T, heads, d]: elements 2i and 2i+1 (i < dims/2) turn by position * base^(-2i/dims); the rest stay."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def softmax_rows(scores, visible):
    """Softmax over the visible entries of every row; scores and visible are [T, T] (query, key)."""
    scores = scores.masked_fill(~visible, -math.inf)
    scores = scores - scores.max(dim=-1, keepdim=True).values
    e = torch.exp(scores)
    return e / e.sum(dim=-1, keepdim=True)


def causal(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def window_with_first(T, size, keep_first):
    """Query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)
    dist = i[:, None] - i[None, :]
    return (dist >= 0) & ((dist < size) | (i[None, :] < keep_first))


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the distance table for distance n >= 0: exact below rows/2, then logarithmic up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def latent_attention(h, m, wt, p, eps):
    """Queries through a normed latent; keys and values from a normed latent ``c`` shared by all heads plus one
    rotated key part shared by all heads; causal softmax."""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms(h @ wt[p + "dq"].T, eps) * wt[p + "dq.norm"]
    q = (cq @ wt[p + "uq"].T).reshape(T, H, d + dr)
    rot = m.get("rot") or {"base": 10000.0, "dims": 0}
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, rot["base"], rot["dims"])
    down = h @ wt[p + "dkv"].T
    c = rms(down[:, :r], eps) * wt[p + "dkv.norm"]
    k_rot = rotate_pairs(down[:, None, r:], pos, rot["base"], rot["dims"])[:, 0]      # [T, dr]
    k_plain = (c @ wt[p + "uk"].T).reshape(T, H, d)
    v = (c @ wt[p + "uv"].T).reshape(T, H, dv)
    out = torch.empty(T, H, dv, dtype=F64)
    vis = causal(T)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out[:, hd] = softmax_rows(s, vis) @ v[:, hd]
    return out.reshape(T, H * dv) @ wt[p + "o"].T


def window_attention(h, m, wt, p, window_delta=0, keep_delta=0):
    """Grouped-query attention whose values are its keys, with a learned bias by distance, a sliding window that
    keeps the first tokens, and a sigmoid gate on the concatenated heads.  The deltas make a deliberately wrong
    window or kept count (for showing that a test would notice)."""
    T = h.shape[0]
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    q = (h @ wt[p + "q"].T + wt[p + "q.b"]).reshape(T, H, d)
    k = (h @ wt[p + "k"].T + wt[p + "k.b"]).reshape(T, G, d)
    rel = wt[p + "rel"]
    rows = rel.shape[0]
    mask = m.get("mask")
    vis = (window_with_first(T, mask["size"] + window_delta, max(mask.get("keep_first", 0) + keep_delta, 0))
           if mask else causal(T))
    idx = torch.tensor([[distance_bucket(max(i - j, 0), rows, m["bias_max"]) for j in range(T)] for i in range(T)])
    out = torch.empty(T, H, d, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] + rel[:, hd][idx]
        out[:, hd] = softmax_rows(s, vis) @ k[:, g]
    gate = torch.sigmoid(h @ wt[p + "g"].T)
    return (out.reshape(T, H * d) * gate) @ wt[p + "o"].T


def causal_conv_silu(x, w, b):
    """x [T, C]; w [C, taps] with the last column the current token's; zeros before the start; then silu."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], dim=0)
    y = b[None, :].expand(T, C).clone()
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return silu(y)


def mamba2(h, m, wt, p, eps):
    """State-space duality layer walked token by token: a scalar decay per head, keys and queries (B, C) per group."""
    T = h.shape[0]
    nh, dv, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner = nh * dv
    proj = h @ wt[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, wt[p + "conv"], wt[p + "conv.b"])
    x = xbc[:, :inner].reshape(T, nh, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + wt[p + "dt_bias"])
    decay = torch.exp(-torch.exp(wt[p + "A_log"]) * dt)                 # [T, nh]
    S = torch.zeros(nh, N, dv, dtype=F64)
    y = torch.empty(T, nh, dv, dtype=F64)
    for t in range(T):
        for hd in range(nh):
            g = hd // (nh // G)
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + wt[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m.get("norm_groups", 1)
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * wt[p + "norm"]
    return y @ wt[p + "o"].T


def expert(h, wt, p):
    return (silu(h @ wt[p + "gate"].T) * (h @ wt[p + "up"].T)) @ wt[p + "down"].T


def mixture(h, mlp, wt, p, choices=None):
    """Sigmoid router; the ``top`` experts with the largest scores; an expert's score multiplies its input; a shared
    expert is added.  ``choices`` ([T, top] expert ids) overrides the selection (for following an engine's choice
    at a near-tie); returns (output, scores, chosen)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.sigmoid(h @ wt[p + "router"].T)                      # [T, E]
    chosen = torch.topk(scores, top, dim=-1).indices if choices is None else choices.to(torch.long)
    out = torch.zeros(h.shape[0], wt[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += expert(scores[t, e] * h[t:t + 1], wt, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + expert(h, wt, p + "shared.")
    return out, scores, chosen


def forward(config: dict, weights: dict, tokens, want_layers: bool = False, choices=None, window_delta=0, keep_delta=0):
    """Logits [T, vocab] for one sequence; with ``want_layers`` also the residual stream after every layer and the
    router scores and choices of every routed layer.  ``choices``: per routed layer (in order) a [T, top] tensor of
    expert ids to follow."""
    wt = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = wt["embed"][torch.tensor(tokens)] * config.get("embedding", {}).get("scale", 1.0)
    after, routed, seen = [], 0, []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = dyt(x, wt[p + "norm1.alpha"], wt[p + "norm1"], wt[p + "norm1.b"])
        if layer["type"] == "latent_attention":
            x = x + latent_attention(h, layer["mixer"], wt, p + "mix.", eps)
        elif layer["type"] == "attention":
            x = x + window_attention(h, layer["mixer"], wt, p + "mix.", window_delta, keep_delta)
        elif layer["type"] == "mamba2":
            x = x + mamba2(h, layer["mixer"], wt, p + "mix.", eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            h = dyt(x, wt[p + "norm2.alpha"], wt[p + "norm2"], wt[p + "norm2.b"])
            y, scores, chosen = mixture(h, layer["mlp"], wt, p + "mlp.", None if choices is None else choices[routed])
            seen.append((scores, chosen))
            routed += 1
            x = x + y
        after.append(x.clone())
    h = dyt(x, wt["final.norm.alpha"], wt["final.norm"], wt["final.norm.b"])
    logits = (h @ wt["head"].T) * config.get("logit_scale", 1.0)
    if want_layers:
        return logits, after, seen
    return logits


def load_folder(model_dir):
    import json
    import os

    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in
         load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


def generate_greedy(config, W, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(torch.argmax(forward(config, W, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
