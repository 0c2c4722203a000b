"""A plain, slow statement of the Gisilix design in float64, one function per mechanism.

Nothing here is shared with the engine: the tests compare the engine's logits with these functions on small random
models.  A model is a configuration dictionary (the keys of ``config.json``) and a dictionary of tensors by file name.

Notation: ``x`` is the residual stream ``[n, W]`` of one sequence whose first row is position 0; matrices are stored
``[out, in]`` and applied as ``x @ W.T``.  A layer is ``x += mixer(ln1(x))``, then ``x += ff(ln2(x))`` when it has a
feed-forward.  ``round_to`` (a torch dtype or None) rounds what the engine rounds before a matrix product, so that a
bfloat16 run can be followed closely; None keeps everything in float64.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def _r(t: torch.Tensor, round_to) -> torch.Tensor:
    return t if round_to is None else t.to(round_to).to(F64)


def layer_norm(x, w, b, eps):
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def softmax_rows(scores, visible, sink=None):
    """Softmax over the visible keys of every query row; ``sink`` [heads] adds ``exp(sink)`` to the denominator of
    every row of its head and nothing to the numerator.  scores: [heads, n, n]; visible: [n, n] bool."""
    s = scores.masked_fill(~visible, -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.view(-1, 1, 1))
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.view(-1, 1, 1) - m)
    return e / den


def causal(n, window=0):
    i = torch.arange(n).view(n, 1)
    j = torch.arange(n).view(1, n)
    vis = j <= i
    if window:
        vis = vis & (i - j < window)
    return vis


def query_temperature(n, coef, every):
    p = torch.arange(n, dtype=F64)
    return 1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)


def yarn_frequencies(dims, base, scaling):
    """Frequencies of the ``dims / 2`` pairs and the factor on cos and sin."""
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def at(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(at(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v, freqs, amplitude, dims):
    """v [n, ..., d]: neighbours (2i, 2i+1) of the first ``dims`` elements turned by position * freqs[i]."""
    n = v.shape[0]
    a = torch.arange(n, dtype=F64).view(n, *([1] * (v.dim() - 1))) * freqs
    cs, sn = torch.cos(a) * amplitude, torch.sin(a) * amplitude
    out = v.clone()
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * cs - w * sn
    out[..., 1:dims:2] = w * cs + u * sn
    return out


# ---------------------------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------------------------
def attention_keys_values(h, m, t, p, eps, round_to=None):
    """The keys (after their norm) and values of an ``attention`` layer, as its cache holds them: [n, G, d], [n, G, dv]."""
    n = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = rms(h @ t[p + "k"].T, t[p + "k.norm"], eps)
    v = h @ t[p + "v"].T
    return _r(k, round_to).view(n, G, d), _r(v, round_to).view(n, G, dv)


def attention(h, m, t, p, eps, kv=None, round_to=None):
    """Grouped attention with a norm over the whole q (and k) projection, a query factor by position, capped scores, a
    sink in the softmax and an element-wise output gate.  ``kv``: keys and values of the layer this one borrows."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = _r(h, round_to)
    q = rms(h @ t[p + "q"].T, t[p + "q.norm"], eps)
    if m.get("q_temp"):
        q = q * query_temperature(n, m["q_temp"]["coef"], m["q_temp"]["every"]).view(n, 1)
    q = _r(q, round_to).view(n, H, d)
    k, v = kv if kv is not None else attention_keys_values(h, m, t, p, eps, round_to)
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)                 # query head a reads key head a // rep
    vh = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    w = softmax_rows(s, causal(n), t[p + "sink"] if (p + "sink") in t else None)
    o = _r(torch.einsum("hij,jhd->ihd", w, vh).reshape(n, H * dv), round_to)
    if (p + "g") in t:
        o = o * torch.sigmoid(h @ t[p + "g"].T)
    return _r(o, round_to) @ t[p + "o"].T


def latent_attention(h, m, t, p, eps, round_to=None):
    """Attention whose keys and values are read out of one normed latent per token; with ``rot_dim`` a rotated key
    part shared by all heads, a sliding window (``mask.size``) and a gate per head (``.g``) when the layer has them."""
    n = h.shape[0]
    H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    dr = m.get("rot_dim", 0)
    h = _r(h, round_to)
    q = (h @ t[p + "q"].T).view(n, H, d + dr)
    down = h @ t[p + "dkv"].T
    c = _r(rms(down[:, :r], t[p + "dkv.norm"], eps), round_to)
    # with ``round_to``: queries, keys and the heads' outputs are rounded once more, as an engine that stores them in
    # that dtype between its products would
    k = _r((c @ t[p + "uk"].T), round_to).view(n, H, d)
    v = (c @ t[p + "uv"].T).view(n, H, dv)
    s = torch.einsum("ihd,jhd->hij", _r(q[..., :d], round_to), k)
    if dr:
        rot = m["rot"]
        f, amp = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        qr = rotate_pairs(q[..., d:], f, amp, rot["dims"])
        kr = rotate_pairs(down[:, r:], f, amp, rot["dims"])
        s = s + torch.einsum("ihd,jd->hij", _r(qr, round_to), _r(kr, round_to))
    s = s * m["scale"]
    window = (m.get("mask") or {}).get("size", 0)
    w = softmax_rows(s, causal(n, window))
    o = _r(torch.einsum("hij,jhd->ihd", w, v), round_to)
    if (p + "g") in t:
        o = o * torch.sigmoid(h @ t[p + "g"].T).view(n, H, 1)
    return _r(o.reshape(n, H * dv), round_to) @ t[p + "o"].T


# ---------------------------------------------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------------------------------------------
def gated(h, t, p, round_to=None):
    g, u = h @ t[p + "gate"].T, h @ t[p + "up"].T
    return _r(g * torch.sigmoid(g) * u, round_to) @ t[p + "down"].T


def route(h, t, p, top):
    """(chosen experts [n, top], weights [n, top]): the largest logits, softmax over the chosen logits alone."""
    z = h @ t[p + "router"].T + t[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def mixture(h, mlp, t, p, round_to=None, choices=None):
    """``choices`` [n, top]: experts to use instead of the router's own (the weights are then the softmax over
    those experts' logits).  Returns (output, chosen experts, router logits)."""
    top, E = mlp["router"]["top"], mlp["router"]["experts"]
    z = h @ t[p + "router"].T + t[p + "router.b"]
    if choices is None:
        idx, w = route(h, t, p, top)
    else:
        idx = choices.to(torch.long)
        w = torch.softmax(torch.gather(z, 1, idx), dim=-1)
    hr = _r(h, round_to)
    out = torch.zeros_like(h)
    for e in range(E):
        rows, slot = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += w[rows, slot].view(-1, 1) * gated(hr[rows], t, f"{p}e{e}.", round_to)
    if mlp.get("shared"):
        out = out + gated(hr, t, p + "shared.", round_to)
    return out, idx, z


def feed_forward(h, mlp, t, p, round_to=None, choices=None):
    if mlp["kind"] == "dense":
        return gated(_r(h, round_to), t, p, round_to), None, None
    return mixture(h, mlp, t, p, round_to, choices)


# ---------------------------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------------------------
def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], round_to=None, layers_out=None,
            choices: Optional[List[torch.Tensor]] = None, choices_out: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the residual stream
    after every layer.  ``choices``: per mixture layer (in order) the experts to follow.  ``choices_out``: a list
    that receives, per mixture layer, (router logits [n, E], chosen experts [n, top])."""
    t = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)]
    kept = {}
    routed = 0
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = layer_norm(x, t[p + "norm1"], t[p + "norm1.b"], eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(_r(h, round_to), m, t, p + "mix.", eps, round_to)
                y = attention(h, m, t, p + "mix.", eps, kv=kept[i], round_to=round_to)
            else:
                y = attention(h, m, t, p + "mix.", eps, kv=kept[src], round_to=round_to)
        elif layer["type"] in ("latent_attention", "latent_attention_2"):
            y = latent_attention(h, m, t, p + "mix.", eps, round_to)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']}")
        x = x + y
        if layer.get("mlp"):
            h = layer_norm(x, t[p + "norm2"], t[p + "norm2.b"], eps)
            follow = None
            if layer["mlp"]["kind"] == "moe":
                follow = choices[routed] if choices is not None else None
                routed += 1
            y, idx, z = feed_forward(h, layer["mlp"], t, p + "mlp.", round_to, follow)
            if idx is not None and choices_out is not None:
                choices_out.append((z, idx))
            x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    h = layer_norm(x, t["final.norm"], t["final.norm.b"], eps)
    return _r(h, round_to) @ t["embed"].T


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

