"""The Gisilix architecture, put together from parts, and its tensor names.

A pre-norm decoder (``x += mixer(norm1(x))``, then ``x += ff(norm2(x))`` where a layer has a feed-forward) whose norms
are layer norms with weight and bias (:class:`LayerNorm`), whose logits come from the embedding table, and whose layers
(``config.layers[i]``, every layer with sizes of its own) have one of three mixers:

* ``attention``: :class:`PagedAttention` with grouped key/value heads, an RMS norm over the whole q and the whole k
  projection (weights of those sizes), no rotation, a query factor that grows with the logarithm of the position,
  capped scores, a learned sink per head in the softmax's denominator and an element-wise sigmoid gate on the heads;
  with ``kv_from`` the layer has queries only and reads the keys and values that an earlier layer cached (a schedule
  entry with ``cache_from``);
* ``latent_attention``: :class:`LatentAttention` without a query latent and without a rotated part: one normed latent a
  token is all that is cached; every earlier position is visible;
* ``latent_attention_2``: the same with a rotated key part shared by the heads (neighbouring pairs, stretched
  frequencies with an amplitude), a sliding window and a sigmoid gate per head.

The feed-forward is a dense gated network (:class:`DenseSwiGLU`) or a mixture of such experts
(:class:`MoESigmoidTopKGated` with a router bias, the softmax over the chosen logits as weights, and the weights on the
experts' outputs) with an optional shared expert.

Tensor names (linear weights ``[out, in]``): ``embed``, ``final.norm`` (+ ``.b``); per layer ``l<i>.norm{1,2}`` (+
``.b``); ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.router`` (+ ``.b``), ``l<i>.mlp.e<j>.{gate,up,down}``,
``l<i>.mlp.shared.{gate,up,down}``; for attention ``l<i>.mix.{q,q.norm,sink,g,o}`` and, unless the layer borrows,
``l<i>.mix.{k,v,k.norm}``; for the latent mixers ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,o}`` and ``l<i>.mix.g`` where there
is a gate.
"""
from __future__ import annotations

import torch

from ..config.gisilix import GisilixConfig, GisilixLayer
from ..parts import (DenseSwiGLU, GroupedLinear, LatentAttention, LayerNorm, Linear, MoESigmoidTopKGated, PagedAttention,
                     PreNormBlock, RotaryEncoding, leading_rotary_inv_freq, yarn_inv_freq)
from ..registry import register_architecture
from ..weights.source import WeightSource
from .model import DecoderModel, ScheduleEntry
from .notedra import _cat


def _on(weights: WeightSource, t: torch.Tensor) -> torch.Tensor:
    return t if weights.device.type == "meta" else t.to(weights.device)


def _norm(weights: WeightSource, name: str, width: int, eps: float) -> LayerNorm:
    return LayerNorm(weights.vector(name, (width,)), weights.vector(name + ".b", (width,), init="normal"), eps)


def _attention(c: GisilixConfig, m: GisilixLayer, p: str, weights: WeightSource, act) -> PagedAttention:
    W, H, G, d, dv = c.width, m.heads, m.kv_heads, m.dim, m.vdim
    borrows = m.kv_from is not None
    rows = [weights.matrix(p + "q", (H * d, W))]                 # file order: q, k, v, norms, sink, g, o
    if not borrows:
        rows += [weights.matrix(p + "k", (G * d, W)), weights.matrix(p + "v", (G * dv, W))]
    q_norm = weights.vector(p + "q.norm", (H * d,))
    k_norm = None if borrows else weights.vector(p + "k.norm", (G * d,))
    sinks = weights.vector(p + "sink", (H,), init="normal")
    rows.append(weights.matrix(p + "g", (H * dv, W)))            # the gate rides in the fused projection
    out = Linear(weights.matrix(p + "o", (W, H * dv)), p + "o")
    return PagedAttention(qkv=Linear(_cat(rows), p + ("q|g" if borrows else "q|k|v|g")), out=out, num_heads=H,
                          num_kv_heads=G, head_dim=d, value_dim=dv, mask="full", position=None, softmax_scale=m.scale,
                          act_dtype=act, wide_norm=(q_norm, k_norm, c.eps), softcap=m.softcap, sinks=sinks,
                          temperature=(m.temp_coef, m.temp_every) if m.temp_every else None, borrows_kv=borrows,
                          gate_fused=True)


def _latent(c: GisilixConfig, m: GisilixLayer, p: str, weights: WeightSource, act) -> LatentAttention:
    W, H, d, dr, dv, r = c.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
    rows = [weights.matrix(p + "q", (H * (d + dr), W)), weights.matrix(p + "dkv", (r + dr, W))]
    c_norm = weights.vector(p + "dkv.norm", (r,))
    uk = weights.matrix(p + "uk", (H * d, r))
    uv = weights.matrix(p + "uv", (H * dv, r))
    if m.head_gate:
        rows.append(weights.matrix(p + "g", (H, W)))
    out = weights.matrix(p + "o", (W, H * dv))
    position = None
    if m.rot_dims:
        if m.yarn is not None:
            y = m.yarn
            inv_freq, amplitude = yarn_inv_freq(m.rot_dims, m.rot_base, y.factor, y.original, y.fast, y.slow)
        else:
            inv_freq, amplitude = leading_rotary_inv_freq(m.rot_dims, m.rot_base), 1.0
        position = RotaryEncoding(_on(weights, inv_freq), "interleaved", m.rot_dims, amplitude=amplitude)
    return LatentAttention(down=Linear(_cat(rows), p + "q|dkv" + ("|g" if m.head_gate else "")), q_norm_weight=None,
                           c_norm_weight=c_norm, up_q=None,
                           up_k=GroupedLinear(uk.reshape(H, d, r).transpose(1, 2).contiguous(), p + "uk"),
                           up_v=GroupedLinear(uv.reshape(H, dv, r).contiguous(), p + "uv"), out=Linear(out, p + "o"),
                           num_heads=H, dim=d, rot_dim=dr, value_dim=dv, q_rank=0, kv_rank=r, eps=c.eps,
                           softmax_scale=m.scale, position=position, act_dtype=act,
                           mask="window" if m.window else "full", span=m.window, head_gate=m.head_gate)


def _gated(weights: WeightSource, p: str, ff: int, W: int, act) -> DenseSwiGLU:
    gate_up = _cat([weights.matrix(p + "gate", (ff, W)), weights.matrix(p + "up", (ff, W))])
    return DenseSwiGLU(gate_up=Linear(gate_up, p + "gate|up"), down=Linear(weights.matrix(p + "down", (W, ff)), p + "down"),
                       act_dtype=act)


def _feed_forward(c: GisilixConfig, layer: GisilixLayer, p: str, weights: WeightSource, act):
    m, W = layer.mlp, c.width
    if m is None:
        return None
    if m.kind == "dense":
        return _gated(weights, p, m.ff, W, act)
    gate_up, down = [], []
    for e in range(m.experts):                 # file order: e0.gate, e0.up, e0.down, e1.gate, ...
        gate_up.append(_cat([weights.matrix(f"{p}e{e}.gate", (m.ff, W)), weights.matrix(f"{p}e{e}.up", (m.ff, W))]))
        down.append(weights.matrix(f"{p}e{e}.down", (W, m.ff)))
    router = weights.vector(p + "router", (m.experts, W), init="normal")
    bias = weights.vector(p + "router.b", (m.experts,), init="normal")
    shared = _gated(weights, p + "shared.", m.shared_ff, W, act) if m.shared_ff else None
    return MoESigmoidTopKGated(router=router, experts_gate_up=GroupedLinear(torch.stack(gate_up).contiguous(), p + "experts.gate|up"),
                               experts_down=GroupedLinear(torch.stack(down).contiguous(), p + "experts.down"),
                               top_k=m.top, shared=shared, act_dtype=act, router_bias=bias, scoring="softmax_chosen",
                               weights_on="output")


def build_gisilix(config: GisilixConfig, weights: WeightSource) -> DecoderModel:
    c, act, W = config, weights.compute_dtype, config.width
    embedding = weights.matrix("embed", (c.vocab, W))
    blocks, schedule = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        norm1 = _norm(weights, p + "norm1", W, c.eps)
        norm2 = None
        if layer.mlp is not None:
            norm2 = _norm(weights, p + "norm2", W, c.eps)
        elif weights.stored(p + "norm2"):         # a folder may keep the norm of a feed-forward that is not there:
            _norm(weights, p + "norm2", W, c.eps)  # asked for so that the folder checks clean, and not used
        if layer.type == "attention":
            mixer = _attention(c, layer, p + "mix.", weights, act)
        else:
            mixer = _latent(c, layer, p + "mix.", weights, act)
        ffn = _feed_forward(c, layer, p + "mlp.", weights, act)
        blocks.append(PreNormBlock(mixer_norm=norm1, mixer=mixer, ffn_norm=norm2, ffn=ffn, act_dtype=act))
        schedule.append(ScheduleEntry(i, cache_from=layer.kv_from))      # layers run once, in order: entry = layer
    final_norm = _norm(weights, "final.norm", W, c.eps)
    return DecoderModel(embedding=embedding, blocks=blocks, final_norm=final_norm, head=Linear(embedding, "embed"),
                        act_dtype=act, config=c, schedule=schedule)


register_architecture("Gisilix", GisilixConfig, build_gisilix)
