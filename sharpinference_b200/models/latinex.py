"""The Latinex architecture, put together from parts, and its tensor names.

A pre-norm decoder (``x += mixer(norm1(x))``, then ``x += ff(norm2(x))``) whose norms are the element-wise ``tanh``
norm (:class:`DynamicTanh`), whose embedding rows are multiplied by a constant, and whose layers (``config.layers[i]``,
every layer with sizes of its own) have one of three mixers:

* ``latent_attention``: :class:`LatentAttention` (queries through a normed latent; one normed key/value latent and one
  rotated key part per token are all that is cached; causal);
* ``attention``: :class:`PagedAttention` with grouped key heads that are also the values, biases on q and k, no
  rotation, a learned bias by distance, a sliding window that keeps the first positions, and a sigmoid gate on the
  heads;
* ``mamba2``: :class:`StateSpaceDualityMixer`.

The feed-forward, where a layer has one, is a sigmoid-routed mixture of gated experts whose chosen scores multiply
the experts' inputs, with a shared expert (:class:`MoESigmoidTop1` when a row uses one expert, else
:class:`MoESigmoidTopKGated`).  The logits are ``head x * logit_scale``.

Tensor names (linear weights ``[out, in]``): ``embed``, ``final.norm`` (+ ``.b``, ``.alpha``), ``head``; per layer
``l<i>.norm{1,2}`` (+ ``.b``, ``.alpha``), ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``,
``l<i>.mlp.shared.{gate,up,down}``; for latent_attention ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}``; for
attention ``l<i>.mix.{q,q.b,k,k.b,rel,g,o}``; for mamba2 ``l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}``.
"""
from __future__ import annotations

import torch

from ..config.latinex import LatinexConfig, LatinexLayer
from ..parts import (DenseSwiGLU, DynamicTanh, GroupedLinear, LatentAttention, Linear, MoESigmoidTop1,
                     MoESigmoidTopKGated, PagedAttention, PreNormBlock, RotaryEncoding, StateSpaceDualityMixer,
                     distance_bias_table, leading_rotary_inv_freq, ssd_projection_order)
from ..registry import register_architecture
from ..weights.source import WeightSource
from .model import DecoderModel
from .notedra import _cat


def _on(weights: WeightSource, t: torch.Tensor) -> torch.Tensor:
    return t if weights.device.type == "meta" else t.to(weights.device)


def _norm(weights: WeightSource, name: str, width: int) -> DynamicTanh:
    return DynamicTanh(weights.vector(name, (width,)), weights.vector(name + ".b", (width,), init="normal"),
                       weights.vector(name + ".alpha", (), init="norm"))


def _latent(c: LatinexConfig, m: LatinexLayer, p: str, weights: WeightSource, act) -> LatentAttention:
    W, H, d, dr, dv, r = c.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank
    down = _cat([weights.matrix(p + "dq", (m.q_rank, W)), weights.matrix(p + "dkv", (r + dr, W))])
    q_norm, c_norm = weights.vector(p + "dq.norm", (m.q_rank,)), weights.vector(p + "dkv.norm", (r,))
    up_q = weights.matrix(p + "uq", (H * (d + dr), m.q_rank))
    uk = weights.matrix(p + "uk", (H * d, r))
    uv = weights.matrix(p + "uv", (H * dv, r))
    out = weights.matrix(p + "o", (W, H * dv))
    position = (RotaryEncoding(_on(weights, leading_rotary_inv_freq(m.rot_dims, m.rot_base)), "interleaved", m.rot_dims)
                if m.rot_dims else None)
    return LatentAttention(down=Linear(down, p + "dq|dkv"), q_norm_weight=q_norm, c_norm_weight=c_norm,
                           up_q=Linear(up_q, p + "uq"),
                           up_k=GroupedLinear(uk.reshape(H, d, r).transpose(1, 2).contiguous(), p + "uk"),
                           up_v=GroupedLinear(uv.reshape(H, dv, r).contiguous(), p + "uv"), out=Linear(out, p + "o"),
                           num_heads=H, dim=d, rot_dim=dr, value_dim=dv, q_rank=m.q_rank, kv_rank=r, eps=c.eps,
                           softmax_scale=m.scale, position=position, act_dtype=act)


def _attention(c: LatinexConfig, m: LatinexLayer, p: str, weights: WeightSource, act) -> PagedAttention:
    W, H, G, d = c.width, m.heads, m.kv_heads, m.dim
    qk = _cat([weights.matrix(p + "q", (H * d, W)), weights.matrix(p + "k", (G * d, W))])
    bias = torch.cat([weights.vector(p + "q.b", (H * d,), init="normal"),
                      weights.vector(p + "k.b", (G * d,), init="normal")]).contiguous()
    rows = m.bias_buckets or (weights.shape_of(p + "rel") or (0,))[0]
    if rows < 2:
        raise ValueError(f"{p}rel: neither the configuration (bias_buckets) nor a stored tensor gives the number of "
                         f"distance buckets")
    rel = weights.vector(p + "rel", (rows, H), init="normal")
    gate = Linear(weights.matrix(p + "g", (H * d, W)), p + "g")
    out = Linear(weights.matrix(p + "o", (W, H * d)), p + "o")
    return PagedAttention(qkv=Linear(qk, p + "q|k", bias=bias), out=out, num_heads=H, num_kv_heads=G, head_dim=d,
                          mask="window" if m.window else "full", span=m.window, position=None, softmax_scale=m.scale,
                          act_dtype=act, values_are_keys=True, keep_first=m.keep_first,
                          distance_bias=distance_bias_table(rel, m.bias_max), gate=gate)


def _mamba2(c: LatinexConfig, m: LatinexLayer, p: str, weights: WeightSource, act) -> StateSpaceDualityMixer:
    W, inner, bc = c.width, m.heads * m.vdim, m.groups * m.state
    w_in = weights.matrix(p + "in", (2 * inner + 2 * bc + m.heads, W))
    if weights.device.type != "meta":          # stored [z | x | B | C | dt]; the mixer reads [x | B | C | z | dt]
        w_in = w_in[ssd_projection_order(m.heads, m.vdim, m.state, m.groups).to(w_in.device)].contiguous()
    return StateSpaceDualityMixer(
        in_proj=Linear(w_in, p + "in"),
        conv_weight=weights.vector(p + "conv", (inner + 2 * bc, m.conv), init="normal"),
        conv_bias=weights.vector(p + "conv.b", (inner + 2 * bc,), init="normal"),
        dt_bias=weights.vector(p + "dt_bias", (m.heads,), init="normal"),
        a_log=weights.vector(p + "A_log", (m.heads,), init="normal"),
        d_skip=weights.vector(p + "D", (m.heads,)),
        norm_weight=weights.vector(p + "norm", (inner,)),
        out=Linear(weights.matrix(p + "o", (W, inner)), p + "o"),
        heads=m.heads, value_dim=m.vdim, states=m.state, groups=m.groups, taps=m.conv, norm_groups=m.norm_groups,
        eps=c.eps, act_dtype=act)


def _mixture(c: LatinexConfig, layer: LatinexLayer, p: str, weights: WeightSource, act):
    m, W = layer.mlp, c.width
    if m is None:
        return None
    gate_up, down = [], []
    for e in range(m.experts):                 # file order: e0.gate, e0.up, e0.down, e1.gate, ...
        gate_up.append(_cat([weights.matrix(f"{p}e{e}.gate", (m.ff, W)), weights.matrix(f"{p}e{e}.up", (m.ff, W))]))
        down.append(weights.matrix(f"{p}e{e}.down", (W, m.ff)))
    router = weights.vector(p + "router", (m.experts, W), init="normal")
    shared = None
    if m.shared_ff:
        shared = DenseSwiGLU(gate_up=Linear(_cat([weights.matrix(p + "shared.gate", (m.shared_ff, W)),
                                                   weights.matrix(p + "shared.up", (m.shared_ff, W))]), p + "shared.gate|up"),
                             down=Linear(weights.matrix(p + "shared.down", (W, m.shared_ff)), p + "shared.down"),
                             act_dtype=act)
    experts_gate_up = GroupedLinear(torch.stack(gate_up).contiguous(), p + "experts.gate|up")
    experts_down = GroupedLinear(torch.stack(down).contiguous(), p + "experts.down")
    if m.top == 1:
        return MoESigmoidTop1(router=router, experts_gate_up=experts_gate_up, experts_down=experts_down, shared=shared,
                              act_dtype=act)
    return MoESigmoidTopKGated(router=router, experts_gate_up=experts_gate_up, experts_down=experts_down, top_k=m.top,
                               shared=shared, act_dtype=act)


_MIXERS = {"latent_attention": _latent, "attention": _attention, "mamba2": _mamba2}


def build_latinex(config: LatinexConfig, weights: WeightSource) -> DecoderModel:
    c, act, W = config, weights.compute_dtype, config.width
    embedding = weights.matrix("embed", (c.vocab, W))
    blocks = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        norm1, norm2 = _norm(weights, p + "norm1", W), _norm(weights, p + "norm2", W)
        mixer = _MIXERS[layer.type](c, layer, p + "mix.", weights, act)
        ffn = _mixture(c, layer, p + "mlp.", weights, act)
        blocks.append(PreNormBlock(mixer_norm=norm1, mixer=mixer, ffn_norm=norm2, ffn=ffn, act_dtype=act))
    final_norm = _norm(weights, "final.norm", W)
    head = Linear(weights.matrix("head", (c.vocab, W)), "head")
    return DecoderModel(embedding=embedding, blocks=blocks, final_norm=final_norm, head=head, act_dtype=act, config=c,
                        logit_scale=c.logit_scale, embedding_scale=c.embedding_scale)


register_architecture("Latinex", LatinexConfig, build_latinex)
