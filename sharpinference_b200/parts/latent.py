"""Latent attention: queries, keys and values all pass through low-rank latents, and only the key/value latent and
one small rotated key part are cached.

For the mixer's input ``h`` (``H`` heads; per head ``dim`` unrotated and ``rot`` rotated query/key elements, values of
``vdim``; latents of ``q_rank`` and ``rank`` elements):

    c_q = rms(W_dq h) * w_q                      q = W_uq c_q          per head [q_plain (dim) | q_rot (rot)]
    [c_raw | k_rot] = W_dkv h                    c = rms(c_raw) * w_c  k_rot is shared by all heads
    score_h(i, j) = (q_plain_h(i) . (W_uk_h c(j)) + R_i q_rot_h(i) . R_j k_rot(j)) * scale,   j <= i
    out = W_o concat_h( softmax_j(score_h) . (W_uv_h c(j)) )

with ``R_p`` the rotation of pairs ``(2i, 2i + 1)`` of the first ``rot_dims`` rotated elements by ``p * f_i``.

The unrotated score is ``(W_uk_h^T q_plain_h(i)) . c(j)``, and a head's value sum is ``W_uv_h (sum_j p_j c(j))``, so the
cache holds one row ``[c | R k_rot]`` per token for all heads (a cache group with one key/value head and keys-only
pages), the query of a head becomes ``[W_uk_h^T q_plain_h | R q_rot_h]``, the paged attention kernels run as for one
shared key/value head whose value is its key row, and ``W_uv_h`` expands the leading ``rank`` elements of a head's
output.  The two per-head products are grouped products with the heads as groups.  Norm sums, angles, scores and
softmax are float32; the latents, queries and the cache are rounded to the activation dtype where they enter a
product.

Variants, each a constructor argument: queries that come straight from the input (``q_rank = 0``: ``q = W_q h``, no
query latent; ``W_q`` then rides in the fused down projection); no rotated part (``rot_dim = 0``); a sliding window
instead of the whole past (``mask="window"``, ``span``); a gate per head, ``out_h *= sigmoid(W_g h)_h``, whose ``H``
rows are the last rows of the fused projection (``head_gate``); a rotation whose cosines and sines carry an amplitude
(``RotaryEncoding(amplitude=...)``, as stretched frequencies bring one).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import CacheSpec, LayerSlot, Mixer, PositionEncoding, StepContext, register_part
from .attention import PagedAttentionPlanner
from .linear import GroupedLinear, Linear


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, *, down: Linear, q_norm_weight: Optional[torch.Tensor], c_norm_weight: torch.Tensor,
                 up_q: Optional[Linear], up_k: GroupedLinear, up_v: GroupedLinear, out: Linear, num_heads: int, dim: int,
                 rot_dim: int, value_dim: int, q_rank: int, kv_rank: int, eps: float, softmax_scale: float,
                 position: Optional[PositionEncoding] = None, act_dtype: torch.dtype = torch.bfloat16,
                 mask: str = "full", span: int = 0, head_gate: bool = False):
        """``down``: the fused down projections, rows ``[W_dq (q_rank) | W_dkv (kv_rank + rot_dim)]``; with
        ``q_rank = 0`` (``up_q`` and ``q_norm_weight`` None) the queries themselves lead it:
        ``[W_q (heads * (dim + rot_dim)) | W_dkv (kv_rank + rot_dim)]``; with ``head_gate`` the gate's ``heads`` rows
        follow.  ``up_k``: per head ``W_uk_h^T`` as a group ``[kv_rank, dim]`` (it maps a head's unrotated query into the
        latent); ``up_v``: per head ``W_uv_h [value_dim, kv_rank]``.  ``position``: a rotary encoding of neighbouring
        pairs over the first ``rot_dims`` of the ``rot_dim`` rotated elements (None: no rotation).  ``mask``:
        ``"full"`` or ``"window"`` of ``span`` positions, the query's own included."""
        H = num_heads
        if mask not in ("full", "window") or (mask == "window" and span <= 0):
            raise ValueError(f"mask '{mask}' must be full or a window of a positive span (found {span})")
        lead = q_rank if q_rank > 0 else H * (dim + rot_dim)
        if down.out_features != lead + kv_rank + rot_dim + (H if head_gate else 0):
            raise ValueError(f"the fused down projection has {down.out_features} rows, expected "
                             f"{lead + kv_rank + rot_dim + (H if head_gate else 0)} (queries or their latent {lead}, "
                             f"key/value latent {kv_rank}, rotated key {rot_dim}, gate {H if head_gate else 0})")
        if (q_rank > 0) != (up_q is not None) or (q_rank > 0) != (q_norm_weight is not None):
            raise ValueError("a query latent (q_rank > 0) comes with its up projection and norm weight, and only then")
        if up_q is not None and (up_q.in_features != q_rank or up_q.out_features != H * (dim + rot_dim)):
            raise ValueError(f"the query up projection is [{up_q.out_features}, {up_q.in_features}], expected "
                             f"[{H * (dim + rot_dim)}, {q_rank}]")
        if (up_k.num_groups, up_k.out_features, up_k.in_features) != (H, kv_rank, dim):
            raise ValueError(f"up_k must hold [{H}, {kv_rank}, {dim}] (a head's key projection, transposed)")
        if (up_v.num_groups, up_v.out_features, up_v.in_features) != (H, value_dim, kv_rank):
            raise ValueError(f"up_v must hold [{H}, {value_dim}, {kv_rank}]")
        if out.in_features != H * value_dim:
            raise ValueError(f"output projection reads {out.in_features} columns, expected {H * value_dim}")
        if (q_norm_weight is not None and q_norm_weight.numel() != q_rank) or c_norm_weight.numel() != kv_rank:
            raise ValueError("the latents' norm weights disagree with q_rank or kv_rank")
        self.inv_freq, self.rot_dims, self.rot_amplitude = None, 0, 1.0
        self.head_gate, self._lead = bool(head_gate), lead
        if position is not None and rot_dim:
            self.rot_amplitude = float(getattr(position, "amplitude", 1.0))
            rot = position.rotary()
            if rot is None or rot[1] != "interleaved":
                raise ValueError("latent attention rotates neighbouring pairs (a rotary encoding, interleaved)")
            self.rot_dims = position.rot_dims if getattr(position, "rot_dims", None) is not None else rot_dim
            if self.rot_dims > rot_dim or self.rot_dims % 2 or rot[0].numel() != self.rot_dims // 2:
                raise ValueError(f"{self.rot_dims} rotated elements do not fit the rotated part of {rot_dim}")
            self.inv_freq = rot[0] if self.rot_dims else None
        self.down, self.up_q, self.up_k, self.up_v, self.out = down, up_q, up_k, up_v, out
        self.q_norm_weight, self.c_norm_weight = q_norm_weight, c_norm_weight
        self.num_heads, self.dim, self.rot_dim, self.value_dim = H, dim, rot_dim, value_dim
        self.q_rank, self.kv_rank, self.eps = q_rank, kv_rank, float(eps)
        self.softmax_scale, self.act_dtype = float(softmax_scale), act_dtype
        # one cached row a token: [c | k_rot], padded to what the attention kernels take as a head size
        D = kv_rank + rot_dim
        if D > 1024:
            raise ValueError(f"kv_rank + rot_dim = {kv_rank + rot_dim} exceeds the largest head size of the attention "
                             f"kernels (1024; the tensor-core kernels take rows of up to 512, longer ones the general kernel)")
        D = (D + 15) // 16 * 16                   # a multiple of 16: the size the tensor-core kernels take
        self.head_dim = D
        self.cache_spec = CacheSpec(mask, span if mask != "full" else 0, 1, D, planes=1)

    def step_planner(self, page_size: int):
        return PagedAttentionPlanner(ops.KEYS_ATTENTION_TILE)

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        T, H, D, act = ctx.num_tokens, self.num_heads, self.head_dim, self.act_dtype
        table = ctx.block_tables[slot.group]
        mask_kind = ops.MASK_WINDOW if self.cache_spec.kind == "window" else ops.MASK_FULL
        mask_span = max(self.cache_spec.span, 1)
        down = self.down(h)                                    # [T, (q_rank or H (dim + rot)) + kv_rank + rot (+ H)] float32
        tail = self.kv_rank + self.rot_dim
        gate = down[:, self._lead + tail:] if self.head_gate else None
        if self.q_rank > 0:
            cq = ops.latent_down_post(down[:, : self._lead + tail], q_rank=self.q_rank, rank=self.kv_rank, rot=self.rot_dim,
                                      rot_dims=self.rot_dims, q_norm_weight=self.q_norm_weight,
                                      c_norm_weight=self.c_norm_weight, eps=self.eps, positions=ctx.positions,
                                      row_req=ctx.row_request, block_table=table, inv_freq=self.inv_freq, kv_layer=slot.kv,
                                      page_size=slot.page_size, write_kv=slot.writes_cache,
                                      rot_amplitude=self.rot_amplitude)
            q = self.up_q(cq)                                                 # [T, H (dim + rot)] float32
        else:                                                                 # the queries lead the fused product
            ops.latent_down_post(down[:, self._lead: self._lead + tail], q_rank=0, rank=self.kv_rank, rot=self.rot_dim,
                                 rot_dims=self.rot_dims, q_norm_weight=None, c_norm_weight=self.c_norm_weight,
                                 eps=self.eps, positions=ctx.positions, row_req=ctx.row_request, block_table=table,
                                 inv_freq=self.inv_freq, kv_layer=slot.kv, page_size=slot.page_size,
                                 write_kv=slot.writes_cache, rot_amplitude=self.rot_amplitude)
            q = down[:, : self._lead]
        q_plain = ops.head_major(q, heads=H, stride=self.dim + self.rot_dim, col0=0, n=self.dim, out_dtype=act)
        qa = self.up_k.per_group(q_plain, T)                                  # [H T, kv_rank] float32
        qj = ops.latent_q_join(qa, q, ctx.positions, self.inv_freq, heads=H, dim=self.dim, rank=self.kv_rank,
                               rot=self.rot_dim, rot_dims=self.rot_dims, D=D, out_dtype=act,
                               rot_amplitude=self.rot_amplitude)
        dv = (self.kv_rank + 15) // 16 * 16
        if ops.keys_attention_supported(act, D, dv) and slot.kv.shape[1] == 1:
            # the tensor-core kernels for keys-only pages: the value sum is taken over the latent's columns only
            plan = ctx.plans[("paged_attention", ops.KEYS_ATTENTION_TILE)]
            o = torch.empty((T, H * dv), dtype=torch.bfloat16, device=h.device)
            kw = dict(nq=H, nkv=1, d=D, dv=dv, page_size=slot.page_size, mask_kind=mask_kind, mask_span=mask_span,
                      scale=self.softmax_scale)
            if plan.num_tiles:
                ops.attention_keys_prefill(qj, slot.kv, table, plan.tiles, o, **kw)
            if plan.num_decode_rows:
                ops.attention_keys_decode(qj, slot.kv, table, ctx.row_request, ctx.positions, o, rows=plan.decode_rows,
                                          num_rows=plan.num_decode_rows, max_context=ctx.max_context, **kw)
            o_lat = ops.head_major(o, heads=H, stride=dv, col0=0, n=self.kv_rank, out_dtype=act)
        else:
            o = ops.paged_attention_generic(qj, slot.kv, table, ctx.row_request, ctx.positions, nq=H, nkv=1, d=D,
                                            page_size=slot.page_size, mask_kind=mask_kind, mask_span=mask_span,
                                            scale=self.softmax_scale)
            o_lat = ops.head_major(o, heads=H, stride=D, col0=0, n=self.kv_rank, out_dtype=act)
        v = self.up_v.per_group(o_lat, T)                                     # [H T, value_dim] float32
        return self.out(ops.head_minor(v, heads=H, out_dtype=act, gate=gate))
