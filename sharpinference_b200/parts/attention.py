"""Grouped-query attention over the paged cache: the mixer of every Llama 4 layer.

Order of operations for the step's rows (reference: src/SharpInference.Engine/ForwardPass.cs:1576-1690):
fused Q|K|V projection; rotary encoding of q and k; weightless L2 norm of q and k per head
(after the rotation); temperature factor on q; k and v into the request's pages; attention of
every row over the positions its mask lets it see; output projection.  Query head ``h`` reads
kv head ``h // (heads / kv_heads)``; scores are ``q . k / sqrt(d)``.

What the reference lacks is a parameter here: the mask (``full``, ``chunk`` of C positions,
``window`` of W positions), the temperature factor
``1 + attn_scale * ln(1 + floor((pos + 1) / floor_scale))``, the score factor (``softmax_scale``), and a value
size that differs from the key size (``value_dim``).

Further parameters that other designs use: values that are the keys themselves (``values_are_keys``: no value
projection, and a page holds keys only), a sliding window that keeps a sequence's first positions visible
(``keep_first``), a learned number added to every score by the distance between query and key
(``distance_bias``, a table by distance built with :func:`distance_bias_table`), and a sigmoid gate on the
concatenated heads before the output projection (``gate``).

And: a q/k norm over the whole projection (``wide_norm``: all heads of q side by side are divided by their common
root mean square and multiplied by a weight of that size, and so is k), a cap on the scaled score
(``softcap``: ``s -> softcap * tanh(s / softcap)``), a learned sink per head whose exponential joins the softmax's
denominator without a key or a value (``sinks``), a layer that brings queries only and reads the keys and values
another layer cached (``borrows_kv``), and the gate's rows riding in the fused projection (``gate_fused``).

Unequal key and value sizes: the kernels and the pages know one head size, so the part pads both to a common
size D once, when it is built: zero rows in the fused projection (a padded q, k or v element is an exact zero),
zero columns in the output projection.  Zeros change neither a score nor a rotation (the padded pairs get
frequency 0) nor an output, and the q/k norm divides its sum of squares by the key size, not by D.
"""
from __future__ import annotations

import math
from typing import Hashable, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import ops
from .base import (CacheSpec, LayerSlot, Mixer, Norm, PositionEncoding, StepContext, StepPlanData, StepPlanner,
                   register_part)
from .linear import Linear

_MASK_CODE = {"full": ops.MASK_FULL, "chunk": ops.MASK_CHUNK, "window": ops.MASK_WINDOW}
_PAIRING_CODE = {"interleaved": ops.ROPE_INTERLEAVED, "halves": ops.ROPE_HALVES}


class PagedAttentionPlanner(StepPlanner):
    """How the attention kernels split a step's rows: portions of prompts become tiles of up to ``tile_rows``
    consecutive rows of one request (int32 ``tiles`` [n, 4]: first row, rows, first position, request index),
    which the prompt kernels serve one CTA (per head) each; entries of up to ``DECODE_ROWS_UP_TO`` rows are
    served row by row by the split-KV kernel (int32 ``decode_rows`` [m]; left out when every row of the step
    is such a row).  ``decode_keys`` bounds the sum of position + 1 over the single rows: the split-KV launch
    holds about as many CTAs as these rows have 256-key splits together."""

    DECODE_ROWS_UP_TO = 4

    def __init__(self, tile_rows: int):
        self.tile_rows = int(tile_rows)
        self.key = ("paged_attention", self.tile_rows)

    @staticmethod
    def keys_bucket(keys: int, rows: int = 1) -> int:
        """``keys`` rounded up to a multiple of a power of two: a sixteenth to an eighth of ``keys``, and at
        least 256 keys a row, so that a batch that gains a key a row each step stays in its bucket for 256
        steps or more (a new bucket means a step run eagerly and a graph captured)."""
        step = 1 << max((256 * max(rows, 1) - 1).bit_length(), keys.bit_length() - 4)
        return (keys + step - 1) // step * step

    def bucket(self, starts: Sequence[int], lengths: Sequence[int]) -> Hashable:
        return self.keys_bucket(sum(s + 1 for s in starts), len(starts))

    def plan(self, starts: Sequence[int], lengths: Sequence[int], bucket: Hashable = None) -> StepPlanData:
        tiles, decode_rows = [], []
        keys = 0                         # sum of position + 1 over the single rows
        r = 0
        for b, (start, n) in enumerate(zip(starts, lengths)):
            if n <= self.DECODE_ROWS_UP_TO:
                decode_rows.extend(range(r, r + n))
                keys += n * start + n * (n + 1) // 2
            else:
                for t0 in range(0, n, self.tile_rows):
                    tiles.append((r + t0, min(self.tile_rows, n - t0), start + t0, b))
            r += n
        all_single = len(decode_rows) == r
        return StepPlanData(
            arrays={"tiles": np.asarray(tiles, dtype=np.int32).reshape(-1, 4),
                    "decode_rows": np.asarray([] if all_single else decode_rows, dtype=np.int32)},
            values={"num_tiles": len(tiles), "num_decode_rows": len(decode_rows), "tile_rows": self.tile_rows,
                    "decode_keys": keys if bucket is None else int(bucket)})


def distance_bucket(n: int, rows: int, far: int) -> int:
    """The row of a distance table with ``rows`` rows for the distance ``n >= 0``: distances below ``rows / 2`` have
    a row each, the rows above are spread logarithmically up to the distance ``far``, beyond which the last row
    stands: ``min(rows - 1, half + floor(ln(n / half) / ln(far / half) * (rows - half)))``, in float64."""
    half = rows // 2
    if n < half:
        return n
    if far <= half:
        return rows - 1
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias_table(rel: torch.Tensor, far: int) -> torch.Tensor:
    """``rel [rows, heads]`` (a learned number per distance bucket and head) laid out by distance: float32
    ``[n + 1, heads]`` whose row ``d`` is the bucket of distance ``d`` and whose last row holds for every larger
    distance (the attention kernels read ``min(distance, n)``).  ``n`` is the first distance whose bucket is the
    last row, so the table is never longer than ``far + 1`` rows."""
    rows = rel.shape[0]
    buckets = []
    for n in range(max(int(far), rows) + 1):
        buckets.append(distance_bucket(n, rows, int(far)))
        if buckets[-1] == rows - 1:
            break
    if rel.device.type == "meta":
        return torch.empty((len(buckets), rel.shape[1]), dtype=torch.float32, device="meta")
    index = torch.tensor(buckets, dtype=torch.long, device=rel.device)
    return rel.to(torch.float32)[index].contiguous()


def _pad_head_rows(block: torch.Tensor, heads: int, size: int, D: int) -> torch.Tensor:
    """``block [heads * size, ...]`` with zero rows behind each head up to ``D`` rows a head."""
    if size == D:
        return block
    wide = torch.zeros((heads, D) + tuple(block.shape[1:]), dtype=block.dtype, device=block.device)
    wide[:, :size] = block.reshape((heads, size) + tuple(block.shape[1:]))
    return wide.reshape((heads * D,) + tuple(block.shape[1:]))


def _pad_projections(qkv: Linear, out: Linear, nq: int, nkv: int, dk: int, dv: int, D: int):
    """The fused q|k|v projection and the output projection with every head padded to ``D`` elements: zero rows
    (and zero bias entries) behind each head of q, k and v, zero columns behind each head in ``out``."""
    def pad_rows(block: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        return _pad_head_rows(block, heads, size, D)

    def pad_qkv(t: torch.Tensor) -> torch.Tensor:
        q, k, v = t[: nq * dk], t[nq * dk: (nq + nkv) * dk], t[(nq + nkv) * dk:]
        return torch.cat([pad_rows(q, nq, dk), pad_rows(k, nkv, dk), pad_rows(v, nkv, dv)]).contiguous()

    w = out.weight
    wide = torch.zeros((w.shape[0], nq, D), dtype=w.dtype, device=w.device)
    wide[:, :, :dv] = w.reshape(w.shape[0], nq, dv)
    return (Linear(pad_qkv(qkv.weight), qkv.name, stream_rows=qkv.stream_rows,
                   bias=None if qkv.bias is None else pad_qkv(qkv.bias)),
            Linear(wide.reshape(w.shape[0], nq * D).contiguous(), out.name, stream_rows=out.stream_rows, bias=out.bias,
                   split_add_rows=out.split_add_rows))


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    def __init__(self, *, qkv: Linear, out: Linear, num_heads: int, num_kv_heads: int, head_dim: int,
                 mask: str = "full", span: int = 0, position: Optional[PositionEncoding] = None,
                 qk_norm: Optional[Norm] = None, qk_norm_first: bool = False,
                 temperature: Optional[Tuple[float, float]] = None,
                 softmax_scale: Optional[float] = None, act_dtype: torch.dtype = torch.bfloat16,
                 value_dim: Optional[int] = None, value_position: Optional[PositionEncoding] = None,
                 k_norm: Optional[Norm] = None, values_are_keys: bool = False, keep_first: int = 0,
                 distance_bias: Optional[torch.Tensor] = None, gate: Optional[Linear] = None,
                 wide_norm: Optional[Tuple[torch.Tensor, Optional[torch.Tensor], float]] = None,
                 softcap: float = 0.0, sinks: Optional[torch.Tensor] = None, borrows_kv: bool = False,
                 gate_fused: bool = False):
        """``qk_norm``: any :class:`Norm` over the head size, applied to every head of q and k; after the
        position encoding (Llama 4's order) unless ``qk_norm_first``.  The weightless L2 norm after a rotation
        runs inside the kernel that rotates and writes the cache; every other combination applies the norm as
        a launch of its own on q and on k.  ``value_dim``: the size of a value head when it is not ``head_dim``
        (``qkv`` then has ``heads * head_dim + kv_heads * (head_dim + value_dim)`` rows and ``out`` reads
        ``heads * value_dim`` columns).

        ``value_position``: a rotary encoding by which every value is turned by its own position before it is
        cached; each head's output (the weighted sum of the values) is turned back by the query's position.
        ``k_norm``: the norm of k when it is not the one of q (``qk_norm``).  A rotation of only the leading
        elements of a head (``RotaryEncoding(rot_dims=...)``), rotated values, and a weighted norm before the
        rotation together with unequal key and value sizes run in the general form of the fused kernel
        (``sharpi_qkv_post_rot``): norm first (``qk_norm_first``), then the rotation, then the cache write.

        ``values_are_keys``: ``qkv`` holds q and k only, a page holds keys only and attention sums the keys it
        weighted.  ``keep_first`` (window mask): the first positions of a sequence stay visible.
        ``distance_bias``: float32 ``[n + 1, heads]`` added to the scaled score by distance
        (:func:`distance_bias_table`).  ``gate``: a projection of the mixer's input whose sigmoid multiplies the
        concatenated heads.  A layer with kept positions or a distance bias, or with keys-only pages, runs the
        general attention kernel.

        ``wide_norm = (q_weight [heads * head_dim], k_weight [kv_heads * head_dim] or None, eps)``: the q/k norm over
        the whole projection, in one kernel with the temperature factor and the cache write (no position encoding
        then).  ``softcap``, ``sinks`` (float32 ``[heads]``): see the module text.  ``borrows_kv``: ``qkv`` holds the
        query rows only, and every schedule entry of the layer reads another entry's cache (``cache_from``); built
        for the whole-projection path.  ``gate_fused``: the gate's ``heads * value_dim`` rows are the last rows of
        ``qkv`` instead of a projection of their own."""
        self.softcap, self.sinks = float(softcap), sinks
        self.borrows_kv, self.gate_fused, self.wide_norm = bool(borrows_kv), bool(gate_fused), None
        if sinks is not None and sinks.numel() != num_heads:
            raise ValueError(f"sinks has {sinks.numel()} entries for {num_heads} heads")
        if (self.softcap > 0.0 or sinks is not None) and values_are_keys:
            raise ValueError("a score cap or sinks are not built for attention whose values are its keys")
        if position is not None and getattr(position, "amplitude", 1.0) != 1.0:
            raise ValueError("a rotation with an amplitude is not built for this mixer")
        if wide_norm is not None or borrows_kv or gate_fused:
            self._init_wide(qkv, out, num_heads, num_kv_heads, head_dim, mask, span, position, qk_norm, temperature,
                            softmax_scale, act_dtype, value_dim, value_position, values_are_keys, keep_first,
                            distance_bias, gate, wide_norm)
            return
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"heads ({num_heads}) must be a multiple of kv heads ({num_kv_heads})")
        key_dim = head_dim
        value_dim = key_dim if value_dim is None else int(value_dim)
        if key_dim <= 0 or value_dim <= 0 or key_dim % 2 != 0 or max(key_dim, value_dim) > 512:
            raise ValueError(f"head sizes {key_dim} (keys) and {value_dim} (values) are not supported: the key size "
                             f"must be even and both at most 512")
        if values_are_keys:
            if value_dim != key_dim or value_position is not None:
                raise ValueError("values that are the keys have the keys' size and no rotation of their own")
            if position is not None and getattr(position, "rot_dims", None) is not None:
                raise ValueError("values that are the keys are not built with a rotation of a head's leading elements")
        if keep_first and mask != "window":
            raise ValueError("kept first positions belong to the window mask")
        if distance_bias is not None and (distance_bias.dim() != 2 or distance_bias.shape[1] != num_heads):
            raise ValueError(f"the distance bias is {tuple(distance_bias.shape)}, expected [distances, {num_heads}]")
        if gate is not None and gate.out_features != num_heads * value_dim:
            raise ValueError(f"the gate has {gate.out_features} rows, expected heads * value_dim = {num_heads * value_dim}")
        v_rows = 0 if values_are_keys else num_kv_heads * value_dim
        if qkv.out_features != (num_heads + num_kv_heads) * key_dim + v_rows:
            raise ValueError(f"fused qkv weight has {qkv.out_features} rows, expected (heads + kv_heads) * head_dim + "
                             f"kv_heads * value_dim = {(num_heads + num_kv_heads) * key_dim + v_rows}")
        if out.in_features != num_heads * value_dim:
            raise ValueError(f"output projection reads {out.in_features} columns, expected {num_heads * value_dim}")
        self.key_dim, self.value_dim = key_dim, value_dim
        self.value_position, self.k_norm = value_position, (k_norm if k_norm is not None else qk_norm)
        rot = position.rotary() if position is not None else None
        self._general = (value_position is not None or getattr(position, "rot_dims", None) is not None
                         or (value_dim != key_dim and (qk_norm_first or (rot is not None and rot[1] == "halves"))))
        if self._general:
            if position is not None and rot is None:
                raise ValueError("the general fused kernel takes rotary (or no) position encodings only")
            if qk_norm is not None and not qk_norm_first:
                raise ValueError("the general fused kernel norms q and k before the rotation (qk_norm_first=True)")
            if value_position is not None and value_position.rotary() is None:
                raise ValueError("values can only be turned by a rotary encoding")
            if value_position is not None and rot is not None and value_position.rotary()[1] != rot[1]:
                raise ValueError("keys and values must pair their elements the same way")
            self._rot_dims = 0 if rot is None else (position.rot_dims if position.rot_dims is not None else key_dim)
            self._v_rot_dims = 0
            if value_position is not None:
                vd = getattr(value_position, "rot_dims", None)
                self._v_rot_dims = vd if vd is not None else value_dim
                if self._v_rot_dims > value_dim:
                    raise ValueError(f"{self._v_rot_dims} rotated value elements exceed the value size {value_dim}")
            if self._rot_dims > key_dim:
                raise ValueError(f"{self._rot_dims} rotated elements exceed the key size {key_dim}")
            if value_dim != key_dim:
                head_dim = max(key_dim, value_dim)
                head_dim = (head_dim + 15) // 16 * 16 if head_dim <= 128 else head_dim + (head_dim & 1)
                qkv, out = _pad_projections(qkv, out, num_heads, num_kv_heads, key_dim, value_dim, head_dim)
        elif value_dim != key_dim:
            head_dim = max(key_dim, value_dim)
            head_dim = (head_dim + 15) // 16 * 16 if head_dim <= 128 else head_dim + (head_dim & 1)
            if qk_norm is not None and not (getattr(qk_norm, "fuses_into_rotation", False) and not qk_norm_first):
                raise ValueError("with unequal key and value sizes only the weightless q/k norm after the position "
                                 "encoding is built (a norm of its own launch would average over the padded size)")
            if position is not None and position.rotary() is None:
                raise ValueError("with unequal key and value sizes only rotary (or no) position encodings are built")
            qkv, out = _pad_projections(qkv, out, num_heads, num_kv_heads, key_dim, value_dim, head_dim)
            if position is not None:
                inv_freq, pairing = position.rotary()
                if pairing != "interleaved":
                    raise ValueError("with unequal key and value sizes the rotation must pair neighbours")
                wide = torch.zeros(head_dim // 2, dtype=inv_freq.dtype, device=inv_freq.device)
                wide[: key_dim // 2] = inv_freq
                position = type(position)(wide, pairing)
        self.qkv, self.out = qkv, out
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.cache_spec = CacheSpec(mask, span if mask != "full" else 0, num_kv_heads, head_dim,
                                    planes=1 if values_are_keys else 2, keep_first=int(keep_first))
        self.values_are_keys, self.keep_first, self.distance_bias, self.gate = values_are_keys, int(keep_first), distance_bias, gate
        # what the tensor-core attention kernels do not take runs the general kernel
        self._general_attention = values_are_keys or self.keep_first > 0 or distance_bias is not None
        self.position = position
        self.qk_norm = qk_norm
        self.qk_norm_first = bool(qk_norm_first)
        rotary = position is not None and position.rotary() is not None
        # the fused kernel's order is rotation, weightless norm, temperature
        self._norm_fused = (qk_norm is not None and not qk_norm_first and not self._general
                            and getattr(qk_norm, "fuses_into_rotation", False))
        self._ones = None
        if qk_norm is not None and not self._norm_fused and not qk_norm_first and rotary:
            raise ValueError(f"a q/k norm of kind '{qk_norm.kind}' after a rotary encoding is not built (only the "
                             f"weightless L2 norm fuses into the rotation kernel): place it before the position "
                             f"encoding (qk_norm_first=True) or use an encoding that edits q and k itself")
        self.temperature = temperature          # (attn_scale, floor_scale) or None
        self.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(key_dim)
        self.act_dtype = act_dtype
        # an encoding that edits q and k itself may look at the step's host-side lists: no graph then
        self.graph_safe = position is None or position.rotary() is not None

    def _init_wide(self, qkv, out, num_heads, num_kv_heads, head_dim, mask, span, position, qk_norm, temperature,
                   softmax_scale, act_dtype, value_dim, value_position, values_are_keys, keep_first, distance_bias, gate,
                   wide_norm) -> None:
        """The layer whose q/k norm runs over the whole projection."""
        nq, nkv, dk = num_heads, num_kv_heads, head_dim
        dv = dk if value_dim is None else int(value_dim)
        if wide_norm is None:
            raise ValueError("a layer that borrows keys and values, or carries its gate in the fused projection, is built "
                             "with the q/k norm over the whole projection (wide_norm)")
        if position is not None or value_position is not None or qk_norm is not None or values_are_keys:
            raise ValueError("the norm over the whole projection comes without position encoding, per-head norm or "
                             "values that are the keys")
        if nq % nkv != 0 or min(dk, dv) <= 0 or max(dk, dv) > 1024:
            raise ValueError(f"heads ({nq}) must be a multiple of kv heads ({nkv}), head sizes ({dk}, {dv}) 1 .. 1024")
        if keep_first and mask != "window":
            raise ValueError("kept first positions belong to the window mask")
        wq, wk, eps = wide_norm
        kv_rows = 0 if self.borrows_kv else nkv * (dk + dv)
        g_rows = nq * dv if self.gate_fused else 0
        if self.gate_fused and gate is not None:
            raise ValueError("the gate is either a projection of its own or part of the fused projection")
        if qkv.out_features != nq * dk + kv_rows + g_rows:
            raise ValueError(f"the fused projection has {qkv.out_features} rows, expected {nq * dk + kv_rows + g_rows} "
                             f"(queries {nq * dk}, keys and values {kv_rows}, gate {g_rows})")
        if qkv.bias is not None:
            raise ValueError("the whole-projection path takes a projection without bias")
        if out.in_features != nq * dv:
            raise ValueError(f"output projection reads {out.in_features} columns, expected {nq * dv}")
        if gate is not None and gate.out_features != nq * dv:
            raise ValueError(f"the gate has {gate.out_features} rows, expected heads * value_dim = {nq * dv}")
        if wq.numel() != nq * dk or (not self.borrows_kv and (wk is None or wk.numel() != nkv * dk)):
            raise ValueError("the norm weights disagree with the sizes of q or k")
        if distance_bias is not None and (distance_bias.dim() != 2 or distance_bias.shape[1] != nq):
            raise ValueError(f"the distance bias is {tuple(distance_bias.shape)}, expected [distances, {nq}]")
        D = dk
        if dk != dv:            # pages and kernels know one head size: pad both with zeros, once
            D = max(dk, dv)
            D = (D + 15) // 16 * 16 if D <= 128 else D + (D & 1)
            w = qkv.weight
            parts = [_pad_head_rows(w[: nq * dk], nq, dk, D)]
            at = nq * dk
            if not self.borrows_kv:
                parts.append(_pad_head_rows(w[at: at + nkv * dk], nkv, dk, D))
                parts.append(_pad_head_rows(w[at + nkv * dk: at + nkv * (dk + dv)], nkv, dv, D))
                at += nkv * (dk + dv)
            if self.gate_fused:
                parts.append(_pad_head_rows(w[at:], nq, dv, D))
            qkv = Linear(torch.cat(parts).contiguous(), qkv.name, stream_rows=qkv.stream_rows)
            ow = out.weight
            wide = torch.zeros((ow.shape[0], nq, D), dtype=ow.dtype, device=ow.device)
            wide[:, :, :dv] = ow.reshape(ow.shape[0], nq, dv)
            out = Linear(wide.reshape(ow.shape[0], nq * D).contiguous(), out.name, stream_rows=out.stream_rows,
                         bias=out.bias, split_add_rows=out.split_add_rows)
            if gate is not None:
                gate = Linear(_pad_head_rows(gate.weight, nq, dv, D).contiguous(), gate.name,
                              bias=None if gate.bias is None else _pad_head_rows(gate.bias, nq, dv, D).contiguous())
            wq = _pad_head_rows(wq, nq, dk, D).contiguous()
            wk = None if wk is None else _pad_head_rows(wk, nkv, dk, D).contiguous()
        self.wide_norm = (wq, wk, float(eps))
        self.qkv, self.out, self.gate = qkv, out, gate
        self.key_dim, self.value_dim, self.head_dim = dk, dv, D
        self.num_heads, self.num_kv_heads = nq, nkv
        self.cache_spec = CacheSpec(mask, span if mask != "full" else 0, nkv, D, planes=2, keep_first=int(keep_first))
        self.values_are_keys, self.keep_first, self.distance_bias = False, int(keep_first), distance_bias
        self._general_attention = self.keep_first > 0 or distance_bias is not None
        self._general = False
        self.position = self.value_position = self.qk_norm = self.k_norm = None
        self.qk_norm_first, self._norm_fused, self._ones = False, False, None
        self.temperature = temperature
        self.softmax_scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(dk)
        self.act_dtype = act_dtype
        self.graph_safe = True

    def _forward_wide(self, ctx: StepContext, slot: LayerSlot, plan, table, qkv: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        T, nq, nkv, d = ctx.num_tokens, self.num_heads, self.num_kv_heads, self.head_dim
        if self.borrows_kv and slot.writes_cache:
            raise ValueError("a layer that brings queries only must read another entry's cache (cache_from)")
        wq, wk, eps = self.wide_norm
        coef, every = self.temperature if self.temperature is not None else (0.0, 0.0)
        first = nq * d + (0 if self.borrows_kv else 2 * nkv * d)
        q = torch.empty((T, nq, d), dtype=self.act_dtype, device=qkv.device)
        ops.qkv_post_wide(qkv[:, :first], ctx.positions, ctx.row_request, table, q, slot.kv, nq=nq, nkv=nkv, d=d,
                          page_size=slot.page_size, q_weight=wq, k_weight=wk, eps=eps, q_count=nq * self.key_dim,
                          k_count=nkv * self.key_dim, temp_coef=coef, temp_every=every, write_kv=slot.writes_cache,
                          has_kv=not self.borrows_kv)
        o = self._attend(ctx, slot, plan, table, q)
        if self.gate_fused:
            o = ops.sigmoid_gate(o.view(T, -1), qkv[:, first:])
        elif self.gate is not None:
            o = ops.sigmoid_gate(o.view(T, -1), self.gate(h))
        return self.out(o)

    def prefill_tile_rows(self, page_size: int) -> int:
        """Rows of one request that one attention CTA serves in a prompt portion: 128 where the tcgen05
        kernel takes this layer (bfloat16, head size 64 or 128, pages of 64 * 2^k), else 64."""
        if self._general_attention:
            return ops.KEYS_ATTENTION_TILE
        return ops.TC_PREFILL_TILE if ops.tc_prefill_supported(self.act_dtype, self.head_dim, page_size) else 64

    def step_planner(self, page_size: int) -> StepPlanner:
        return PagedAttentionPlanner(self.prefill_tile_rows(page_size))

    def _norm_heads(self, qkv: torch.Tensor, T: int) -> None:
        """The q/k norm as a part of its own: every head of q and of k is a row of width head_dim."""
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        for first, heads in ((0, nq), (nq * d, nkv)):
            cols = qkv[:, first:first + heads * d]
            rows = cols.reshape(T * heads, d).contiguous()
            normed, _ = self.qk_norm.apply(rows, None, rows=None, out_dtype=torch.float32)
            cols.copy_(normed.view(T, heads * d))

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        T = ctx.num_tokens
        plan = ctx.plans[("paged_attention", self.prefill_tile_rows(slot.page_size))]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        table = ctx.block_tables[slot.group]
        qkv = self.qkv(h)                                                       # [T, (nq + 2 nkv) d] float32
        if self.wide_norm is not None:
            return self._forward_wide(ctx, slot, plan, table, qkv, h)
        if self._general:
            return self._forward_general(ctx, slot, plan, table, qkv, h)

        rot = self.position.rotary() if self.position is not None else None
        if self.position is not None and rot is None and type(self.position).apply is not PositionEncoding.apply:
            # an encoding that is no plain rotation edits q and k itself, before norm and cache write
            q3 = qkv[:, : nq * d].view(T, nq, d)
            k3 = qkv[:, nq * d: (nq + nkv) * d].view(T, nkv, d)
            if self.qk_norm is not None and self.qk_norm_first:
                self._norm_heads(qkv, T)
            self.position.apply(ctx, q3, k3)
            if self.qk_norm is not None and not self.qk_norm_first and not self._norm_fused:
                self._norm_heads(qkv, T)
        elif self.qk_norm is not None and not self._norm_fused:
            self._norm_heads(qkv, T)             # before a rotation, or with no position encoding at all
        inv_freq, pairing = (rot[0], _PAIRING_CODE[rot[1]]) if rot is not None else (None, ops.ROPE_NONE)
        attn_scale, floor_scale = self.temperature if self.temperature is not None else (0.0, 0.0)

        q = torch.empty((T, nq, d), dtype=self.act_dtype, device=h.device)
        ops.qkv_post(qkv, ctx.positions, ctx.row_request, table, inv_freq, q, slot.kv, nq=nq, nkv=nkv, d=d,
                     page_size=slot.page_size, pairing=pairing,
                     l2_eps=self.qk_norm.eps if self._norm_fused else -1.0,
                     temp_attn_scale=attn_scale, temp_floor_scale=floor_scale, write_kv=slot.writes_cache,
                     l2_count=self.key_dim, kv_planes=self.cache_spec.planes)
        o = self._attend(ctx, slot, plan, table, q)
        if self.gate is not None:
            o = ops.sigmoid_gate(o.view(T, -1), self.gate(h))
        return self.out(o)

    def _norm_weight(self, norm: Optional[Norm], device) -> Optional[torch.Tensor]:
        if norm is None:
            return None
        w = getattr(norm, "weight", None)
        if w is None:                       # a weightless norm: the kernel multiplies by ones
            if self._ones is None:
                self._ones = torch.ones(self.key_dim, dtype=torch.float32, device=device)
            w = self._ones
        return w

    def _forward_general(self, ctx: StepContext, slot: LayerSlot, plan, table, qkv: torch.Tensor,
                         h: torch.Tensor) -> torch.Tensor:
        T, nq, nkv, d = ctx.num_tokens, self.num_heads, self.num_kv_heads, self.head_dim
        rot = self.position.rotary() if self.position is not None else None
        vrot = self.value_position.rotary() if self.value_position is not None else None
        pairing = _PAIRING_CODE[(rot or vrot or (None, "halves"))[1]]
        q = torch.empty((T, nq, d), dtype=self.act_dtype, device=qkv.device)
        ops.qkv_post_rot(qkv, ctx.positions, ctx.row_request, table, q, slot.kv, nq=nq, nkv=nkv, D=d,
                         key_dim=self.key_dim, value_dim=self.value_dim, page_size=slot.page_size, pairing=pairing,
                         q_norm_weight=self._norm_weight(self.qk_norm, qkv.device),
                         k_norm_weight=self._norm_weight(self.k_norm, qkv.device),
                         eps=self.qk_norm.eps if self.qk_norm is not None else 0.0,
                         inv_freq=rot[0] if rot is not None else None, rot_dims=self._rot_dims,
                         inv_freq_v=vrot[0] if vrot is not None else None, v_rot_dims=self._v_rot_dims,
                         write_kv=slot.writes_cache)
        o = self._attend(ctx, slot, plan, table, q)
        if vrot is not None:                # every head's sum of rotated values, turned back by the row's position
            o = ops.rotate_heads(o, ctx.positions, vrot[0], heads=nq, D=d, rot_dims=self._v_rot_dims, pairing=pairing,
                                 sign=-1.0, out_dtype=self.act_dtype)
        if self.gate is not None:
            o = ops.sigmoid_gate(o.view(T, -1), self.gate(h))
        return self.out(o)

    def _attend(self, ctx: StepContext, slot: LayerSlot, plan, table, q: torch.Tensor) -> torch.Tensor:
        T, nq, nkv, d = ctx.num_tokens, self.num_heads, self.num_kv_heads, self.head_dim
        h = q
        mask_kind, mask_span = _MASK_CODE[self.cache_spec.kind], max(self.cache_spec.span, 1)
        if self.act_dtype == torch.bfloat16 and d in ops.FAST_ATTENTION_HEAD_SIZES and not self._general_attention:
            # tensor-core kernels: tiles of prompt rows, and single rows split over their keys
            o = torch.empty((T, nq * d), dtype=torch.bfloat16, device=h.device)
            if plan.num_tiles:
                prefill = ops.attention_prefill_tc if plan.tile_rows == ops.TC_PREFILL_TILE else ops.attention_prefill
                prefill(q, slot.kv, table, plan.tiles, o, nq=nq, nkv=nkv, d=d, page_size=slot.page_size,
                        mask_kind=mask_kind, mask_span=mask_span, scale=self.softmax_scale, softcap=self.softcap,
                        sinks=self.sinks)
            if plan.num_decode_rows:
                ops.attention_decode(q, slot.kv, table, ctx.row_request, ctx.positions, o, rows=plan.decode_rows,
                                     num_rows=plan.num_decode_rows, nq=nq, nkv=nkv, d=d, page_size=slot.page_size,
                                     mask_kind=mask_kind, mask_span=mask_span, scale=self.softmax_scale,
                                     max_context=ctx.max_context, max_keys=plan.decode_keys, softcap=self.softcap,
                                     sinks=self.sinks)
        elif self.values_are_keys and ops.keys_attention_supported(self.act_dtype, d, d):
            # keys-only pages: the tensor-core kernels that read a key once for scores and value sum
            o = torch.empty((T, nq * d), dtype=torch.bfloat16, device=h.device)
            kw = dict(nq=nq, nkv=nkv, d=d, dv=d, page_size=slot.page_size, mask_kind=mask_kind, mask_span=mask_span,
                      scale=self.softmax_scale, keep_first=self.keep_first, dist_bias=self.distance_bias)
            if plan.num_tiles:
                ops.attention_keys_prefill(q, slot.kv, table, plan.tiles, o, **kw)
            if plan.num_decode_rows:
                ops.attention_keys_decode(q, slot.kv, table, ctx.row_request, ctx.positions, o, rows=plan.decode_rows,
                                          num_rows=plan.num_decode_rows, max_context=ctx.max_context, **kw)
        else:
            o = ops.paged_attention_generic(q, slot.kv, table, ctx.row_request, ctx.positions, nq=nq, nkv=nkv, d=d,
                                            page_size=slot.page_size, mask_kind=mask_kind, mask_span=mask_span,
                                            scale=self.softmax_scale, keep_first=self.keep_first,
                                            dist_bias=self.distance_bias, softcap=self.softcap, sinks=self.sinks)
        return o
