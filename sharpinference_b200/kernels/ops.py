"""Tensor-level wrappers of the kernel entry points.

Each function checks what the kernel cannot check itself (device, dtype, contiguity, shapes),
launches on torch's current CUDA stream and raises :class:`KernelError` on a refusal.  There
is no CPU path: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import KernelError, check, kernel

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

MASK_FULL, MASK_CHUNK, MASK_WINDOW = 0, 1, 2
ROPE_NONE, ROPE_INTERLEAVED, ROPE_HALVES = 0, 1, 2


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the engine has no CPU path); found device {t.device}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must have dtype {dtype}, found {t.dtype}")


def _need_columns(t: torch.Tensor, name: str, dtype=None) -> int:
    """A 2-D tensor whose rows are contiguous but may lie apart (a column range of a wider product); the distance
    between two rows in elements."""
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the engine has no CPU path); found device {t.device}")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with contiguous rows")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must have dtype {dtype}, found {t.dtype}")
    return int(t.stride(0)) if t.shape[0] > 1 else int(t.shape[1])


# ---------------------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` as fp32.  ``ids`` int32 [T], ``table`` [V, H] fp32 or bf16."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32)
    check(kernel("sharpi_embed_gather")(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), out.data_ptr(),
                                        T, H, V, _stream()), "sharpi_embed_gather")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, *, rows: Optional[torch.Tensor] = None, want_fp32: bool = False,
                out: Optional[torch.Tensor] = None, out32: Optional[torch.Tensor] = None):
    """Residual add fused with RMSNorm.

    Without ``rows``: ``x += delta`` in place (when ``delta`` is given) and the norm of every
    row is returned.  With ``rows`` (int32 indices): the norm of ``x[rows] + delta[rows]``, and
    ``x`` stays as it is.  Returns ``(out, out32)``; ``out32`` is the unrounded fp32 copy when
    ``want_fp32`` (or ``out32``) is given, else ``None``.
    """
    _need(x, "x", torch.float32)
    if weight is not None:                  # None: the weightless norm
        _need(weight, "weight", torch.float32)
    H = x.shape[-1]
    if delta is not None:
        _need(delta, "delta", torch.float32)
        if delta.shape != x.shape:
            raise KernelError(f"delta shape {tuple(delta.shape)} differs from x shape {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        T = rows.numel()
    else:
        T = x.numel() // H
    if out is None:
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    if want_fp32 and out32 is None:
        out32 = out if out_dtype == torch.float32 else torch.empty((T, H), dtype=torch.float32, device=x.device)
    alias = out32 is not None and out32.data_ptr() == out.data_ptr()
    check(kernel("sharpi_add_rmsnorm")(x.data_ptr(), _ptr(delta), _ptr(weight), float(eps), _ptr(rows), T, H,
                                       out.data_ptr(), dtype_code(out.dtype), None if alias else _ptr(out32),
                                       _stream()), "sharpi_add_rmsnorm")
    return out, out32


def swiglu(gate_up: torch.Tensor, out_dtype: torch.dtype, *, row_scale: Optional[torch.Tensor] = None,
           scale_rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(s g) * (s u)`` over a fused ``[M, 2I]`` gate|up product (fp32 in)."""
    _need(gate_up, "gate_up", torch.float32)
    M, I2 = gate_up.shape
    I = I2 // 2
    if out is None:
        out = torch.empty((M, I), dtype=out_dtype, device=gate_up.device)
    check(kernel("sharpi_swiglu")(gate_up.data_ptr(), _ptr(row_scale), _ptr(scale_rows), out.data_ptr(),
                                  dtype_code(out.dtype), M, I, _stream()), "sharpi_swiglu")
    return out


def timestamp(slots: torch.Tensor, index: int) -> None:
    """Write the GPU's nanosecond clock into ``slots[index]`` (int64) at this point of the current stream."""
    _need(slots, "slots", torch.int64)
    if not 0 <= index < slots.numel():
        raise KernelError(f"timestamp slot {index} outside 0 .. {slots.numel() - 1}")
    check(kernel("sharpi_timestamp")(slots.data_ptr(), index, _stream()), "sharpi_timestamp")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``y[m, :] += bias`` in place (float32)."""
    _need(y, "y", torch.float32)
    _need(bias, "bias", torch.float32)
    M, N = y.shape
    if bias.numel() != N:
        raise KernelError(f"bias has {bias.numel()} entries, the rows have {N}")
    check(kernel("sharpi_add_bias")(y.data_ptr(), bias.data_ptr(), M, N, _stream()), "sharpi_add_bias")
    return y


def add(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(a, "a", torch.float32)
    _need(b, "b", torch.float32)
    if out is None:
        out = torch.empty_like(a)
    check(kernel("sharpi_add")(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream()), "sharpi_add")
    return out


ACT_RELU2, ACT_GELU_TANH, ACT_SILU, ACT_SOFTPLUS = 0, 1, 2, 3
ACTIVATIONS = {"relu2": ACT_RELU2, "gelu_tanh": ACT_GELU_TANH, "silu": ACT_SILU, "softplus": ACT_SOFTPLUS}


def bias_act(y: torch.Tensor, bias: Optional[torch.Tensor], act: int, out_dtype: torch.dtype,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(y + bias)`` over a float32 product ``[M, N]`` (``bias`` float32 ``[N]`` or None), in ``out_dtype``:
    the square of relu, tanh-GELU, SiLU or softplus.  ``out`` may be ``y`` itself."""
    _need(y, "y", torch.float32)
    M, N = y.shape
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError(f"bias has {bias.numel()} entries, the rows have {N}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=y.device)
    check(kernel("sharpi_bias_act")(y.data_ptr(), _ptr(bias), out.data_ptr(), dtype_code(out.dtype), M, N, int(act),
                                    _stream()), "sharpi_bias_act")
    return out


def concat2(a: torch.Tensor, delta: Optional[torch.Tensor], b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``[a + delta | b]`` row by row (float32 ``[T, H]`` each, ``delta`` may be None) as ``[T, 2H]`` in ``out_dtype``."""
    _need(a, "a", torch.float32)
    _need(b, "b", torch.float32)
    if delta is not None:
        _need(delta, "delta", torch.float32)
    T, H = a.shape
    if b.shape != a.shape or (delta is not None and delta.shape != a.shape):
        raise KernelError(f"shapes differ: {tuple(a.shape)}, {tuple(b.shape)}")
    out = torch.empty((T, 2 * H), dtype=out_dtype, device=a.device)
    check(kernel("sharpi_concat2")(a.data_ptr(), _ptr(delta), b.data_ptr(), out.data_ptr(), dtype_code(out_dtype), T, H,
                                   _stream()), "sharpi_concat2")
    return out


def qkv_post(qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor,
             inv_freq: Optional[torch.Tensor], q_out: torch.Tensor, kv_layer: torch.Tensor, *, nq: int, nkv: int,
             d: int, page_size: int, pairing: int, l2_eps: float, temp_attn_scale: float, temp_floor_scale: float,
             write_kv: bool, l2_count: int = 0, kv_planes: int = 2) -> None:
    """RoPE, per-head L2 norm, temperature factor, q store and K/V scatter into pages.

    ``qkv`` fp32 [T, (nq + 2 nkv) d]; ``kv_layer`` is one layer's pages
    ``[pages, 2, nkv, page_size, d]`` in the dtype of ``q_out``; ``l2_eps < 0`` and
    ``temp_floor_scale <= 0`` switch the norm and the temperature factor off.  ``l2_count`` (default ``d``) is the
    number of elements the norm's mean of squares divides by: fewer than ``d`` when the heads are padded with zeros.
    ``kv_planes=1``: the values are the keys; ``qkv`` is [T, (nq + nkv) d] and a page holds keys only.
    """
    _need(qkv, "qkv", torch.float32)
    _need(positions, "positions", torch.int32)
    _need(row_req, "row_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    _need(q_out, "q_out")
    _need(kv_layer, "kv_layer", q_out.dtype)
    T = positions.numel()
    if qkv.shape != (T, (nq + kv_planes * nkv) * d):
        raise KernelError(f"qkv shape {tuple(qkv.shape)} is not [T={T}, (nq + {kv_planes} nkv) d = "
                          f"{(nq + kv_planes * nkv) * d}]")
    if tuple(kv_layer.shape[1:]) != (kv_planes, nkv, page_size, d):
        raise KernelError(f"kv_layer shape {tuple(kv_layer.shape)} is not [pages, {kv_planes}, {nkv}, {page_size}, {d}]")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != d // 2:
            raise KernelError(f"inv_freq has {inv_freq.numel()} entries, head size {d} needs {d // 2}")
    check(kernel("sharpi_qkv_post")(qkv.data_ptr(), positions.data_ptr(), row_req.data_ptr(),
                                    block_table.data_ptr(), _ptr(inv_freq), q_out.data_ptr(), kv_layer.data_ptr(),
                                    dtype_code(q_out.dtype), T, nq, nkv, d, block_table.shape[-1], page_size,
                                    pairing, float(l2_eps), float(temp_attn_scale), float(temp_floor_scale),
                                    int(write_kv), int(l2_count), int(kv_planes), _stream()), "sharpi_qkv_post")


def paged_attention_generic(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor,
                            row_req: torch.Tensor, positions: torch.Tensor, *, nq: int, nkv: int, d: int,
                            page_size: int, mask_kind: int, mask_span: int, scale: float,
                            out: Optional[torch.Tensor] = None, keep_first: int = 0,
                            dist_bias: Optional[torch.Tensor] = None, softcap: float = 0.0,
                            sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of every row over the keys it may see in its request's pages; [T, nq d].  A ``kv_layer`` with one
    plane (``[pages, 1, nkv, page_size, d]``) holds keys only and the values are the keys.  ``keep_first``: under
    a window mask the first positions of a sequence stay visible.  ``dist_bias`` float32 ``[far + 1, nq]`` is added
    to the scaled score by the distance between query and key (distances beyond ``far`` read the last row).
    ``softcap`` > 0: the scaled score ``s`` becomes ``softcap * tanh(s / softcap)``.  ``sinks`` float32 ``[nq]``:
    ``exp(sinks[h])`` joins the softmax's denominator of head ``h`` (no key, no value)."""
    _need(q, "q")
    _need(kv_layer, "kv_layer", q.dtype)
    _check_sinks(sinks, nq)
    _need(block_table, "block_table", torch.int32)
    _need(row_req, "row_req", torch.int32)
    _need(positions, "positions", torch.int32)
    T = positions.numel()
    if out is None:
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
    if dist_bias is not None:
        _need(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[1] != nq or dist_bias.shape[0] < 1:
            raise KernelError(f"dist_bias is {tuple(dist_bias.shape)}, expected [far + 1, {nq}]")
    check(kernel("sharpi_paged_attention_generic")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                                   row_req.data_ptr(), positions.data_ptr(), out.data_ptr(),
                                                   dtype_code(q.dtype), T, nq, nkv, d, block_table.shape[-1],
                                                   page_size, mask_kind, mask_span, float(scale),
                                                   int(kv_layer.shape[1]), int(keep_first), _ptr(dist_bias),
                                                   0 if dist_bias is None else dist_bias.shape[0] - 1,
                                                   float(softcap), _ptr(sinks), _stream()),
          "sharpi_paged_attention_generic")
    return out


def _check_sinks(sinks: Optional[torch.Tensor], nq: int) -> None:
    if sinks is not None:
        _need(sinks, "sinks", torch.float32)
        if sinks.numel() != nq:
            raise KernelError(f"sinks has {sinks.numel()} entries for {nq} heads")


FAST_ATTENTION_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128)
DECODE_SPLIT = 256


_ticket_buffers = {}


def zeroed_tickets(device, count: int) -> torch.Tensor:
    """``count`` int32 zeros for kernels whose last CTA finishes a piece of work (it counts arrivals there and
    leaves the counters at zero).  One buffer per device and stream, so that launches that may overlap on two
    streams never share counters; it grows when a launch needs more."""
    key = (torch.device(device), torch.cuda.current_stream(device).cuda_stream)
    buf = _ticket_buffers.get(key)
    if buf is None or buf.numel() < count:
        buf = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _ticket_buffers[key] = buf
    return buf


def decode_splits(max_context: int, mask_kind: int, mask_span: int) -> int:
    """An upper bound on the 256-key splits a decode row needs (the kernel skips the empty ones)."""
    full = (max_context + DECODE_SPLIT - 1) // DECODE_SPLIT
    if mask_kind == MASK_FULL:
        return max(full, 1)
    return max(1, min(full, (mask_span + DECODE_SPLIT - 1) // DECODE_SPLIT + 1))


def attention_decode(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, row_req: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, *, rows: Optional[torch.Tensor], num_rows: int,
                     nq: int, nkv: int, d: int, page_size: int, mask_kind: int, mask_span: int, scale: float,
                     max_context: int, max_keys: Optional[int] = None, softcap: float = 0.0,
                     sinks: Optional[torch.Tensor] = None) -> None:
    """Split-KV paged attention for rows that bring one query each (bfloat16).  ``rows`` (int32) names
    the rows to serve, or None for rows ``0 .. num_rows - 1``; results go to ``out[row]``.  ``max_context`` bounds
    the longest row (position + 1), ``max_keys`` the sum of position + 1 over the served rows: with it the launch
    holds about as many CTAs as the rows have splits together, not rows times the longest row's splits."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    _check_sinks(sinks, nq)
    if d not in FAST_ATTENTION_HEAD_SIZES:
        raise KernelError(f"head size {d} is not served by the tensor-core attention kernels "
                          f"({FAST_ATTENTION_HEAD_SIZES}); use the generic kernel")
    splits = decode_splits(max_context, mask_kind, mask_span)
    # a row at position p has at most p // 256 + 1 splits, so the rows together at most max_keys // 256 + rows
    items = num_rows * splits if max_keys is None else min(num_rows * splits, max_keys // DECODE_SPLIT + num_rows)
    part_o = torch.empty((num_rows, nq, splits, d), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((num_rows, nq, splits, 2), dtype=torch.float32, device=q.device)
    check(kernel("sharpi_attention_decode")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                            row_req.data_ptr(), positions.data_ptr(), _ptr(rows), part_o.data_ptr(),
                                            part_ml.data_ptr(), out.data_ptr(), status_word(q.device).data_ptr(),
                                            kv_layer.shape[0], num_rows, nq, nkv, d,
                                            block_table.shape[-1], page_size, mask_kind, mask_span, splits, items,
                                            float(scale), float(softcap), _ptr(sinks), _stream()),
          "sharpi_attention_decode")


KEYS_ATTENTION_TILE = 64


def keys_attention_supported(dtype: torch.dtype, d: int, dv: int) -> bool:
    """Whether the tensor-core kernels for keys-only pages take a cached row of ``d`` elements of which the first
    ``dv`` are the value: bfloat16, both multiples of 16, ``dv <= d <= 512``."""
    return dtype == torch.bfloat16 and d % 16 == 0 and dv % 16 == 0 and 0 < dv <= d <= 512


def attention_keys_prefill(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor,
                           out: torch.Tensor, *, nq: int, nkv: int, d: int, dv: int, page_size: int, mask_kind: int,
                           mask_span: int, scale: float, keep_first: int = 0,
                           dist_bias: Optional[torch.Tensor] = None) -> None:
    """Paged attention over keys-only pages ``[pages, 1, nkv, page_size, d]`` for tiles of up to 64 consecutive rows of
    one request (bfloat16): a key's value is the first ``dv`` elements of its row; ``out`` is ``[T, nq * dv]``.
    ``keep_first`` and ``dist_bias`` as in :func:`paged_attention_generic`."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(tiles, "tiles", torch.int32)
    if not keys_attention_supported(q.dtype, d, dv) or tuple(kv_layer.shape[1:]) != (1, nkv, page_size, d):
        raise KernelError(f"kv_layer {tuple(kv_layer.shape)} is not [pages, 1, {nkv}, {page_size}, {d}] or the sizes "
                          f"({d}, {dv}) are no multiples of 16 up to 512")
    if dist_bias is not None:
        _need(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[1] != nq:
            raise KernelError(f"dist_bias is {tuple(dist_bias.shape)}, expected [far + 1, {nq}]")
    check(kernel("sharpi_attention_keys_prefill")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(), tiles.data_ptr(),
                                                  out.data_ptr(), tiles.shape[0], nq, nkv, d, dv, block_table.shape[-1],
                                                  page_size, mask_kind, mask_span, int(keep_first), _ptr(dist_bias),
                                                  0 if dist_bias is None else dist_bias.shape[0] - 1, float(scale),
                                                  _stream()), "sharpi_attention_keys_prefill")


def attention_keys_decode(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, row_req: torch.Tensor,
                          positions: torch.Tensor, out: torch.Tensor, *, rows: Optional[torch.Tensor], num_rows: int,
                          nq: int, nkv: int, d: int, dv: int, page_size: int, mask_kind: int, mask_span: int, scale: float,
                          max_context: int, keep_first: int = 0, dist_bias: Optional[torch.Tensor] = None) -> None:
    """The same attention for rows that bring one query each, split over the keys in 256s; ``max_context`` bounds the
    longest row (position + 1).  Results go to ``out[row]`` (``[T, nq * dv]``)."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    if not keys_attention_supported(q.dtype, d, dv) or tuple(kv_layer.shape[1:]) != (1, nkv, page_size, d):
        raise KernelError(f"kv_layer {tuple(kv_layer.shape)} is not [pages, 1, {nkv}, {page_size}, {d}] or the sizes "
                          f"({d}, {dv}) are no multiples of 16 up to 512")
    if dist_bias is not None:
        _need(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[1] != nq:
            raise KernelError(f"dist_bias is {tuple(dist_bias.shape)}, expected [far + 1, {nq}]")
    splits = max(1, (max_context + DECODE_SPLIT - 1) // DECODE_SPLIT)
    part_o = torch.empty((num_rows, nq, splits, dv), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((num_rows, nq, splits, 2), dtype=torch.float32, device=q.device)
    check(kernel("sharpi_attention_keys_decode")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(), row_req.data_ptr(),
                                                 positions.data_ptr(), _ptr(rows), part_o.data_ptr(), part_ml.data_ptr(),
                                                 out.data_ptr(), num_rows, nq, nkv, d, dv, block_table.shape[-1], page_size,
                                                 mask_kind, mask_span, int(keep_first), _ptr(dist_bias),
                                                 0 if dist_bias is None else dist_bias.shape[0] - 1, splits, float(scale),
                                                 _stream()), "sharpi_attention_keys_decode")


def attention_prefill(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor,
                      out: torch.Tensor, *, nq: int, nkv: int, d: int, page_size: int, mask_kind: int,
                      mask_span: int, scale: float, softcap: float = 0.0,
                      sinks: Optional[torch.Tensor] = None) -> None:
    """Paged attention for tiles of up to 64 consecutive rows of one request (bfloat16).  ``tiles`` is
    int32 [n, 4]: first row, number of rows, position of the first row, request index."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(tiles, "tiles", torch.int32)
    _check_sinks(sinks, nq)
    if d not in FAST_ATTENTION_HEAD_SIZES:
        raise KernelError(f"head size {d} is not served by the tensor-core attention kernels "
                          f"({FAST_ATTENTION_HEAD_SIZES}); use the generic kernel")
    check(kernel("sharpi_attention_prefill")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                             tiles.data_ptr(), out.data_ptr(), tiles.shape[0], nq, nkv, d,
                                             block_table.shape[-1], page_size, mask_kind, mask_span, float(scale),
                                             float(softcap), _ptr(sinks), _stream()), "sharpi_attention_prefill")


TC_PREFILL_TILE = 128


def tc_prefill_supported(dtype: torch.dtype, d: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention kernel takes this layer: bfloat16, head size 64 or 128,
    pages of a power of two >= 64 positions."""
    return dtype == torch.bfloat16 and d in (64, 128) and page_size >= 64 and (page_size & (page_size - 1)) == 0


def attention_prefill_tc(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor,
                         out: torch.Tensor, *, nq: int, nkv: int, d: int, page_size: int, mask_kind: int,
                         mask_span: int, scale: float, softcap: float = 0.0,
                         sinks: Optional[torch.Tensor] = None) -> None:
    """Paged attention for tiles of up to 128 consecutive rows of one request on tcgen05 / TMEM / TMA."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(tiles, "tiles", torch.int32)
    _check_sinks(sinks, nq)
    if not tc_prefill_supported(q.dtype, d, page_size):
        raise KernelError(f"the tcgen05 attention kernel takes head sizes 64 and 128 and pages of 64 * 2^k positions, "
                          f"found head size {d}, page size {page_size}")
    check(kernel("sharpi_attention_prefill_tc")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                                tiles.data_ptr(), out.data_ptr(), status_word(q.device).data_ptr(),
                                                q.shape[0], kv_layer.shape[0], tiles.shape[0], nq, nkv, d,
                                                block_table.shape[-1], page_size, mask_kind, mask_span, float(scale),
                                                float(softcap), _ptr(sinks), _stream()), "sharpi_attention_prefill_tc")


def gemm_nt(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
            group_offsets: Optional[torch.Tensor] = None, a_rows: Optional[torch.Tensor] = None,
            out_rows: Optional[torch.Tensor] = None, rows: Optional[int] = None, accumulate: bool = False,
            bias: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
            scale_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C = A . W^T`` with fp32 accumulation on the CUDA cores.

    Dense: ``w`` is [N, K].  Grouped: ``w`` is [E, N, K] and ``group_offsets`` (int32 [E+1])
    gives the first sorted row of every expert.  ``a_rows`` / ``out_rows`` (int32 [rows]) make
    sorted row r read ``A[a_rows[r]]`` and write ``C[out_rows[r]]``.  ``row_scale`` (float32)
    multiplies row r of the product by ``row_scale[scale_rows[r] or r]``, ``bias`` (float32 [N]) is
    added to it, before the row is stored or added in.
    """
    _need(a, "a")
    _need(w, "w")
    K = a.shape[-1]
    if w.shape[-1] != K:
        raise KernelError(f"inner sizes differ: a [..., {K}] against w [..., {w.shape[-1]}]")
    if group_offsets is not None:
        _need(group_offsets, "group_offsets", torch.int32)
        if w.dim() != 3 or group_offsets.numel() != w.shape[0] + 1:
            raise KernelError("a grouped product needs w [E, N, K] and group_offsets [E + 1]")
        E, N = w.shape[0], w.shape[1]
    else:
        if w.dim() != 2:
            raise KernelError("a dense product needs w [N, K]")
        E, N = 1, w.shape[0]
    M = rows if rows is not None else (a_rows.numel() if a_rows is not None else a.shape[0])
    if out is None:
        if accumulate:
            raise KernelError("accumulate=True needs an output tensor to add to")
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _need(out, "out", torch.float32)
    if a_rows is not None:
        _need(a_rows, "a_rows", torch.int32)
    if out_rows is not None:
        _need(out_rows, "out_rows", torch.int32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError(f"bias has {bias.numel()} entries, the product has {N} columns")
    if row_scale is not None:
        _need(row_scale, "row_scale", torch.float32)
    if scale_rows is not None:
        _need(scale_rows, "scale_rows", torch.int32)
    check(kernel("sharpi_gemm_nt")(a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype),
                                   out.data_ptr(), _ptr(group_offsets), _ptr(a_rows), _ptr(out_rows), M, N, K, E,
                                   int(accumulate), _ptr(bias), _ptr(row_scale), _ptr(scale_rows), _stream()),
          "sharpi_gemm_nt")
    return out


# ---------------------------------------------------------------------------------------
# tensor-core kernels (tcgen05 / TMEM / TMA)
# ---------------------------------------------------------------------------------------
_status_words = {}


def status_word(device) -> torch.Tensor:
    """The device word in which a tensor-core kernel records a wait that gave up (0 = none)."""
    device = torch.device(device)
    w = _status_words.get(device)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = w
    return w


def check_status(device) -> None:
    """Raise if a tensor-core kernel gave up on a wait since the last check (synchronises)."""
    w = _status_words.get(torch.device(device))
    if w is not None:
        code = int(w.item())
        if code != 0:
            w.zero_()
            for buf in list(_ticket_buffers.values()) + list(_argmax_scratches.values()) + list(_sliced_work.values()):
                buf.zero_()               # a kernel that gave up may have left counters behind
            raise KernelError(f"a tensor-core kernel gave up (code {code}: 1 = wait for a free stage, 2 = for a loaded "
                              f"stage, 3 = for the accumulator, 4 = for a key/value copy, 5 = misaligned staging "
                              f"buffer, 6 = misaligned shared memory, 7 = for drained tensor memory, 11-18 = "
                              f"attention: queries, keys, values, scores, probabilities, outputs, free stage, "
                              f"misaligned shared memory); its output is incomplete")


TC_MODE_STORE, TC_MODE_SWIGLU = 0, 1


TC_PERSISTENT = 0            # row_tile value that selects the persistent kernel
TC_PERSISTENT_MAX_GROUPS = 256


def tc_row_tile(rows: int, mode: Optional[int] = None, groups: int = 1) -> int:
    """Activation rows per CTA for a grouped product over `rows` rows in all; TC_PERSISTENT for the kernel
    that walks work items (gate|up products of 1024 rows and more: measured 406 vs 455 us at 1024 rows,
    490 vs 563 us at 2048 unevenly spread rows, 634 vs 753 us at 4096; the down product has too few items
    per SM to gain and stays on the tiled kernel)."""
    if mode == TC_MODE_SWIGLU and rows >= 1024 and groups <= TC_PERSISTENT_MAX_GROUPS:
        return TC_PERSISTENT
    if rows <= 128:
        return 16
    if rows <= 256:
        return 32
    if rows <= 512:
        return 64
    return 128


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once)."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def tc_k_split(rows: int, n_out: int, sms: int = 148) -> int:
    """Into how many CTAs a tile's K range is cut.  With few rows few experts are active (at most one
    per row), so 128-row weight tiles alone cannot fill the GPU; cutting K makes up to four times as many
    CTAs.  The CTA of a tile that finishes last adds the parts in a fixed order."""
    if rows > 16:
        return 1
    ctas = rows * ((n_out + 127) // 128)
    if ctas >= sms:
        return 1
    return max(1, min(4, (2 * sms + ctas - 1) // ctas))


def gather_rows_bf16(x: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[r] = x[rows[r]]`` for bfloat16 rows whose width is a multiple of 8."""
    _need(x, "x", torch.bfloat16)
    _need(rows, "rows", torch.int32)
    R, K = rows.numel(), x.shape[-1]
    if out is None:
        out = torch.empty((R, K), dtype=torch.bfloat16, device=x.device)
    check(kernel("sharpi_gather_rows_bf16")(x.data_ptr(), rows.data_ptr(), out.data_ptr(), R, K, _stream()),
          "sharpi_gather_rows_bf16")
    return out


def tc_grouped_gemm(a: torch.Tensor, w: torch.Tensor, group_offsets: torch.Tensor, *, mode: int,
                    out: Optional[torch.Tensor] = None, out_rows: Optional[torch.Tensor] = None,
                    row_scale: Optional[torch.Tensor] = None, scale_rows: Optional[torch.Tensor] = None,
                    accumulate: bool = False, row_tile: Optional[int] = None,
                    k_split: Optional[int] = None, max_ctas: int = 0) -> torch.Tensor:
    """Per-expert products on the tensor cores.  ``a`` bfloat16 [rows, K] sorted by expert,
    ``w`` bfloat16 [E, N, K], ``group_offsets`` int32 [E + 1].

    ``mode=TC_MODE_STORE``: float32 ``out[out_rows[r] or r] (+)= s * a[r] . w[e(r)]^T``, shape [*, N], with
    ``s = row_scale[scale_rows[r] or r]`` when ``row_scale`` is given (a router that weights outputs), else 1.
    ``mode=TC_MODE_SWIGLU``: ``w`` holds gate rows then up rows (N = 2 I); bfloat16
    ``out[r] = silu(s g) * (s u)``, shape [rows, I], ``s = row_scale[scale_rows[r]]``.
    ``max_ctas`` > 0 (persistent kernel only) keeps the launch to that many SMs, for running beside another kernel.
    """
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    _need(group_offsets, "group_offsets", torch.int32)
    rows, K = a.shape
    E, N, Kw = w.shape
    if Kw != K or group_offsets.numel() != E + 1:
        raise KernelError(f"shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, offsets {group_offsets.numel()}")
    if K % 8 != 0:
        raise KernelError(f"the tensor-core product needs an inner size that is a multiple of 8, found {K}")
    if out is None:
        if accumulate:
            raise KernelError("accumulate=True needs an output tensor to add to")
        out = (torch.empty((rows, N // 2), dtype=torch.bfloat16, device=a.device) if mode == TC_MODE_SWIGLU
               else torch.empty((rows, N), dtype=torch.float32, device=a.device))
    _need(out, "out", torch.bfloat16 if mode == TC_MODE_SWIGLU else torch.float32)
    status = status_word(a.device)
    if k_split is None:
        k_split = tc_k_split(rows, (N // 2 if mode == TC_MODE_SWIGLU else N), sm_count(a.device))
    partial = torch.empty((k_split, rows, N), dtype=torch.float32, device=a.device) if k_split > 1 else None
    if row_tile is None:
        row_tile = tc_row_tile(rows, mode, E)
    tickets = None
    if k_split > 1:           # one counter per (weight tile, row tile) of the launch grid
        tickets = zeroed_tickets(a.device, ((N + 127) // 128) * (rows // max(row_tile, 1) + min(rows, E)))
    check(kernel("sharpi_tc_grouped_gemm")(a.data_ptr(), w.data_ptr(), group_offsets.data_ptr(), out.data_ptr(),
                                           _ptr(out_rows), _ptr(row_scale), _ptr(scale_rows), status.data_ptr(),
                                           _ptr(partial), _ptr(tickets), rows, N, K, E, mode, row_tile,
                                           int(accumulate), k_split, int(max_ctas) if row_tile == TC_PERSISTENT else 0,
                                           _stream()), "sharpi_tc_grouped_gemm")
    return out


_TC_STORE_ACT = {ACT_RELU2: 1, ACT_GELU_TANH: 2, ACT_SILU: 3}


def tc_grouped_gemm_act(a: torch.Tensor, w: torch.Tensor, group_offsets: torch.Tensor, act: int,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The first product of two-layer experts on the tensor cores with the activation in the epilogue:
    bfloat16 ``out[r] = act(a[r] . w[e(r)]^T)``, ``[rows, N]`` in sorted row order (``act``: ``ACT_RELU2``,
    ``ACT_GELU_TANH`` or ``ACT_SILU``).  Operands as in :func:`tc_grouped_gemm`."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    _need(group_offsets, "group_offsets", torch.int32)
    rows, K = a.shape
    E, N, Kw = w.shape
    if Kw != K or group_offsets.numel() != E + 1:
        raise KernelError(f"shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, offsets {group_offsets.numel()}")
    if K % 8 != 0:
        raise KernelError(f"the tensor-core product needs an inner size that is a multiple of 8, found {K}")
    if act not in _TC_STORE_ACT:
        raise KernelError(f"unknown activation code {act}")
    if out is None:
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=a.device)
    _need(out, "out", torch.bfloat16)
    k_split = tc_k_split(rows, N, sm_count(a.device))
    partial = torch.empty((k_split, rows, N), dtype=torch.float32, device=a.device) if k_split > 1 else None
    row_tile = tc_row_tile(rows, TC_MODE_STORE, E)
    tickets = None
    if k_split > 1:
        tickets = zeroed_tickets(a.device, ((N + 127) // 128) * (rows // max(row_tile, 1) + min(rows, E)))
    check(kernel("sharpi_tc_grouped_gemm_act")(a.data_ptr(), w.data_ptr(), group_offsets.data_ptr(), out.data_ptr(),
                                               status_word(a.device).data_ptr(), _ptr(partial), _ptr(tickets), rows, N,
                                               K, E, row_tile, k_split, _TC_STORE_ACT[act], _stream()),
          "sharpi_tc_grouped_gemm_act")
    return out


def tc_set_wait_test(limit: int, drop_from: int) -> None:
    """Test hook: the next ``tc_grouped_gemm`` launch (tiled kernel) polls each wait at most ``limit`` times and
    loads nothing from K block ``drop_from`` on, so a wait runs out, the kernel records its code in the status
    word and returns; ``check_status`` then raises.  Consumed by that one launch."""
    import ctypes
    from .library import load_library
    fn = load_library("tc_gemm").sharpi_tc_set_wait_test
    fn.argtypes, fn.restype = [ctypes.c_uint, ctypes.c_int], None
    fn(int(limit), int(drop_from))


_dense_offsets = {}


def tc_dense(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
             accumulate: bool = False) -> torch.Tensor:
    """A dense product ``a . w^T`` for a few rows on the grouped tensor-core kernel with one group: the
    weights stream once through 128-row tiles, K cut over CTAs when the tiles alone would not fill the GPU.
    float32 ``[M, N]``, added into ``out`` with reductions when ``accumulate`` (so that another launch may add
    into the same rows meanwhile).  Alone it is slower than :func:`dense_rows` and the library; its small CTAs
    run well beside the routed experts' kernels, which is where the mixture part uses it."""
    M = a.shape[0]
    key = (a.device, M)
    offsets = _dense_offsets.get(key)
    if offsets is None:
        offsets = torch.tensor([0, M], dtype=torch.int32, device=a.device)
        _dense_offsets[key] = offsets
    N = w.shape[0]
    n_tiles = (N + 127) // 128
    sms = sm_count(a.device)
    k_split = 1 if n_tiles >= sms else max(1, min(4, (2 * sms + n_tiles - 1) // n_tiles))
    row_tile = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    return tc_grouped_gemm(a, w.unsqueeze(0), offsets, mode=TC_MODE_STORE, out=out, row_tile=row_tile,
                           k_split=k_split, accumulate=accumulate)


DENSE_ROWS_MAX = 16           # rows the weight-streaming dense kernel takes


def dense_rows(a: torch.Tensor, w: torch.Tensor, *, swiglu: bool = False, out: Optional[torch.Tensor] = None,
               accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a . w^T`` for up to 16 bfloat16 rows against a bfloat16 weight ``[N, K]`` that streams in once
    (``dense_rows.cu``): float32 ``[M, N]`` (plus ``bias``), added into ``out`` with reductions when
    ``accumulate``, or with ``swiglu`` (``w`` = gate rows then up rows) ``silu(g) * u`` in bfloat16 ``[M, N / 2]``."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)}, activations have width {K}")
    if M > DENSE_ROWS_MAX:
        raise KernelError(f"dense_rows takes up to {DENSE_ROWS_MAX} rows, found {M}")
    if swiglu and (accumulate or bias is not None):
        raise KernelError("the SwiGLU epilogue neither accumulates nor takes a bias")
    if accumulate and out is None:
        raise KernelError("accumulate needs an output to add to")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device) if swiglu else \
            torch.empty((M, N), dtype=torch.float32, device=a.device)
    else:
        _need(out, "out", torch.bfloat16 if swiglu else torch.float32)
        if tuple(out.shape) != ((M, N // 2) if swiglu else (M, N)):
            raise KernelError(f"out is {tuple(out.shape)} for a product of {M} rows and a weight of {N} rows")
    mode = 2 if swiglu else 1 if accumulate else 0
    check(kernel("sharpi_dense_rows")(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, mode,
                                      _stream()), "sharpi_dense_rows")
    return out


def router_top1(h32: torch.Tensor, router_weight: torch.Tensor, *, want_logits: bool = False, sort: bool = False):
    """Top-1 sigmoid routing.  Returns ``(expert_id int32 [T], weight fp32 [T], logits or None)``; with
    ``sort`` also ``offsets`` and ``sorted_rows`` as :func:`moe_sort` gives them (from the same launch for
    steps of up to 32 tokens)."""
    _need(h32, "h32", torch.float32)
    _need(router_weight, "router_weight", torch.float32)
    T, H = h32.shape
    E = router_weight.shape[0]
    if router_weight.shape[1] != H:
        raise KernelError(f"router weight is {tuple(router_weight.shape)}, activations have width {H}")
    expert = torch.empty((T,), dtype=torch.int32, device=h32.device)
    weight = torch.empty((T,), dtype=torch.float32, device=h32.device)
    logits = torch.empty((T, E), dtype=torch.float32, device=h32.device) if want_logits else None
    scratch = _router_scratch(h32.device, E) if T <= 32 else None
    offsets = sorted_rows = None
    if sort:
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=h32.device)
        sorted_rows = torch.empty((T,), dtype=torch.int32, device=h32.device)
    check(kernel("sharpi_router_top1")(h32.data_ptr(), router_weight.data_ptr(), T, H, E, 0, expert.data_ptr(),
                                       weight.data_ptr(), _ptr(logits), _ptr(scratch), _ptr(offsets), _ptr(sorted_rows),
                                       _stream()), "sharpi_router_top1")
    if sort:
        return expert, weight, logits, offsets, sorted_rows
    return expert, weight, logits


_router_scratches = {}


def _router_scratch(device, num_experts: int) -> torch.Tensor:
    """Scratch of the few-token router kernel: 32 x E logits, then 32 ticket counters that start at zero
    and are left at zero by every launch.  One per device and expert count, shared by all layers (launches
    on one stream run one after the other)."""
    key = (torch.device(device), num_experts)
    buf = _router_scratches.get(key)
    if buf is None:
        buf = torch.zeros(32 * num_experts + 33, dtype=torch.float32, device=device)
        _router_scratches[key] = buf
    return buf


def moe_sort(expert_id: torch.Tensor, num_experts: int):
    """Stable sort of rows by expert: ``(offsets int32 [E+1], sorted_rows int32 [T])``."""
    _need(expert_id, "expert_id", torch.int32)
    T = expert_id.numel()
    offsets = torch.empty((num_experts + 1,), dtype=torch.int32, device=expert_id.device)
    sorted_rows = torch.empty((T,), dtype=torch.int32, device=expert_id.device)
    check(kernel("sharpi_moe_sort")(expert_id.data_ptr(), T, num_experts, offsets.data_ptr(),
                                    sorted_rows.data_ptr(), _stream()), "sharpi_moe_sort")
    return offsets, sorted_rows


ROUTER_SCORING = {"sigmoid": 0, "softmax_chosen": 1}


def router_topk(h32: torch.Tensor, router_weight: torch.Tensor, k: int, *, correction: Optional[torch.Tensor] = None,
                scale: float = 1.0, renormalize: bool = False, want_scores: bool = False,
                bias: Optional[torch.Tensor] = None, scoring: str = "sigmoid"):
    """Sigmoid routing to ``k`` experts a row.  ``s = sigmoid(h . Wr^T)`` in float32; the ``k`` largest of
    ``s + correction`` are chosen (the lowest index among equals); the weights are ``scale * s`` of the chosen,
    divided by their sum first when ``renormalize``.  ``bias`` float32 ``[E]`` is added to the logits.
    ``scoring="softmax_chosen"``: the ``k`` largest logits are chosen and the weights are ``scale`` times the softmax
    over the chosen logits alone (``scores`` are then the logits).  Returns ``(expert_id int32 [T, k], weight float32
    [T, k], scores [T, E] or None)``."""
    _need(h32, "h32", torch.float32)
    _need(router_weight, "router_weight", torch.float32)
    T, H = h32.shape
    E = router_weight.shape[0]
    if router_weight.shape[1] != H:
        raise KernelError(f"router weight is {tuple(router_weight.shape)}, activations have width {H}")
    if correction is not None:
        _need(correction, "correction", torch.float32)
        if correction.numel() != E:
            raise KernelError(f"correction has {correction.numel()} entries for {E} experts")
    if not (1 <= k <= min(E, 32)):
        raise KernelError(f"experts per row must be 1 .. min(experts, 32), found {k} of {E}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != E:
            raise KernelError(f"router bias has {bias.numel()} entries for {E} experts")
    if scoring not in ROUTER_SCORING:
        raise KernelError(f"router scoring '{scoring}' is not one of {', '.join(ROUTER_SCORING)}")
    expert = torch.empty((T, k), dtype=torch.int32, device=h32.device)
    weight = torch.empty((T, k), dtype=torch.float32, device=h32.device)
    scores = torch.empty((T, E), dtype=torch.float32, device=h32.device) if want_scores else None
    check(kernel("sharpi_router_topk")(h32.data_ptr(), router_weight.data_ptr(), _ptr(correction), T, H, E, k,
                                       float(scale), int(renormalize), expert.data_ptr(), weight.data_ptr(),
                                       _ptr(scores), _ptr(bias), ROUTER_SCORING[scoring], _stream()), "sharpi_router_topk")
    return expert, weight, scores


def moe_pair_tokens(sorted_pairs: torch.Tensor, k: int) -> torch.Tensor:
    """For (row, choice) pairs numbered ``row * k + choice`` and sorted by expert: the row of every sorted pair."""
    _need(sorted_pairs, "sorted_pairs", torch.int32)
    out = torch.empty_like(sorted_pairs)
    check(kernel("sharpi_moe_pair_tokens")(sorted_pairs.data_ptr(), sorted_pairs.numel(), k, out.data_ptr(), _stream()),
          "sharpi_moe_pair_tokens")
    return out


def moe_combine(y_pairs: torch.Tensor, k: int, *, add: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = add[t] + sum_j y_pairs[t * k + j]`` (float32), the choices added in their order."""
    _need(y_pairs, "y_pairs", torch.float32)
    P, H = y_pairs.shape
    if P % k:
        raise KernelError(f"{P} pair rows are no multiple of k = {k}")
    T = P // k
    if add is not None:
        _need(add, "add", torch.float32)
        if tuple(add.shape) != (T, H):
            raise KernelError(f"add is {tuple(add.shape)}, expected {(T, H)}")
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=y_pairs.device)
    _need(out, "out", torch.float32)
    check(kernel("sharpi_moe_combine")(y_pairs.data_ptr(), _ptr(add), out.data_ptr(), T, k, H, _stream()),
          "sharpi_moe_combine")
    return out


MLSTM_MAX_KEY_SIZE = 512


def mlstm_state_floats(heads: int, d: int, dv: int):
    """``(floats per head, floats per request)`` of the matrix-memory state: per head, for every slice of 32 value
    columns ``[d, 32]`` of the memory, then the normaliser ``[d]``, then the running maximum (padded to four
    floats)."""
    slices = (dv + 31) // 32
    per_head = slices * d * 32 + d + 4
    return per_head, heads * per_head


def mlstm_recurrence(proj: torch.Tensor, *, col_q: int, col_k: int, col_v: int, col_i: int, col_f: int,
                     bias_i: torch.Tensor, bias_f: torch.Tensor, row_offsets: torch.Tensor, state_slots: torch.Tensor,
                     state: torch.Tensor, heads: int, d: int, dv: int, cap: float, q_scale: float):
    """The matrix-memory recurrence over the step's rows (``mlstm.cu``): reads q, k, v and the raw gates from the
    fused float32 projection ``proj [T, ld]`` at the given first columns and advances ``state [slots, floats]`` of
    the step's requests (``state_slots [B]``, rows ``row_offsets [B + 1]``).  Returns ``(num, nq, coef)``: the
    numerators ``S^T q`` float32 ``[T, heads * dv]``, ``n . q`` ``[T, heads]`` and per row and head ``(log a, log b,
    m, -)``, which :func:`mlstm_out` turns into the mixer's output."""
    _need(proj, "proj", torch.float32)
    _need(bias_i, "bias_i", torch.float32)
    _need(bias_f, "bias_f", torch.float32)
    _need(row_offsets, "row_offsets", torch.int32)
    _need(state_slots, "state_slots", torch.int32)
    _need(state, "state", torch.float32)
    T, ld = proj.shape
    B = state_slots.numel()
    per_head, per_request = mlstm_state_floats(heads, d, dv)
    if state.dim() != 2 or state.shape[1] != per_request:
        raise KernelError(f"state is {tuple(state.shape)}, expected [slots, {per_request}]")
    if d > MLSTM_MAX_KEY_SIZE:
        raise KernelError(f"key size {d} is beyond the {MLSTM_MAX_KEY_SIZE} the recurrence kernels take")
    if max(col_q + heads * d, col_k + heads * d, col_v + heads * dv, col_i + heads, col_f + heads) > ld:
        raise KernelError("a part of the fused projection lies outside its columns")
    coef = torch.empty((T, heads, 4), dtype=torch.float32, device=proj.device)
    o_raw = torch.empty((T, heads * dv), dtype=torch.float32, device=proj.device)
    nq = torch.empty((T, heads), dtype=torch.float32, device=proj.device)
    check(kernel("sharpi_mlstm_recurrence")(proj.data_ptr(), ld, col_q, col_k, col_v, col_i, col_f, bias_i.data_ptr(),
                                            bias_f.data_ptr(), row_offsets.data_ptr(), state_slots.data_ptr(),
                                            state.data_ptr(), state.stride(0), per_head, B, T, heads, d, dv,
                                            float(cap), float(q_scale), coef.data_ptr(), o_raw.data_ptr(), nq.data_ptr(),
                                            _stream()),
          "sharpi_mlstm_recurrence")
    return o_raw, nq, coef


def mlstm_out(o_raw: torch.Tensor, nq: torch.Tensor, coef: torch.Tensor, proj: torch.Tensor, col_g: int,
              weight: torch.Tensor, eps: float, heads: int, dv: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Per row and head: ``o = num / (max(|n . q|, exp(-m)) + 1e-6)``, then ``o / rms(o) * weight * sigmoid(gate)``
    with the gate read from ``proj[:, col_g:]``."""
    _need(o_raw, "o_raw", torch.float32)
    _need(nq, "nq", torch.float32)
    _need(coef, "coef", torch.float32)
    if nq.numel() != o_raw.shape[0] * heads or coef.numel() != 4 * nq.numel():
        raise KernelError("n . q and the coefficients must hold one entry (four) per row and head")
    _need(proj, "proj", torch.float32)
    _need(weight, "weight", torch.float32)
    T = o_raw.shape[0]
    if weight.numel() != heads * dv or o_raw.shape[1] != heads * dv or col_g + heads * dv > proj.shape[1]:
        raise KernelError("head outputs, gate columns and norm weight disagree on heads * value size")
    out = torch.empty((T, heads * dv), dtype=out_dtype, device=o_raw.device)
    gate = proj[:, col_g:]
    check(kernel("sharpi_mlstm_out")(o_raw.data_ptr(), nq.data_ptr(), coef.data_ptr(), gate.data_ptr(), proj.shape[1], weight.data_ptr(), float(eps), T,
                                     heads, dv, out.data_ptr(), dtype_code(out_dtype), _stream()), "sharpi_mlstm_out")
    return out


_argmax_scratches = {}


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest entry of every row (the lowest index among equals), int32 [R]."""
    _need(logits, "logits", torch.float32)
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    scratch = None
    if R <= 64:       # few rows: every row is cut over 32 blocks; 64 counters (kept at zero), then the slices' candidates
        key = (logits.device, torch.cuda.current_stream(logits.device).cuda_stream)
        scratch = _argmax_scratches.get(key)
        if scratch is None:
            scratch = _argmax_scratches[key] = torch.zeros(64 + 64 * 32 * 2, dtype=torch.int32, device=logits.device)
    check(kernel("sharpi_argmax_rows")(logits.data_ptr(), R, V, out.data_ptr(), _ptr(scratch), _stream()),
          "sharpi_argmax_rows")
    return out


def apply_penalties(logits: torch.Tensor, entry_row: torch.Tensor, entry_token: torch.Tensor,
                    entry_count: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32)
    for name, t in (("entry_row", entry_row), ("entry_token", entry_token), ("entry_count", entry_count)):
        _need(t, name, torch.int32)
    for name, t in (("rep", rep), ("freq", freq), ("pres", pres)):
        _need(t, name, torch.float32)
    check(kernel("sharpi_apply_penalties")(logits.data_ptr(), logits.shape[1], entry_row.data_ptr(),
                                           entry_token.data_ptr(), entry_count.data_ptr(), rep.data_ptr(),
                                           freq.data_ptr(), pres.data_ptr(), entry_row.numel(), _stream()),
          "sharpi_apply_penalties")


def add_logit_bias(logits: torch.Tensor, entry_row: torch.Tensor, entry_token: torch.Tensor,
                   entry_bias: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32)
    _need(entry_row, "entry_row", torch.int32)
    _need(entry_token, "entry_token", torch.int32)
    _need(entry_bias, "entry_bias", torch.float32)
    check(kernel("sharpi_add_logit_bias")(logits.data_ptr(), logits.shape[1], entry_row.data_ptr(),
                                          entry_token.data_ptr(), entry_bias.data_ptr(), entry_row.numel(),
                                          _stream()), "sharpi_add_logit_bias")


_sliced_work = {}
SLICED_SAMPLER_FROM = 4096        # vocabularies from this size on take the sampler that cuts rows over 32 blocks
_SLICED_ROW_BYTES = 56 + 32 * 16 + 2048 * 12


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                min_p: torch.Tensor, uniform: torch.Tensor, *, probs: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, any_top_k: bool = True, any_top_p: bool = True,
                sliced: Optional[bool] = None) -> torch.Tensor:
    """One token per row: greedy where ``temperature <= 0``, else filtered temperature sampling.

    Large vocabularies take the sampler that cuts every row over 32 blocks and finds the thresholds by
    radix selection (``sliced``; ``any_top_k`` / ``any_top_p`` = False skip the passes of a filter that no
    row uses); small ones the one-block-per-row sampler with its ``probs`` work area."""
    _need(logits, "logits", torch.float32)
    R, V = logits.shape
    _need(temperature, "temperature", torch.float32)
    _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32)
    _need(min_p, "min_p", torch.float32)
    _need(uniform, "uniform", torch.float32)
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    if sliced is None:
        sliced = V >= SLICED_SAMPLER_FROM and probs is None
    if sliced:
        key = (logits.device, torch.cuda.current_stream(logits.device).cuda_stream)
        work = _sliced_work.get(key)
        need = R * _SLICED_ROW_BYTES + 256
        if work is None or work.numel() < need:        # all zero before the first call; every call leaves it so
            work = _sliced_work[key] = torch.zeros(max(need, 64 * _SLICED_ROW_BYTES), dtype=torch.uint8,
                                                   device=logits.device)
        check(kernel("sharpi_sample_rows_sliced")(logits.data_ptr(), R, V, temperature.data_ptr(), top_k.data_ptr(),
                                                  top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(),
                                                  work.data_ptr(), int(any_top_k), int(any_top_p), out.data_ptr(),
                                                  _stream()), "sharpi_sample_rows_sliced")
        return out
    if probs is None:
        probs = torch.empty((R, V), dtype=torch.float32, device=logits.device)
    check(kernel("sharpi_sample_rows")(logits.data_ptr(), R, V, temperature.data_ptr(), top_k.data_ptr(),
                                       top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(), probs.data_ptr(),
                                       out.data_ptr(), _stream()), "sharpi_sample_rows")
    return out


# ---------------------------------------------------------------------------------------
# Several residual streams, token shift, hashed pair embedding (hyper.cu)
HC_MAX_STREAMS = 8


def embed_pair(ids: torch.Tensor, embed: torch.Tensor, pairs: torch.Tensor, *, row_request: torch.Tensor,
               row_offsets: torch.Tensor, state_slots: torch.Tensor, prev_state: torch.Tensor, streams: int,
               buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """``embed[token] + pairs[(prev * mul_prev + token * mul_cur) mod buckets]`` (row ``buckets`` for a sequence's
    first token) as float32, written ``streams`` times side by side: ``[T, streams * H]``.  ``prev_state`` int32
    ``[slots]`` holds every request's last token plus one (0: none yet) and is moved on."""
    _need(ids, "ids", torch.int32)
    _need(embed, "embed")
    _need(pairs, "pairs", embed.dtype)
    _need(prev_state, "prev_state", torch.int32)
    for name, t in (("row_request", row_request), ("row_offsets", row_offsets), ("state_slots", state_slots)):
        _need(t, name, torch.int32)
    T, (V, H) = ids.numel(), embed.shape
    if pairs.shape != (buckets + 1, H):
        raise KernelError(f"pair table is {tuple(pairs.shape)}, expected [{buckets + 1}, {H}]")
    out = torch.empty((T, streams * H), dtype=torch.float32, device=embed.device)
    check(kernel("sharpi_embed_pair")(ids.data_ptr(), embed.data_ptr(), pairs.data_ptr(), dtype_code(embed.dtype),
                                      row_request.data_ptr(), row_offsets.data_ptr(), state_slots.data_ptr(),
                                      prev_state.data_ptr(), out.data_ptr(), T, H, streams, V, int(buckets),
                                      int(mul_prev), int(mul_cur), _stream()), "sharpi_embed_pair")
    return out


def hc_mix_norm(x: torch.Tensor, pending, inc: Optional[torch.Tensor], weight: torch.Tensor, *, streams: int,
                groups: int, eps: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x`` float32 ``[T, streams * H]``.  With ``pending = (y, mix, out)``: every stream becomes
    ``x_t <- sum_s mix[s, t] x_s + out[t] y`` (in place; not stored when ``rows`` gathers).  Returns the norm in
    ``groups`` consecutive parts, times ``weight``, of ``sum_t inc[t] x_t`` (the plain sum when ``inc`` is None)
    for every row, or for the rows named by ``rows``."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    H = weight.numel()
    if x.shape[-1] != streams * H:
        raise KernelError(f"x has rows of {x.shape[-1]}, expected streams * width = {streams * H}")
    y = mix = outc = None
    if pending is not None:
        y, mix, outc = pending
        _need(y, "y", torch.float32)
        _need(mix, "mix", torch.float32)
        _need(outc, "out coefficients", torch.float32)
        if mix.numel() != streams * streams or outc.numel() != streams or y.shape[-1] != H:
            raise KernelError("pending update disagrees with the number of streams or the width")
    if inc is not None:
        _need(inc, "in coefficients", torch.float32)
    if rows is not None:
        _need(rows, "rows", torch.int32)
    R = rows.numel() if rows is not None else x.shape[0]
    h = torch.empty((R, H), dtype=out_dtype, device=x.device)
    check(kernel("sharpi_hc_mix_norm")(x.data_ptr(), _ptr(y), _ptr(mix), _ptr(outc), _ptr(inc), weight.data_ptr(),
                                       _ptr(rows), h.data_ptr(), dtype_code(out_dtype), R, H, streams, int(groups),
                                       float(eps), _stream()), "sharpi_hc_mix_norm")
    return h


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, *, row_request: torch.Tensor,
                row_offsets: torch.Tensor, state_slots: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``out[k] = h + (h' - h) * mu[k]`` for the K rows of ``mu`` ``[K, H]``; ``h'`` is the previous row of the same
    request, or ``state[slot]`` for the first row of a portion; ``state[slot]`` becomes the portion's last ``h``.
    ``[K, T, H]`` in ``out_dtype``."""
    _need(h, "h", torch.float32)
    _need(mu, "mu", torch.float32)
    _need(state, "state", torch.float32)
    T, H = h.shape
    K = mu.numel() // H
    if mu.numel() != K * H or state.shape[-1] != H:
        raise KernelError("mu or state disagree with the width")
    out = torch.empty((K, T, H), dtype=out_dtype, device=h.device)
    check(kernel("sharpi_token_shift")(h.data_ptr(), mu.data_ptr(), state.data_ptr(), state.stride(0),
                                       row_request.data_ptr(), row_offsets.data_ptr(), state_slots.data_ptr(),
                                       out.data_ptr(), dtype_code(out_dtype), T, H, K, _stream()), "sharpi_token_shift")
    return out


def norm_mean2(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, eps: float,
               scale: float = 0.5) -> torch.Tensor:
    """``scale * (rms(a) * wa + rms(b) * wb)`` row by row, float32."""
    for name, t in (("a", a), ("b", b), ("wa", wa), ("wb", wb)):
        _need(t, name, torch.float32)
    T, H = a.shape
    if b.shape != a.shape or wa.numel() != H or wb.numel() != H:
        raise KernelError("branches and weights disagree on the width")
    out = torch.empty_like(a)
    check(kernel("sharpi_norm_mean2")(a.data_ptr(), wa.data_ptr(), b.data_ptr(), wb.data_ptr(), out.data_ptr(), T, H,
                                      float(eps), float(scale), _stream()), "sharpi_norm_mean2")
    return out


# ---------------------------------------------------------------------------------------
# WKV recurrence (wkv.cu)
WKV_MAX_HEAD_SIZE = 256


def wkv_recurrence(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, wraw: torch.Tensor, w0: torch.Tensor,
                   u: torch.Tensor, *, row_offsets: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor,
                   heads: int, d: int) -> torch.Tensor:
    """``o_t = (S + diag(u) k_t v_t^T)^T r_t``, ``S <- diag(exp(-exp(wraw_t + w0))) S + k_t v_t^T`` per head over
    the rows of every request, from and into ``state [slots, heads * d * d]``; float32 ``[T, heads * d]``.
    ``wraw`` is overwritten (with the decay, for heads of up to 128 elements)."""
    for name, t in (("r", r), ("k", k), ("v", v), ("wraw", wraw), ("w0", w0), ("u", u), ("state", state)):
        _need(t, name, torch.float32)
    T = r.shape[0]
    if any(t.shape != (T, heads * d) for t in (r, k, v, wraw)) or w0.numel() != heads * d or u.numel() != heads * d:
        raise KernelError("r, k, v, the raw decay, w0 and u must all be heads * d wide")
    if state.shape[-1] != heads * d * d:
        raise KernelError(f"state is {tuple(state.shape)}, expected [slots, {heads * d * d}]")
    o = torch.empty((T, heads * d), dtype=torch.float32, device=r.device)
    bonus = torch.empty((T, heads), dtype=torch.float32, device=r.device)
    check(kernel("sharpi_wkv_recurrence")(r.data_ptr(), k.data_ptr(), v.data_ptr(), wraw.data_ptr(), w0.data_ptr(),
                                          u.data_ptr(), row_offsets.data_ptr(), state_slots.data_ptr(),
                                          state.data_ptr(), state.stride(0), o.data_ptr(), bonus.data_ptr(), T,
                                          state_slots.numel(), heads, d, _stream()), "sharpi_wkv_recurrence")
    return o


def wkv_out(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, heads: int, d: int,
            out_dtype: torch.dtype) -> torch.Tensor:
    """Every head of ``o`` divided by its root mean square, times ``weight`` and ``silu(gate)``."""
    _need(o, "o", torch.float32)
    _need(gate, "gate", torch.float32)
    _need(weight, "weight", torch.float32)
    T = o.shape[0]
    out = torch.empty((T, heads * d), dtype=out_dtype, device=o.device)
    check(kernel("sharpi_wkv_out")(o.data_ptr(), gate.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                   dtype_code(out_dtype), T, heads, d, float(eps), _stream()), "sharpi_wkv_out")
    return out


# ---------------------------------------------------------------------------------------
# Selective scan and its convolution (mamba.cu)
SCAN_MAX_STATES = 256


def causal_conv(xz: torch.Tensor, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                state: torch.Tensor, *, row_request: torch.Tensor, row_offsets: torch.Tensor,
                state_slots: torch.Tensor, act_dtype: torch.dtype, gate_col: int = -1):
    """``silu`` of the causal convolution of the first ``channels`` columns of ``xz`` (float32 ``[T, ld]``) with
    ``weight [channels, taps]`` (last column: the current token) and ``bias``; inputs before a portion come from
    ``state [slots, (taps - 1) * channels]``, which is moved on.  Returns ``(x32, x_act)``.  With ``gate_col`` the
    columns ``gate_col .. gate_col + channels - 1`` of ``xz`` are replaced by their ``silu`` in the same pass."""
    _need(xz, "xz", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(state, "state", torch.float32)
    T, ld = xz.shape
    taps = weight.numel() // channels
    if weight.numel() != channels * taps or state.shape[-1] != max(taps - 1, 1) * channels or channels > ld:
        raise KernelError("convolution weight, state and input disagree on channels or taps")
    x32 = torch.empty((T, channels), dtype=torch.float32, device=xz.device)
    xact = x32 if act_dtype == torch.float32 else torch.empty((T, channels), dtype=act_dtype, device=xz.device)
    check(kernel("sharpi_causal_conv")(xz.data_ptr(), ld, weight.data_ptr(), _ptr(bias), state.data_ptr(),
                                       state.stride(0), row_request.data_ptr(), row_offsets.data_ptr(),
                                       state_slots.data_ptr(), x32.data_ptr(),
                                       None if act_dtype == torch.float32 else xact.data_ptr(), dtype_code(act_dtype),
                                       T, state_slots.numel(), channels, taps, int(gate_col), _stream()),
          "sharpi_causal_conv")
    return x32, xact


def slice_cols(src: torch.Tensor, col0: int, ncols: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Columns ``col0 .. col0 + ncols - 1`` of a float32 matrix, contiguous, in ``out_dtype``."""
    _need(src, "src", torch.float32)
    T, ld = src.shape
    out = torch.empty((T, ncols), dtype=out_dtype, device=src.device)
    check(kernel("sharpi_slice_cols")(src.data_ptr(), ld, col0, ncols, out.data_ptr(), dtype_code(out_dtype), T,
                                      _stream()), "sharpi_slice_cols")
    return out


def selective_scan(x: torch.Tensor, dt: torch.Tensor, bc: torch.Tensor, col_b: int,
                   col_c: int, a_log: torch.Tensor, dskip: torch.Tensor, xz: torch.Tensor, col_z: int, *,
                   row_offsets: torch.Tensor, state_slots: torch.Tensor, state: torch.Tensor,
                   out_dtype: torch.dtype) -> torch.Tensor:
    """The selective scan over the rows of every request from and into ``state [slots, channels * states]``:
    ``(S C + D x) * g`` in ``out_dtype``, with ``dt`` the step sizes themselves (after their softplus) and ``g`` the
    gate (already ``silu(z)``) in the columns of ``xz`` from ``col_z``."""
    for name, t in (("x", x), ("dt", dt), ("bc", bc), ("a_log", a_log), ("dskip", dskip),
                    ("xz", xz), ("state", state)):
        _need(t, name, torch.float32)
    T, C = x.shape
    N = a_log.numel() // C
    if dt.shape != (T, C) or a_log.numel() != C * N or state.shape[-1] != C * N or max(col_b, col_c) + N > bc.shape[1]:
        raise KernelError("scan inputs disagree on channels or states")
    if col_z + C > xz.shape[1]:
        raise KernelError("the gate's columns lie outside the fused projection")
    out = torch.empty((T, C), dtype=out_dtype, device=x.device)
    z = xz[:, col_z:]
    check(kernel("sharpi_selective_scan")(x.data_ptr(), dt.data_ptr(), bc.data_ptr(),
                                          bc.shape[1], col_b, col_c, a_log.data_ptr(), dskip.data_ptr(), z.data_ptr(),
                                          xz.shape[1], row_offsets.data_ptr(), state_slots.data_ptr(), state.data_ptr(),
                                          state.stride(0), out.data_ptr(), dtype_code(out_dtype), T, state_slots.numel(),
                                          C, N, _stream()), "sharpi_selective_scan")
    return out


# ---------------------------------------------------------------------------------------
def qkv_post_rot(qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor,
                 q_out: torch.Tensor, kv_layer: torch.Tensor, *, nq: int, nkv: int, D: int, key_dim: int,
                 value_dim: int, page_size: int, pairing: int, q_norm_weight: Optional[torch.Tensor],
                 k_norm_weight: Optional[torch.Tensor], eps: float, inv_freq: Optional[torch.Tensor], rot_dims: int,
                 inv_freq_v: Optional[torch.Tensor], v_rot_dims: int, write_kv: bool = True) -> None:
    """The general form of :func:`qkv_post`: weighted RMS norm of q and k before the rotation, rotation of the first
    ``rot_dims`` elements, values rotated over their first ``v_rot_dims`` elements with ``inv_freq_v``."""
    _need(qkv, "qkv", torch.float32)
    T = positions.numel()
    if qkv.shape != (T, (nq + 2 * nkv) * D):
        raise KernelError(f"qkv is {tuple(qkv.shape)}, expected [{T}, {(nq + 2 * nkv) * D}]")
    for name, t in (("q norm weight", q_norm_weight), ("k norm weight", k_norm_weight)):
        if t is not None:
            _need(t, name, torch.float32)
            if t.numel() != key_dim:
                raise KernelError(f"{name} has {t.numel()} entries, the key size is {key_dim}")
    if inv_freq is not None and inv_freq.numel() != rot_dims // 2:
        raise KernelError(f"inv_freq has {inv_freq.numel()} entries, {rot_dims} rotated elements need {rot_dims // 2}")
    if inv_freq_v is not None and inv_freq_v.numel() != v_rot_dims // 2:
        raise KernelError(f"the values' inv_freq has {inv_freq_v.numel()} entries, expected {v_rot_dims // 2}")
    check(kernel("sharpi_qkv_post_rot")(qkv.data_ptr(), positions.data_ptr(), row_req.data_ptr(), block_table.data_ptr(),
                                        _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps), _ptr(inv_freq),
                                        int(rot_dims if inv_freq is not None else 0), _ptr(inv_freq_v),
                                        int(v_rot_dims if inv_freq_v is not None else 0), pairing, q_out.data_ptr(),
                                        kv_layer.data_ptr(), dtype_code(q_out.dtype), T, nq, nkv, D, key_dim, value_dim,
                                        block_table.shape[-1], page_size, int(write_kv), _stream()),
          "sharpi_qkv_post_rot")


def rotate_heads(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, *, heads: int, D: int,
                 rot_dims: int, pairing: int, sign: float, out_dtype: torch.dtype) -> torch.Tensor:
    """Every head of ``x [T, heads * D]`` turned by ``sign * position`` over its first ``rot_dims`` elements."""
    _need(x, "x")
    _need(inv_freq, "inv_freq", torch.float32)
    T = positions.numel()
    out = torch.empty((T, heads * D), dtype=out_dtype, device=x.device)
    check(kernel("sharpi_rotate_heads")(x.data_ptr(), dtype_code(x.dtype), positions.data_ptr(), inv_freq.data_ptr(),
                                        out.data_ptr(), dtype_code(out_dtype), T, heads, D, rot_dims, pairing,
                                        float(sign), _stream()), "sharpi_rotate_heads")
    return out


def gated_act(gate_up: torch.Tensor, act: int, out_dtype: torch.dtype) -> torch.Tensor:
    """``act(g) * u`` over a fused ``[M, 2I]`` gate|up product (float32 in)."""
    _need(gate_up, "gate_up", torch.float32)
    M, I2 = gate_up.shape
    out = torch.empty((M, I2 // 2), dtype=out_dtype, device=gate_up.device)
    check(kernel("sharpi_gated_act")(gate_up.data_ptr(), out.data_ptr(), dtype_code(out_dtype), M, I2 // 2, int(act),
                                     _stream()), "sharpi_gated_act")
    return out


def tanh(y: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    _need(y, "y", torch.float32)
    out = torch.empty(y.shape, dtype=out_dtype, device=y.device)
    check(kernel("sharpi_tanh")(y.data_ptr(), out.data_ptr(), dtype_code(out_dtype), y.numel(), _stream()), "sharpi_tanh")
    return out


def scale_(y: torch.Tensor, s: float) -> torch.Tensor:
    _need(y, "y", torch.float32)
    check(kernel("sharpi_scale")(y.data_ptr(), float(s), y.numel(), _stream()), "sharpi_scale")
    return y


# ---------------------------------------------------------------------------------------
# the element-wise squashing norm, latent attention, the state-space-duality scan
# ---------------------------------------------------------------------------------------
def add_dyt(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
            alpha: torch.Tensor, out_dtype: torch.dtype, *, rows: Optional[torch.Tensor] = None,
            want_fp32: bool = False):
    """Residual add fused with ``tanh(alpha x) w + b`` (``alpha`` a float32 tensor of one element).  The interface of
    :func:`add_rmsnorm`: without ``rows`` ``x += delta`` in place, with ``rows`` the gathered rows and ``x`` stays.
    Returns ``(out, out32)``."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(alpha, "alpha", torch.float32)
    H = x.shape[-1]
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if weight.numel() != H or (bias is not None and bias.numel() != H) or alpha.numel() != 1:
        raise KernelError(f"weight, bias or alpha disagree with the width {H}")
    if delta is not None:
        _need(delta, "delta", torch.float32)
        if delta.shape != x.shape:
            raise KernelError(f"delta shape {tuple(delta.shape)} differs from x shape {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        T = rows.numel()
    else:
        T = x.numel() // H
    out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    out32 = None
    if want_fp32:
        out32 = out if out_dtype == torch.float32 else torch.empty((T, H), dtype=torch.float32, device=x.device)
    alias = out32 is not None and out32.data_ptr() == out.data_ptr()
    check(kernel("sharpi_add_dyt")(x.data_ptr(), _ptr(delta), weight.data_ptr(), _ptr(bias), alpha.data_ptr(), _ptr(rows),
                                   T, H, out.data_ptr(), dtype_code(out_dtype), None if alias else _ptr(out32), _stream()),
          "sharpi_add_dyt")
    return out, out32


def latent_down_post(down: torch.Tensor, *, q_rank: int, rank: int, rot: int, rot_dims: int,
                     q_norm_weight: Optional[torch.Tensor], c_norm_weight: torch.Tensor, eps: float,
                     positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor,
                     inv_freq: Optional[torch.Tensor], kv_layer: torch.Tensor, page_size: int,
                     write_kv: bool = True, rot_amplitude: float = 1.0) -> torch.Tensor:
    """Behind the fused down projection ``down`` float32 ``[T, q_rank + rank + rot]`` of latent attention: the normed
    query latent ``[T, q_rank]`` in the cache's dtype (returned), and ``[c | k_rot | 0]`` written into every row's
    place in ``kv_layer [pages, planes, 1, page_size, D]`` (``[c | 0]`` into the value plane when there are two).
    ``down`` may be a column range of a wider product (rows apart); ``rot_amplitude`` multiplies the rotation's
    cosines and sines."""
    ld = _need_columns(down, "down", torch.float32)
    _need(c_norm_weight, "c_norm_weight", torch.float32)
    _need(kv_layer, "kv_layer")
    T = down.shape[0]
    planes, D = int(kv_layer.shape[1]), int(kv_layer.shape[-1])
    if tuple(kv_layer.shape[1:]) != (planes, 1, page_size, D) or down.shape[1] != q_rank + rank + rot:
        raise KernelError(f"kv_layer {tuple(kv_layer.shape)} or the projection's width {ld} disagree with the sizes")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rot_dims // 2:
            raise KernelError(f"{rot_dims} rotated elements need {rot_dims // 2} frequencies, found {inv_freq.numel()}")
    cq = torch.empty((T, q_rank), dtype=kv_layer.dtype, device=down.device)
    check(kernel("sharpi_latent_down_post")(down.data_ptr(), ld, q_rank, rank, rot, rot_dims if inv_freq is not None else 0,
                                            _ptr(q_norm_weight), c_norm_weight.data_ptr(), float(eps), positions.data_ptr(),
                                            row_req.data_ptr(), block_table.data_ptr(), block_table.shape[-1], page_size,
                                            _ptr(inv_freq), cq.data_ptr(), kv_layer.data_ptr(), planes, D, int(write_kv),
                                            dtype_code(kv_layer.dtype), T, float(rot_amplitude), _stream()),
          "sharpi_latent_down_post")
    return cq


def head_major(src: torch.Tensor, *, heads: int, stride: int, col0: int, n: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Columns ``[col0, col0 + n)`` of every head of ``src [T, heads * stride]`` as ``[heads * T, n]`` (head by head,
    the rows of a head in order) in ``out_dtype``: the operand of a product with one weight a head.  ``src`` may be a
    column range of a wider tensor."""
    ld = _need_columns(src, "src")
    T = src.shape[0]
    if src.shape[1] != heads * stride:
        raise KernelError(f"src is {tuple(src.shape)}, expected [T, {heads} * {stride}]")
    out = torch.empty((heads * T, n), dtype=out_dtype, device=src.device)
    check(kernel("sharpi_head_major")(src.data_ptr(), dtype_code(src.dtype), T, heads, stride, col0, n, out.data_ptr(),
                                      dtype_code(out_dtype), ld, _stream()), "sharpi_head_major")
    return out


def head_minor(src: torch.Tensor, *, heads: int, out_dtype: torch.dtype, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``src`` float32 ``[heads * T, n]`` (head by head) as ``[T, heads * n]`` in ``out_dtype``.  ``gate`` float32
    ``[T, heads]`` (possibly a column range of a wider product): head ``h`` of row ``t`` is multiplied by
    ``sigmoid(gate[t, h])``."""
    _need(src, "src", torch.float32)
    n = src.shape[1]
    T = src.shape[0] // heads
    gate_ld = 0
    if gate is not None:
        gate_ld = _need_columns(gate, "gate", torch.float32)
        if tuple(gate.shape) != (T, heads):
            raise KernelError(f"gate is {tuple(gate.shape)}, expected [{T}, {heads}]")
    out = torch.empty((T, heads * n), dtype=out_dtype, device=src.device)
    check(kernel("sharpi_head_minor")(src.data_ptr(), T, heads, n, 0, n, out.data_ptr(), dtype_code(out_dtype),
                                      _ptr(gate), gate_ld, _stream()), "sharpi_head_minor")
    return out


def latent_q_join(qa: torch.Tensor, q: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], *,
                  heads: int, dim: int, rank: int, rot: int, rot_dims: int, D: int, out_dtype: torch.dtype,
                  rot_amplitude: float = 1.0) -> torch.Tensor:
    """The query rows of latent attention, ``[T, heads, D]``: ``[qa[h, t] | rotate(q[t, h, dim:]) | 0]`` with ``qa``
    float32 ``[heads * T, rank]`` (head by head) and ``q`` float32 ``[T, heads * (dim + rot)]`` (possibly a column range
    of a wider product); ``rot_amplitude`` multiplies the rotation's cosines and sines."""
    _need(qa, "qa", torch.float32)
    ldq = _need_columns(q, "q", torch.float32)
    T = q.shape[0]
    if q.shape[1] != heads * (dim + rot) or tuple(qa.shape) != (heads * T, rank):
        raise KernelError(f"q {tuple(q.shape)} or qa {tuple(qa.shape)} disagree with the sizes")
    out = torch.empty((T, heads, D), dtype=out_dtype, device=q.device)
    check(kernel("sharpi_latent_q_join")(qa.data_ptr(), q.data_ptr(), positions.data_ptr(), _ptr(inv_freq), T, heads, dim,
                                         rank, rot, rot_dims if inv_freq is not None else 0, D, out.data_ptr(),
                                         dtype_code(out_dtype), ldq, float(rot_amplitude), _stream()), "sharpi_latent_q_join")
    return out


SSD_MAX_STATES = 256


def ssd_scan(xbc: torch.Tensor, proj: torch.Tensor, *, col_x: int, col_b: int, col_c: int, col_dt: int,
             dt_bias: torch.Tensor, a_log: torch.Tensor, dskip: torch.Tensor, row_offsets: torch.Tensor,
             state_slots: torch.Tensor, state: torch.Tensor, heads: int, groups: int, states: int, vdim: int) -> torch.Tensor:
    """The state-space-duality recurrence over the rows of every request, from and into ``state [slots, heads *
    states * vdim]``: ``y`` float32 ``[T, heads * vdim]``.  ``xbc`` float32 holds x, B and C at the given columns,
    ``proj`` float32 the raw step sizes at ``col_dt``; ``dt = softplus(raw + dt_bias)``, decay ``exp(-exp(A_log) dt)``."""
    for name, t in (("xbc", xbc), ("proj", proj), ("dt_bias", dt_bias), ("a_log", a_log), ("dskip", dskip), ("state", state)):
        _need(t, name, torch.float32)
    T = xbc.shape[0]
    if state.shape[-1] != heads * states * vdim or min(dt_bias.numel(), a_log.numel(), dskip.numel()) < heads:
        raise KernelError("scan inputs disagree on heads, states or the value size")
    y = torch.empty((T, heads * vdim), dtype=torch.float32, device=xbc.device)
    check(kernel("sharpi_ssd_scan")(xbc.data_ptr(), xbc.shape[1], col_x, col_b, col_c, proj.data_ptr(), proj.shape[1], col_dt,
                                    dt_bias.data_ptr(), a_log.data_ptr(), dskip.data_ptr(), row_offsets.data_ptr(),
                                    state_slots.data_ptr(), state.data_ptr(), state.stride(0), y.data_ptr(), T,
                                    state_slots.numel(), heads, groups, states, vdim, _stream()), "sharpi_ssd_scan")
    return y


def gated_group_norm(y: torch.Tensor, proj: torch.Tensor, col_z: int, weight: torch.Tensor, eps: float, parts: int,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """``u = y * silu(z)`` with ``z`` the columns of ``proj`` from ``col_z``; ``u`` divided by its root mean square in
    ``parts`` equal parts of the width, times ``weight``; ``[T, width]`` in ``out_dtype``."""
    _need(y, "y", torch.float32)
    _need(proj, "proj", torch.float32)
    _need(weight, "weight", torch.float32)
    T, width = y.shape
    if col_z + width > proj.shape[1] or weight.numel() != width or width % parts:
        raise KernelError("the gate's columns, the weight or the parts disagree with the width")
    out = torch.empty((T, width), dtype=out_dtype, device=y.device)
    z = proj[:, col_z:]
    check(kernel("sharpi_gated_group_norm")(y.data_ptr(), z.data_ptr(), proj.shape[1], weight.data_ptr(), float(eps), T, width,
                                            parts, out.data_ptr(), dtype_code(out_dtype), _stream()), "sharpi_gated_group_norm")
    return out


def sigmoid_gate(o: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """``o * sigmoid(g)`` element by element: ``o [rows, cols]`` in the activation dtype, ``g`` float32 of the same
    shape (possibly a column range of a wider product)."""
    _need(o, "o")
    g_ld = _need_columns(g, "g", torch.float32)
    if o.shape != g.shape:
        raise KernelError(f"shapes differ: {tuple(o.shape)}, {tuple(g.shape)}")
    out = torch.empty_like(o)
    check(kernel("sharpi_sigmoid_gate")(o.data_ptr(), g.data_ptr(), out.data_ptr(), dtype_code(o.dtype), o.numel(),
                                        int(o.shape[1]), g_ld, _stream()), "sharpi_sigmoid_gate")
    return out


def add_layernorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
                  eps: float, out_dtype: torch.dtype, *, rows: Optional[torch.Tensor] = None, want_fp32: bool = False):
    """Residual add fused with a layer norm, ``(x - mean) / sqrt(var + eps) * w + b`` with ``var`` the mean of the
    squared deviations.  The interface of :func:`add_rmsnorm`: without ``rows`` ``x += delta`` in place, with ``rows``
    the gathered rows and ``x`` stays.  Returns ``(out, out32)``."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    H = x.shape[-1]
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if weight.numel() != H or (bias is not None and bias.numel() != H):
        raise KernelError(f"weight or bias disagree with the width {H}")
    if delta is not None:
        _need(delta, "delta", torch.float32)
        if delta.shape != x.shape:
            raise KernelError(f"delta shape {tuple(delta.shape)} differs from x shape {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        T = rows.numel()
    else:
        T = x.numel() // H
    out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    out32 = None
    if want_fp32:
        out32 = out if out_dtype == torch.float32 else torch.empty((T, H), dtype=torch.float32, device=x.device)
    alias = out32 is not None and out32.data_ptr() == out.data_ptr()
    check(kernel("sharpi_add_layernorm")(x.data_ptr(), _ptr(delta), weight.data_ptr(), _ptr(bias), float(eps), _ptr(rows),
                                         T, H, out.data_ptr(), dtype_code(out_dtype), None if alias else _ptr(out32),
                                         _stream()), "sharpi_add_layernorm")
    return out, out32


def qkv_post_wide(qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor,
                  q_out: torch.Tensor, kv_layer: torch.Tensor, *, nq: int, nkv: int, d: int, page_size: int,
                  q_weight: torch.Tensor, k_weight: Optional[torch.Tensor], eps: float, q_count: int, k_count: int,
                  temp_coef: float, temp_every: float, write_kv: bool, has_kv: bool) -> None:
    """Behind a fused projection ``qkv`` float32 ``[T, (nq + 2 nkv) d]`` (or ``[T, nq d]`` when ``has_kv`` is false: the
    layer reads another layer's cache): q as a whole is divided by its root mean square (``sqrt(sum / q_count + eps)``)
    and multiplied by ``q_weight [nq d]``, k likewise with ``k_weight``; q also by ``1 + temp_coef * ln(1 + floor((pos +
    1) / temp_every))`` when ``temp_every > 0``; q goes to ``q_out [T, nq, d]``, k and v into ``kv_layer [pages, 2, nkv,
    page_size, d]`` at every row's position."""
    ld = _need_columns(qkv, "qkv", torch.float32)
    _need(q_out, "q_out")
    _need(kv_layer, "kv_layer", q_out.dtype)
    _need(q_weight, "q_weight", torch.float32)
    T = positions.numel()
    width = (nq + 2 * nkv) * d if has_kv else nq * d
    if tuple(qkv.shape) != (T, width) or q_weight.numel() != nq * d:
        raise KernelError(f"qkv {tuple(qkv.shape)} is not [{T}, {width}] or the q weight has {q_weight.numel()} entries")
    if has_kv:
        _need(k_weight, "k_weight", torch.float32)
        if k_weight.numel() != nkv * d:
            raise KernelError(f"the k weight has {k_weight.numel()} entries, expected {nkv * d}")
    if tuple(kv_layer.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv_layer shape {tuple(kv_layer.shape)} is not [pages, 2, {nkv}, {page_size}, {d}]")
    check(kernel("sharpi_qkv_post_wide")(qkv.data_ptr(), ld, positions.data_ptr(), row_req.data_ptr(),
                                         block_table.data_ptr(), q_weight.data_ptr(), _ptr(k_weight), float(eps),
                                         int(q_count), int(k_count), q_out.data_ptr(), kv_layer.data_ptr(),
                                         dtype_code(q_out.dtype), T, nq, nkv, d, block_table.shape[-1], page_size,
                                         float(temp_coef), float(temp_every), int(write_kv), int(has_kv), _stream()),
          "sharpi_qkv_post_wide")
