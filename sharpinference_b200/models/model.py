"""``DecoderModel``: embedding, a schedule of blocks, final norm and output head.

The schedule is data: a list of entries that name the block to run and, optionally, an earlier
entry whose cache this one reads instead of writing its own.  A block may be named more than
once (its weights are shared; each entry has a cache of its own unless it borrows one).  The
reference's precedent for borrowing is its key/value sharing between layers
(src/SharpInference.Engine/CudaSequenceKvCache.cs:25-33); its layer loop is fixed,
``for layer in 0..L`` (src/SharpInference.Engine/ForwardPass.cs:1539-1730).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from ..parts.base import Block, Norm, StepContext, StreamOp
from ..parts.linear import Linear


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                          # index into DecoderModel.blocks
    cache_from: Optional[int] = None    # schedule index whose cache this entry reads (no write of its own)
    before: Optional[int] = None        # index into DecoderModel.stream_ops: run on the stream before this block


class DecoderModel:
    def __init__(self, *, embedding: torch.Tensor, blocks: Sequence[Block], final_norm: Norm, head: Linear,
                 act_dtype: torch.dtype, schedule: Optional[Sequence[ScheduleEntry]] = None,
                 eos_token_ids: Sequence[int] = (), config=None, stream_ops: Sequence[StreamOp] = (),
                 embedder=None, logit_scale: float = 1.0, embedding_scale: float = 1.0):
        """``embedder``: a part whose ``forward(ctx)`` gives the float32 residual stream(s) of the step's rows
        in place of the plain table lookup (its ``state_specs`` become per-request state of the model);
        ``logit_scale`` multiplies the head's output, ``embedding_scale`` the looked-up embedding row."""
        self.embedding = embedding                  # [V, H]
        self.blocks: List[Block] = list(blocks)
        self.stream_ops: List[StreamOp] = list(stream_ops)
        self.final_norm = final_norm
        self.head = head
        self.act_dtype = act_dtype
        self.schedule: List[ScheduleEntry] = (list(schedule) if schedule is not None
                                              else [ScheduleEntry(i) for i in range(len(self.blocks))])
        self.vocab_size, self.hidden_size = embedding.shape
        self.eos_token_ids = tuple(eos_token_ids)
        self.config = config
        self.embedder = embedder
        self.state_specs = dict(getattr(embedder, "state_specs", None) or {})
        self.logit_scale = float(logit_scale)
        self.embedding_scale = float(embedding_scale)
        self._validate_schedule()

    def set_schedule(self, schedule: Sequence[ScheduleEntry]) -> "DecoderModel":
        """Replace the order in which blocks run (before a cache manager is made for the model)."""
        self.schedule = list(schedule)
        self._validate_schedule()
        return self

    def _validate_schedule(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"schedule entry {i} names block {e.layer}; the model has {len(self.blocks)}")
            if e.before is not None and not (0 <= e.before < len(self.stream_ops)):
                raise ValueError(f"schedule entry {i} names stream operation {e.before}; the model has "
                                 f"{len(self.stream_ops)}")
            if e.cache_from is not None:
                if not (0 <= e.cache_from < i):
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which must come earlier")
                src = self.schedule[e.cache_from]
                if src.cache_from is not None:
                    raise ValueError(f"schedule entry {i} reads entry {e.cache_from}, which itself borrows a cache")
                a = self.blocks[e.layer].mixer.cache_spec
                b = self.blocks[src.layer].mixer.cache_spec
                if a is None or b is None or a != b:
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {e.cache_from}: "
                                     f"their cache needs differ ({a} against {b})")

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Run the step's rows through every scheduled block; float32 logits ``[R, V]`` at
        ``ctx.want_rows`` (None if no logits are wanted)."""
        x = self.embedder.forward(ctx) if self.embedder is not None else ops.embed_gather(ctx.token_ids, self.embedding)
        if self.embedding_scale != 1.0:
            ops.scale_(x, self.embedding_scale)
        # stream operations read the embedding output; the blocks add into x in place, so it is gathered twice
        x0 = ops.embed_gather(ctx.token_ids, self.embedding) if self.stream_ops else None
        pending = None
        norms = ctx.extras.get("layer_norms")        # tracing: see StepRunner.trace_layers
        streams = ctx.extras.get("layer_streams")    # tracing: the whole residual stream after every block
        for index, entry in enumerate(self.schedule):
            if entry.before is not None:
                x, pending = self.stream_ops[entry.before].forward(ctx, x, pending, x0)
            x, pending = self.blocks[entry.layer].forward(ctx, ctx.slots[index], x, pending)
            if norms is not None or streams is not None:
                traced = getattr(self.blocks[entry.layer], "traced_stream", None)
                if traced is not None:
                    after = traced(x, pending)
                else:
                    after = x.float() if pending is None else x.float() + pending.float()
                if norms is not None:
                    norms.append(after.square().sum(dim=1).sqrt())
                if streams is not None:
                    streams.append(after.clone())
        if ctx.want_rows is None or ctx.want_rows.numel() == 0:
            return None
        h, _ = self.final_norm.apply(x, pending, rows=ctx.want_rows, out_dtype=self.act_dtype)
        logits = self.head(h)
        return ops.scale_(logits, self.logit_scale) if self.logit_scale != 1.0 else logits
