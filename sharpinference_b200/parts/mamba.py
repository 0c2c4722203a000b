"""The selective state-space mixer (Mamba), its state-space-duality form with a scalar decay per head (Mamba-2), and
the mixer that runs two mixers side by side.

``SelectiveScanMixer``: ``W_in h = [x | z]`` (``inner`` channels each).  ``x`` passes a causal convolution per channel
(``taps`` inputs, the last weight column is the current token's, zeros before a sequence's start) with a bias, then
silu.  ``W_x x = [dt_in (dt_rank) | B (states) | C (states)]``; ``dt = softplus(W_dt dt_in + dt_bias)`` per channel;
``A = -exp(A_log)`` ``[inner, states]``.  Per channel c and state n:

    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n ;   y_c = sum_n S[c, n] C_n + D_c x_c

and the result is ``W_o (y * silu(z))``.  The convolution, step sizes, exponentials, state and sums are float32;
the projections round their inputs to the activation dtype.  Per-request state: ``S`` (``state_specs["S"]``) and
the convolution's last ``taps - 1`` inputs (``state_specs["conv"]``), both zero at a sequence's start
(``csrc/mamba.cu``).

``StateSpaceDualityMixer``: ``W_in h = [x (heads * vdim) | B (groups * states) | C (groups * states) | z (heads * vdim)
| dt (heads)]`` (the builder orders the projection's rows so).  ``x``, ``B`` and ``C`` together pass the causal
convolution with its bias and silu.  ``dt = softplus(dt + dt_bias)`` per head; per head ``h`` of group ``g``:

    S_h <- exp(-exp(A_log_h) dt_h) S_h + dt_h B_g x_h^T     (S_h is states x vdim) ;   y_h = S_h^T C_g + D_h x_h

then ``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts of its width, each by its own root mean square,
times a weight, and ``W_o`` follows.  Convolution, step sizes, decays, state, sums and the norm are float32.
Per-request state: ``S`` and the convolution's last ``taps - 1`` inputs (``csrc/mamba2.cu``, ``csrc/mamba.cu``).

``BranchPair``: two mixers that read the same input; the result is ``scale * (rms(left) * w_left + rms(right) *
w_right)``, each branch's output normed over the model width with a plain weight first.  The pair owns the cache
of whichever branch keeps keys and values and the state of both (names prefixed ``left.`` / ``right.``).
"""
from __future__ import annotations

from dataclasses import replace
from typing import Optional

import torch

from ..kernels import ops
from .base import LayerSlot, Mixer, StateSpec, StepContext, register_part
from .linear import Linear


@register_part("mixer", "selective_scan")
class SelectiveScanMixer(Mixer):
    graph_safe = True
    cache_spec = None

    def __init__(self, *, in_proj: Linear, conv_weight: torch.Tensor, conv_bias: Optional[torch.Tensor],
                 x_proj: Linear, dt_proj: Linear, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
                 out: Linear, inner: int, states: int, dt_rank: int, taps: int,
                 act_dtype: torch.dtype = torch.bfloat16):
        if in_proj.out_features != 2 * inner or x_proj.in_features != inner or out.in_features != inner:
            raise ValueError(f"the projections disagree with the inner size {inner}")
        if x_proj.out_features != dt_rank + 2 * states or dt_proj.in_features != dt_rank or dt_proj.out_features != inner:
            raise ValueError("the step-size projections disagree with dt_rank, the number of states or the inner size")
        if conv_weight.numel() != inner * taps or a_log.numel() != inner * states:
            raise ValueError("the convolution weight or A_log disagree with inner, taps or states")
        if states > ops.SCAN_MAX_STATES or taps < 1:
            raise ValueError(f"{states} states (at most {ops.SCAN_MAX_STATES}) or {taps} taps are not supported")
        self.in_proj, self.x_proj, self.dt_proj, self.out = in_proj, x_proj, dt_proj, out
        self.conv_weight, self.conv_bias, self.dt_bias, self.a_log, self.d_skip = conv_weight, conv_bias, dt_bias, a_log, d_skip
        self.inner, self.states, self.dt_rank, self.taps, self.act_dtype = inner, states, dt_rank, taps, act_dtype
        self.state_specs = {"S": StateSpec((inner * states,), torch.float32),
                            "conv": StateSpec((max(taps - 1, 1) * inner,), torch.float32)}

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        xz = self.in_proj(h)                                                     # [T, 2 inner] float32
        x32, xact = ops.causal_conv(xz, self.inner, self.conv_weight, self.conv_bias, slot.states["conv"],
                                    row_request=ctx.row_request, row_offsets=ctx.row_offsets,
                                    state_slots=ctx.state_slots, act_dtype=self.act_dtype, gate_col=self.inner)
        dbc = self.x_proj(xact)                                                  # [T, dt_rank + 2 states] float32
        dt = self.dt_proj(ops.slice_cols(dbc, 0, self.dt_rank, self.act_dtype))
        ops.bias_act(dt, self.dt_bias, ops.ACT_SOFTPLUS, torch.float32, out=dt)  # the step sizes, in place
        y = ops.selective_scan(x32, dt, dbc, self.dt_rank, self.dt_rank + self.states, self.a_log,
                               self.d_skip, xz, self.inner, row_offsets=ctx.row_offsets, state_slots=ctx.state_slots,
                               state=slot.states["S"], out_dtype=self.act_dtype)
        return self.out(y)


@register_part("mixer", "state_space_duality")
class StateSpaceDualityMixer(Mixer):
    graph_safe = True
    cache_spec = None

    def __init__(self, *, in_proj: Linear, conv_weight: torch.Tensor, conv_bias: Optional[torch.Tensor],
                 dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor, norm_weight: torch.Tensor,
                 out: Linear, heads: int, value_dim: int, states: int, groups: int, taps: int, norm_groups: int,
                 eps: float, act_dtype: torch.dtype = torch.bfloat16):
        """``in_proj``: rows ``[x | B | C | z | dt]`` (see :func:`ssd_projection_order` for the order a file that
        stores ``[z | x | B | C | dt]`` is brought into)."""
        inner, bc = heads * value_dim, groups * states
        if heads % groups:
            raise ValueError(f"heads ({heads}) must be a multiple of groups ({groups})")
        if in_proj.out_features != 2 * inner + 2 * bc + heads or out.in_features != inner:
            raise ValueError(f"the projections disagree with the inner size {inner}, {groups} groups of {states} states "
                             f"and {heads} heads")
        if conv_weight.numel() != (inner + 2 * bc) * taps or taps < 1:
            raise ValueError("the convolution weight disagrees with the channels or the taps")
        if states > ops.SSD_MAX_STATES or inner % norm_groups or norm_weight.numel() != inner:
            raise ValueError(f"{states} states (at most {ops.SSD_MAX_STATES}) or {norm_groups} norm groups over {inner} "
                             f"are not supported")
        if min(dt_bias.numel(), a_log.numel(), d_skip.numel()) != heads:
            raise ValueError("dt_bias, A_log and D hold one number a head")
        self.in_proj, self.out = in_proj, out
        self.conv_weight, self.conv_bias = conv_weight, conv_bias
        self.dt_bias, self.a_log, self.d_skip, self.norm_weight = dt_bias, a_log, d_skip, norm_weight
        self.heads, self.value_dim, self.states, self.groups = heads, value_dim, states, groups
        self.taps, self.norm_groups, self.eps, self.act_dtype = taps, norm_groups, float(eps), act_dtype
        self.inner, self.channels = inner, inner + 2 * bc
        self.state_specs = {"S": StateSpec((heads * states * value_dim,), torch.float32),
                            "conv": StateSpec((max(taps - 1, 1) * self.channels,), torch.float32)}

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        proj = self.in_proj(h)                                                   # [T, channels + inner + heads] float32
        xbc, _ = ops.causal_conv(proj, self.channels, self.conv_weight, self.conv_bias, slot.states["conv"],
                                 row_request=ctx.row_request, row_offsets=ctx.row_offsets,
                                 state_slots=ctx.state_slots, act_dtype=torch.float32)
        y = ops.ssd_scan(xbc, proj, col_x=0, col_b=self.inner, col_c=self.inner + self.groups * self.states,
                         col_dt=self.channels + self.inner, dt_bias=self.dt_bias, a_log=self.a_log, dskip=self.d_skip,
                         row_offsets=ctx.row_offsets, state_slots=ctx.state_slots, state=slot.states["S"],
                         heads=self.heads, groups=self.groups, states=self.states, vdim=self.value_dim)
        u = ops.gated_group_norm(y, proj, self.channels, self.norm_weight, self.eps, self.norm_groups, self.act_dtype)
        return self.out(u)


def ssd_projection_order(heads: int, value_dim: int, states: int, groups: int) -> torch.Tensor:
    """Row indices that bring an input projection stored as ``[z | x | B | C | dt]`` into the order
    ``[x | B | C | z | dt]`` that :class:`StateSpaceDualityMixer` reads (the convolved channels first)."""
    inner, bc = heads * value_dim, groups * states
    z = torch.arange(0, inner)
    xbc = torch.arange(inner, 2 * inner + 2 * bc)
    dt = torch.arange(2 * inner + 2 * bc, 2 * inner + 2 * bc + heads)
    return torch.cat([xbc, z, dt])


@register_part("mixer", "branch_pair")
class BranchPair(Mixer):
    def __init__(self, *, left: Mixer, right: Mixer, left_weight: torch.Tensor, right_weight: torch.Tensor, eps: float,
                 scale: float = 0.5):
        if left.cache_spec is not None and right.cache_spec is not None:
            raise ValueError("only one branch of a pair may keep keys and values")
        self.left, self.right, self.left_weight, self.right_weight = left, right, left_weight, right_weight
        self.eps, self.scale = float(eps), float(scale)
        self.cache_spec = left.cache_spec if left.cache_spec is not None else right.cache_spec
        self.state_spec = None
        self.state_specs = {}
        for prefix, m in (("left.", left), ("right.", right)):
            if m.state_spec is not None:
                self.state_specs[prefix + "state"] = m.state_spec
            for name, spec in (m.state_specs or {}).items():
                self.state_specs[prefix + name] = spec
        self.graph_safe = bool(getattr(left, "graph_safe", False) and getattr(right, "graph_safe", False))
        self.wants_fp32_input = False

    def step_planner(self, page_size: int):
        return self.left.step_planner(page_size) or self.right.step_planner(page_size)

    @staticmethod
    def _branch_slot(slot: LayerSlot, prefix: str, mixer: Mixer) -> LayerSlot:
        states = {name[len(prefix):]: t for name, t in slot.states.items() if name.startswith(prefix)}
        return replace(slot, states=states, state=states.get("state") if mixer.state_spec is not None else None)

    def forward(self, ctx: StepContext, slot: LayerSlot, h: torch.Tensor) -> torch.Tensor:
        a = self.left.forward(ctx, self._branch_slot(slot, "left.", self.left), h)
        b = self.right.forward(ctx, self._branch_slot(slot, "right.", self.right), h)
        return ops.norm_mean2(a, self.left_weight, b, self.right_weight, self.eps, self.scale)
