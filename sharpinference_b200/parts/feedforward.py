"""Feed-forward parts: dense SwiGLU, a top-1 sigmoid-routed mixture of experts with an
always-on shared expert, a dense two-layer network with a plain activation (``DenseMLP``) and a
sigmoid-routed mixture in which every row uses k such networks (``MoESigmoidTopK``).

Dense (src/SharpInference.Engine/ForwardPass.cs:2006-2015): ``y = (silu(h Wg^T) * (h Wu^T)) Wd^T``.

Mixture (src/SharpInference.Engine/ForwardPass.cs:2021-2098): router logits ``r = h Wr^T``,
``p = sigmoid(r)``, the expert with the largest ``p`` (first wins), ``w = p[e]``; the routed
expert computes ``(silu(w g) * (w u)) Wd[e]^T`` with ``g = h Wg[e]^T``, ``u = h Wu[e]^T`` (the
weight scales gate and up, which is scaling the expert's input); the shared expert is a dense
SwiGLU on the unscaled ``h``; the two are summed.  Routing stays on the device: the step's rows
are sorted by expert and each expert multiplies its rows in one grouped product.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import FeedForward, StepContext, register_part
from .linear import GroupedLinear, Linear


@register_part("feed_forward", "dense_swiglu")
class DenseSwiGLU(FeedForward):
    graph_safe = True        # reads the step through device tensors only: may be captured in a CUDA graph
    def __init__(self, *, gate_up: Linear, down: Linear, act_dtype: torch.dtype = torch.bfloat16,
                 activation: str = "silu"):
        """``activation``: what is applied to the gate half, ``silu`` (SwiGLU), ``gelu_tanh`` or ``relu2``."""
        if gate_up.out_features != 2 * down.in_features:
            raise ValueError(f"fused gate|up weight has {gate_up.out_features} rows, expected 2 * {down.in_features}")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not one of {', '.join(sorted(ops.ACTIVATIONS))}")
        self.gate_up, self.down, self.act_dtype, self.activation = gate_up, down, act_dtype, activation

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        if self.activation != "silu":
            act = ops.gated_act(self.gate_up(h), ops.ACTIVATIONS[self.activation], self.act_dtype)
        elif self.act_dtype == torch.bfloat16 and self.gate_up.streams(h) and self.gate_up.bias is None:
            act = ops.dense_rows(h, self.gate_up.weight, swiglu=True)     # SwiGLU in the product's epilogue
        else:
            act = ops.swiglu(self.gate_up(h), self.act_dtype)
        return self.down(act, out=out, accumulate=accumulate)


_side_streams: dict = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """The second stream of a device, on which the shared expert runs beside the routed ones."""
    key = torch.device(device).index
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


def _urgent_stream(device: torch.device) -> "torch.cuda.Stream":
    """A stream of higher priority for short kernels that a longer chain waits for."""
    key = ("urgent", torch.device(device).index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device, priority=-1)
    return _side_streams[key]


@register_part("feed_forward", "moe_sigmoid_top1")
class MoESigmoidTop1(FeedForward):
    wants_fp32_input = True
    graph_safe = True
    # Steps of more rows than this keep the routed gate|up product on the routing's stream (see forward).
    SMALL_STEP_ROWS = 256
    # Up to this many rows the shared expert's down product adds into the output on the grouped tensor-core
    # kernel (one group, K cut over CTAs) instead of the library's product and an addition: alone the library is
    # a little faster on that shape, but beside the routed gate|up product the step is not (Scout sizes, 8
    # layers: batch 1 614 -> 644 tok/s; no difference from batch 8 on).  Both experts then add into a zeroed
    # output with reductions and no longer wait for each other.
    SHARED_DOWN_SPLIT_ADD_ROWS = 4

    def __init__(self, *, router: torch.Tensor, experts_gate_up: GroupedLinear, experts_down: GroupedLinear,
                 shared: Optional[DenseSwiGLU], act_dtype: torch.dtype = torch.bfloat16):
        E = experts_gate_up.num_groups
        if router.shape != (E, experts_gate_up.in_features):
            raise ValueError(f"router weight is {tuple(router.shape)}, expected [{E}, {experts_gate_up.in_features}]")
        if experts_down.num_groups != E or experts_gate_up.out_features != 2 * experts_down.in_features:
            raise ValueError("expert gate|up and down weights disagree on the number or width of the experts")
        self.router = router
        self.experts_gate_up, self.experts_down = experts_gate_up, experts_down
        self.shared = shared
        shared_down = getattr(shared, "down", None)
        if isinstance(shared_down, Linear) and shared_down.split_add_rows == 0:
            shared_down.split_add_rows = self.SHARED_DOWN_SPLIT_ADD_ROWS
        self.num_experts = E
        self.act_dtype = act_dtype
        # the tensor-core path takes bfloat16 weights whose inner sizes are multiples of 8 (TMA rows
        # must start on 16 bytes); everything else runs the CUDA-core kernels
        self._tensor_core = (experts_gate_up.weight.dtype == torch.bfloat16
                             and experts_down.weight.dtype == torch.bfloat16 and act_dtype == torch.bfloat16
                             and experts_gate_up.in_features % 8 == 0 and experts_down.in_features % 8 == 0)

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None) -> torch.Tensor:
        T = h.shape[0]
        if h32 is None:
            h32 = h.to(torch.float32)
        # The shared expert and the routed ones meet only where the routed outputs are added, so the shared
        # expert runs on a second stream (inside a graph capture: a fork and a join), forked off before the
        # routing, and the streams join before the routed down product.  Routing, sorting and gathering are
        # short kernels that everything routed waits for, and behind the shared product's many blocks they
        # would queue, so they run on a third stream of higher priority.  Small steps: the routed gate|up
        # product returns to the main stream and streams its weights beside the shared expert's (two streams
        # of weights keep the memory system busier than one; with priority over the shared expert it measured
        # slower).  Large steps: every product fills the GPU by itself; the routed gate|up product stays on the
        # third stream and takes over the SMs as the shared expert's products drain.
        # When the shared expert's down product adds with reductions too (few rows, see SHARED_DOWN_SPLIT_ADD_ROWS),
        # both experts add into a zeroed output and the streams need not meet before the end: each element is
        # 0 + a + b in one order or the other, which is the same number.
        tensor_core = self._tensor_core and h.dtype == torch.bfloat16
        main = torch.cuda.current_stream(h.device)
        side = routed = None
        apart = False
        if self.shared is not None:
            shared_down = getattr(self.shared, "down", None)
            apart = tensor_core and isinstance(shared_down, Linear) and shared_down.adds_with_reductions(h)
            make = torch.zeros if apart else torch.empty
            y = make((T, self.experts_down.out_features), dtype=torch.float32, device=h.device)
            side, routed = _side_stream(h.device), _urgent_stream(h.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                if apart:
                    self.shared.forward(ctx, h, out=y, accumulate=True)
                else:
                    self.shared.forward(ctx, h, out=y)
            routed.wait_stream(main)
        else:
            y = torch.zeros((T, self.experts_down.out_features), dtype=torch.float32, device=h.device)
        act = None
        with torch.cuda.stream(routed if routed is not None else main):
            expert, weight, _, offsets, sorted_rows = ops.router_top1(h32, self.router, sort=True)
            # one row is its own sorted order: nothing to gather
            h_sorted = (h if T == 1 else ops.gather_rows_bf16(h, sorted_rows)) if tensor_core else None
            if tensor_core and T > self.SMALL_STEP_ROWS:
                act = ops.tc_grouped_gemm(h_sorted, self.experts_gate_up.weight, offsets, mode=ops.TC_MODE_SWIGLU,
                                          row_scale=weight, scale_rows=sorted_rows)
        if routed is not None:
            main.wait_stream(routed)
        if "router_choices" in ctx.extras:          # tracing: which expert every row went to
            ctx.extras["router_choices"].append(expert)
        if tensor_core:
            if act is None:
                act = ops.tc_grouped_gemm(h_sorted, self.experts_gate_up.weight, offsets, mode=ops.TC_MODE_SWIGLU,
                                          row_scale=weight, scale_rows=sorted_rows)
            if side is not None and not apart:
                main.wait_stream(side)
            ops.tc_grouped_gemm(act, self.experts_down.weight, offsets, mode=ops.TC_MODE_STORE, out=y,
                                out_rows=sorted_rows, accumulate=True)
            if apart:
                main.wait_stream(side)
            return y
        gu = self.experts_gate_up(h, offsets, rows=T, a_rows=sorted_rows)          # sorted order
        act = ops.swiglu(gu, self.act_dtype, row_scale=weight, scale_rows=sorted_rows)
        if side is not None:
            main.wait_stream(side)
        self.experts_down(act, offsets, rows=T, out_rows=sorted_rows, out=y, accumulate=True)
        return y


@register_part("feed_forward", "dense_mlp")
class DenseMLP(FeedForward):
    """``W_down act(W_up h + b_up) + b_down`` with ``act`` one of ``ops.ACTIVATIONS`` (the square of relu,
    tanh-GELU, SiLU); the biases are optional.  The bias of the first product and the activation are one kernel
    over the product's float32 result."""

    graph_safe = True
    adds_to = True

    def __init__(self, *, up: Linear, down: Linear, activation: str = "relu2", act_dtype: torch.dtype = torch.bfloat16):
        if up.out_features != down.in_features:
            raise ValueError(f"up projection has {up.out_features} rows, down projection reads {down.in_features}")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not one of {', '.join(sorted(ops.ACTIVATIONS))}")
        # the first product leaves its bias to the activation kernel
        self.up = Linear(up.weight, up.name, stream_rows=up.stream_rows)
        self.up_bias = up.bias
        self.down, self.activation, self.act_dtype = down, activation, act_dtype

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None,
                add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
        act = ops.bias_act(self.up(h), self.up_bias, ops.ACTIVATIONS[self.activation], self.act_dtype)
        y = self.down(act)
        return y if add_to is None else ops.add(add_to, y, out=add_to)


@register_part("feed_forward", "moe_sigmoid_topk")
class MoESigmoidTopK(FeedForward):
    """A mixture of ``E`` two-layer experts (``W_down act(W_up h)``, no biases) of which every row uses ``top_k``.

    Router: ``s = sigmoid(Wr h)`` in float32 on the unrounded activations; the ``top_k`` experts with the largest
    ``s + correction`` are chosen (``correction`` may be None; the lowest index wins among equals); an expert's
    output is weighted by ``route_scale * s`` (without the correction), the chosen ``s`` divided by their sum
    first when ``renormalize``.  The (row, choice) pairs are sorted by expert on the device; each expert multiplies
    its rows in one grouped product (tcgen05 for bfloat16 weights whose inner sizes are multiples of 8, with the
    activation in the first product's epilogue; CUDA cores otherwise), the second product scales each pair's row by its weight, and the pairs of a row are added in the
    order of the choices, so a row's result does not depend on the rest of the step.

    The reference's mixture (src/SharpInference.Engine/ForwardPass.cs:2021-2098) is top-1 with a shared expert.
    """

    wants_fp32_input = True
    graph_safe = True
    adds_to = True

    def __init__(self, *, router: torch.Tensor, experts_up: GroupedLinear, experts_down: GroupedLinear, top_k: int,
                 correction: Optional[torch.Tensor] = None, route_scale: float = 1.0, renormalize: bool = False,
                 activation: str = "relu2", act_dtype: torch.dtype = torch.bfloat16):
        E = experts_up.num_groups
        if router.shape != (E, experts_up.in_features):
            raise ValueError(f"router weight is {tuple(router.shape)}, expected [{E}, {experts_up.in_features}]")
        if experts_down.num_groups != E or experts_up.out_features != experts_down.in_features:
            raise ValueError("expert up and down weights disagree on the number or width of the experts")
        if not (1 <= top_k <= min(E, 32)):
            raise ValueError(f"experts per row must be 1 .. min(experts, 32), found {top_k} of {E}")
        if correction is not None and correction.numel() != E:
            raise ValueError(f"router correction has {correction.numel()} entries for {E} experts")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not one of {', '.join(sorted(ops.ACTIVATIONS))}")
        self.router, self.correction = router, correction
        self.experts_up, self.experts_down = experts_up, experts_down
        self.num_experts, self.top_k = E, int(top_k)
        self.route_scale, self.renormalize = float(route_scale), bool(renormalize)
        self.activation, self.act_dtype = activation, act_dtype
        self._tensor_core = (experts_up.weight.dtype == torch.bfloat16 and experts_down.weight.dtype == torch.bfloat16
                             and act_dtype == torch.bfloat16 and experts_up.in_features % 8 == 0
                             and experts_down.in_features % 8 == 0)

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None,
                add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, k = h.shape[0], self.top_k
        if h32 is None:
            h32 = h.to(torch.float32)
        expert, weight, _ = ops.router_topk(h32, self.router, k, correction=self.correction, scale=self.route_scale,
                                            renormalize=self.renormalize)
        if "router_choices" in ctx.extras:          # tracing: which experts every row went to
            ctx.extras["router_choices"].append(expert)
        offsets, sorted_pairs = ops.moe_sort(expert.view(-1), self.num_experts)     # pair = row * k + choice
        pair_rows = ops.moe_pair_tokens(sorted_pairs, k) if k > 1 else sorted_pairs
        act_code = ops.ACTIVATIONS[self.activation]
        y = torch.empty((T * k, self.experts_down.out_features), dtype=torch.float32, device=h.device)
        if self._tensor_core and h.dtype == torch.bfloat16:
            h_sorted = ops.gather_rows_bf16(h, pair_rows)
            act = ops.tc_grouped_gemm_act(h_sorted, self.experts_up.weight, offsets, act_code)   # activation in the epilogue
            ops.tc_grouped_gemm(act, self.experts_down.weight, offsets, mode=ops.TC_MODE_STORE, out=y,
                                out_rows=sorted_pairs, row_scale=weight.view(-1), scale_rows=sorted_pairs)
        else:
            up = self.experts_up(h, offsets, rows=T * k, a_rows=pair_rows)             # sorted order
            act = ops.bias_act(up, None, act_code, self.act_dtype)
            ops.gemm_nt(act, self.experts_down.weight, out=y, group_offsets=offsets, out_rows=sorted_pairs, rows=T * k,
                        row_scale=weight.view(-1), scale_rows=sorted_pairs)
        return ops.moe_combine(y, k, add=add_to, out=add_to)


@register_part("feed_forward", "moe_sigmoid_topk_gated")
class MoESigmoidTopKGated(FeedForward):
    """A mixture of ``E`` gated experts (``W_down (silu(W_gate u) * (W_up u))``, no biases) of which every row uses
    ``top_k``, with an optional shared expert of the same form that every row uses.

    Router: ``s = sigmoid(Wr h)`` in float32 on the unrounded activations; the ``top_k`` experts with the largest
    ``s`` are chosen (the lowest index wins among equals); the chosen scores are the weights as they are (divided by
    their sum first when ``renormalize``).  A weight multiplies its expert's *input*: the routed output is
    ``sum_e expert_e(s_e h)``.  Because gate and up are linear in their input, the weight is applied to both products
    in the first grouped product's epilogue, before the nonlinearity.  The (row, choice) pairs are sorted by expert on
    the device, each expert multiplies its rows in one grouped product (tcgen05 for bfloat16 weights whose inner
    sizes are multiples of 8, CUDA cores otherwise), and the pairs of a row are added in the order of the choices
    together with the shared expert's output, so a row's result does not depend on the rest of the step.

    With one expert a row this is the arithmetic of :class:`MoESigmoidTop1`, which fuses more and is what a builder
    should pick then; this part takes any ``top_k``.

    Other routers of the same mixture, by argument: ``router_bias`` ``[E]`` is added to the logits;
    ``scoring="softmax_chosen"`` picks the ``top_k`` largest logits and weights them by the softmax over the chosen
    logits alone; ``weights_on="output"`` multiplies an expert's *output* by its weight (in the second grouped
    product's epilogue) instead of its input.
    """

    wants_fp32_input = True
    graph_safe = True
    adds_to = True

    def __init__(self, *, router: torch.Tensor, experts_gate_up: GroupedLinear, experts_down: GroupedLinear, top_k: int,
                 shared: Optional[DenseSwiGLU] = None, renormalize: bool = False,
                 act_dtype: torch.dtype = torch.bfloat16, router_bias: Optional[torch.Tensor] = None,
                 scoring: str = "sigmoid", weights_on: str = "input"):
        E = experts_gate_up.num_groups
        if scoring not in ops.ROUTER_SCORING:
            raise ValueError(f"router scoring '{scoring}' is not one of {', '.join(ops.ROUTER_SCORING)}")
        if weights_on not in ("input", "output"):
            raise ValueError(f"weights_on '{weights_on}' is not one of input, output")
        if router_bias is not None and router_bias.numel() != E:
            raise ValueError(f"router bias has {router_bias.numel()} entries for {E} experts")
        self.router_bias, self.scoring, self.weights_on = router_bias, scoring, weights_on
        if router.shape != (E, experts_gate_up.in_features):
            raise ValueError(f"router weight is {tuple(router.shape)}, expected [{E}, {experts_gate_up.in_features}]")
        if experts_down.num_groups != E or experts_gate_up.out_features != 2 * experts_down.in_features:
            raise ValueError("expert gate|up and down weights disagree on the number or width of the experts")
        if not (1 <= top_k <= min(E, 32)):
            raise ValueError(f"experts per row must be 1 .. min(experts, 32), found {top_k} of {E}")
        self.router = router
        self.experts_gate_up, self.experts_down, self.shared = experts_gate_up, experts_down, shared
        self.num_experts, self.top_k, self.renormalize, self.act_dtype = E, int(top_k), bool(renormalize), act_dtype
        self._tensor_core = (experts_gate_up.weight.dtype == torch.bfloat16
                             and experts_down.weight.dtype == torch.bfloat16 and act_dtype == torch.bfloat16
                             and experts_gate_up.in_features % 8 == 0 and experts_down.in_features % 8 == 0)

    def forward(self, ctx: StepContext, h: torch.Tensor, h32: Optional[torch.Tensor] = None,
                add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, k = h.shape[0], self.top_k
        if h32 is None:
            h32 = h.to(torch.float32)
        # the shared expert meets the routed ones only in the last sum: it runs on a second stream meanwhile
        main = torch.cuda.current_stream(h.device)
        base = add_to
        side = None
        if self.shared is not None:
            side = _side_stream(h.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                if base is not None:
                    self.shared.forward(ctx, h, out=base, accumulate=True)
                else:
                    base = self.shared.forward(ctx, h)
        expert, weight, _ = ops.router_topk(h32, self.router, k, renormalize=self.renormalize, bias=self.router_bias,
                                            scoring=self.scoring)
        if "router_choices" in ctx.extras:          # tracing: which experts every row went to
            ctx.extras["router_choices"].append(expert)
        offsets, sorted_pairs = ops.moe_sort(expert.view(-1), self.num_experts)     # pair = row * k + choice
        pair_rows = ops.moe_pair_tokens(sorted_pairs, k) if k > 1 else sorted_pairs
        y = torch.empty((T * k, self.experts_down.out_features), dtype=torch.float32, device=h.device)
        # the weight scales gate and up before the nonlinearity (the expert's input), or the second product's rows
        w_in = weight.view(-1) if self.weights_on == "input" else None
        w_out = weight.view(-1) if self.weights_on == "output" else None
        if self._tensor_core and h.dtype == torch.bfloat16:
            h_sorted = ops.gather_rows_bf16(h, pair_rows)
            act = ops.tc_grouped_gemm(h_sorted, self.experts_gate_up.weight, offsets, mode=ops.TC_MODE_SWIGLU,
                                      row_scale=w_in, scale_rows=sorted_pairs if w_in is not None else None)
            ops.tc_grouped_gemm(act, self.experts_down.weight, offsets, mode=ops.TC_MODE_STORE, out=y,
                                out_rows=sorted_pairs, row_scale=w_out,
                                scale_rows=sorted_pairs if w_out is not None else None)
        else:
            gu = self.experts_gate_up(h, offsets, rows=T * k, a_rows=pair_rows)        # sorted order
            act = ops.swiglu(gu, self.act_dtype, row_scale=w_in, scale_rows=sorted_pairs if w_in is not None else None)
            w_down = self.experts_down.weight
            if w_down.dtype == torch.float32 and act.dtype != torch.float32:
                act = act.to(torch.float32)
            ops.gemm_nt(act, w_down, out=y, group_offsets=offsets, out_rows=sorted_pairs, rows=T * k,
                        row_scale=w_out, scale_rows=sorted_pairs if w_out is not None else None)
        if side is not None:
            main.wait_stream(side)
        return ops.moe_combine(y, k, add=base, out=base)
