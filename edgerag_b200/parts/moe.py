"""A feed-forward of routed experts: every token is sent to the ``top`` experts its router scores highest, and
optionally through a shared expert that every token uses.

    z = W_router x (float32),   s = sigmoid(z),   chosen = the ``top`` largest s (the lower index wins a tie)
    y = sum over chosen e of expert_e(w_e x) + shared(x),      expert(r) = W_down (silu(W_gate r) * (W_up r))

``weights`` says what ``w_e`` is: ``"score"`` (the score itself; ``"score_normed"``, the chosen scores divided by their
sum, is not built).  With ``scale_input`` the weight multiplies the expert's input (rounded once to the element type),
otherwise its output: ``y = sum_e w_e expert_e(x)``, the weight applied in float to the down product's sums.  Experts
have no biases.  The experts' tensors are ``e<i>.{gate, up, down}`` below the part's prefix, the router ``router``, the
shared expert a feed-forward part of its own under ``shared.``.

Further options: ``scores = "softmax"`` (the scores are the softmax of the logits over all experts; the choice still
goes by the largest); ``groups = (count, keep)``: the experts form ``count`` equal groups of neighbours, a group's score
is its best expert's, and only experts of the ``keep`` best groups can be chosen; ``gated = False`` with ``act =
"relu_squared"``: experts without a gate branch, ``W_down relu(W_up r)^2`` (tensors ``e<i>.{up, down}``).

Nothing here goes through the host: the router's kernel leaves, on the device, every expert's list of (token, choice)
pairs, and the two product kernels walk row tiles of those lists, so the launches of a step depend on its number of
tokens only and the step can be replayed from a CUDA graph.  The update leaves as float32 partial sums, one per choice
plus one for the shared expert, which whoever adds the update sums in that order.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import FeedForward, PartSpec, WeightSpec, build_part, register_part


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, n_experts: int, top: int, dtype: torch.dtype, device: torch.device,
                 shared: PartSpec | None = None, weights: str = "score", scale_input: bool = True,
                 names: tuple[str, str, str] = ("gate", "up", "down"), router: str = "router", expert: str = "e{}.",
                 scores: str = "sigmoid", groups: tuple[int, int] | None = None, gated: bool = True,
                 act: str = "silu") -> None:
        if not 0 < top <= n_experts:
            raise ValueError(f"routed_experts: top {top} of {n_experts} experts")
        if weights != "score":
            raise ValueError("routed_experts: only the scores themselves are built as weights")
        if scores not in kernels.MOE_SCORES:
            raise ValueError(f"routed_experts: scores {scores!r}; known: {sorted(kernels.MOE_SCORES)}")
        if (gated and act != "silu") or (not gated and act != "relu_squared"):
            raise ValueError("routed_experts: gated experts use silu, experts without a gate branch relu_squared")
        if groups is not None:
            count, keep = (int(v) for v in groups)
            if count < 1 or n_experts % count or not 1 <= keep <= count or top > keep * (n_experts // count):
                raise ValueError(f"routed_experts: {count} groups of which {keep} are kept cannot give {top} of {n_experts} experts")
            groups = (count, keep)
        self.scores, self.groups, self.gated, self.scale_input = scores, groups, bool(gated), bool(scale_input)
        self.hidden, self.intermediate, self.n_experts, self.top = hidden, intermediate, n_experts, top
        self.dtype, self.device = dtype, device
        self.names, self.router_name, self.expert_fmt = tuple(names), router, expert
        self._shared_prefix = shared.prefix if shared is not None else ""
        self.shared = build_part("ffn", shared, dtype, device) if shared is not None else None
        self.graph_safe = self.shared is None or bool(getattr(self.shared, "graph_safe", False))
        self.w_router = self.w_gate_up = self.w_down = None

    def weight_specs(self) -> list[WeightSpec]:
        gate, up, down = self.names
        specs = [WeightSpec(self.router_name, (self.n_experts, self.hidden), "vector32")]
        for e in range(self.n_experts):
            pre = self.expert_fmt.format(e)
            if self.gated:
                specs.append(WeightSpec(pre + gate, (self.intermediate, self.hidden)))
            specs += [WeightSpec(pre + up, (self.intermediate, self.hidden)), WeightSpec(pre + down, (self.hidden, self.intermediate))]
        if self.shared is not None:
            specs += [WeightSpec(self._shared_prefix + s.name, s.shape, s.kind, s.fallback) for s in self.shared.weight_specs()]
        return specs

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        gate, up, down = self.names
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)  # noqa: E731
        self.w_router = tensors[self.router_name].to(device=self.device, dtype=torch.float32).contiguous()
        pres = [self.expert_fmt.format(e) for e in range(self.n_experts)]
        if self.gated:
            self.w_gate_up = torch.stack([torch.cat([cast(tensors[p + gate]), cast(tensors[p + up])], 0) for p in pres]).contiguous()
        else:       # (the one matrix of an expert without a gate branch, under the same attribute)
            self.w_gate_up = torch.stack([cast(tensors[p + up]) for p in pres]).contiguous()
        self.w_down = torch.stack([cast(tensors[p + down]) for p in pres]).contiguous()
        if self.shared is not None:
            self.shared.load_weights({s.name: tensors[self._shared_prefix + s.name] for s in self.shared.weight_specs()})

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n, top = x.shape[0], self.top
        lists = ctx.buf("moe.lists", (kernels.moe_lists_ints(n, self.n_experts, top),), torch.int32)
        score = ctx.buf("moe.score", (n * top,), torch.float32)
        act = ctx.buf("moe.act", (n * top, self.intermediate), self.dtype)
        parts = ctx.buf("ffn.out_parts", (top + (self.shared is not None), n, self.hidden), torch.float32)
        in_score, out_score = (score, None) if self.scale_input else (None, score)
        if kernels.moe_tc_supported(self.dtype, self.hidden, self.intermediate):
            # tensor cores: row tiles sized by the step's tokens, the (scaled) rows gathered once in list order
            tile_rows = kernels.moe_tc_tile_rows(n, self.n_experts, top)
            kernels.moe_route(x, self.w_router, top, lists, score, tile_rows, scores=self.scores, groups=self.groups)
            xs = ctx.buf("moe.rows", (n * top, self.hidden), self.dtype)
            kernels.moe_tc_gather(x, lists, in_score, self.n_experts, top, xs)
            if self.gated:
                kernels.moe_tc_gate_up(xs, self.w_gate_up, lists, top, tile_rows, act)
            else:
                kernels.moe_tc_up_act(xs, self.w_gate_up, lists, top, tile_rows, act)
            kernels.moe_tc_down(act, self.w_down, lists, top, tile_rows, parts, out_score=out_score)
        else:
            kernels.moe_route(x, self.w_router, top, lists, score, scores=self.scores, groups=self.groups)
            if self.gated:
                if in_score is None:
                    raise ValueError("routed_experts: gated experts on the general kernels take their weight on the input")
                kernels.moe_gate_up(x, self.w_gate_up, lists, score, top, act)
            else:
                if in_score is not None:
                    raise ValueError("routed_experts: experts without a gate branch take their weight on the output")
                kernels.moe_up_act(x, self.w_gate_up, lists, top, act)
            kernels.moe_down(act, self.w_down, lists, top, parts, out_score=out_score)
        if self.shared is not None:
            self.shared.forward_into(x, ctx, parts[top])
        return parts
