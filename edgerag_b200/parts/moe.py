"""A feed-forward of routed experts: every token is sent to the ``top`` experts its router scores highest, and
optionally through a shared expert that every token uses.

    z = W_router x (float32),   s = sigmoid(z),   chosen = the ``top`` largest s (the lower index wins a tie)
    y = sum over chosen e of expert_e(w_e x) + shared(x),      expert(r) = W_down (silu(W_gate r) * (W_up r))

``weights`` says what ``w_e`` is: ``"score"`` (the sigmoid score itself) or ``"score_normed"`` (the chosen scores
divided by their sum).  The weight multiplies the expert's input, as this part's ``scale_input`` says (the only
form built; a weight on the output would be another kernel epilogue).  Experts have no biases.  The experts' tensors
are ``e<i>.{gate, up, down}`` below the part's prefix, the router ``router``, the shared expert a feed-forward part of
its own under ``shared.``.

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
                 names: tuple[str, str, str] = ("gate", "up", "down"), router: str = "router", expert: str = "e{}.") -> None:
        if not 0 < top <= n_experts:
            raise ValueError(f"routed_experts: top {top} of {n_experts} experts")
        if weights != "score" or not scale_input:
            raise ValueError("routed_experts: only sigmoid scores that multiply the expert's input are built")
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
            specs += [WeightSpec(pre + gate, (self.intermediate, self.hidden)), WeightSpec(pre + up, (self.intermediate, self.hidden)),
                      WeightSpec(pre + down, (self.hidden, self.intermediate))]
        if self.shared is not None:
            specs += [WeightSpec(self._shared_prefix + s.name, s.shape, s.kind, s.fallback) for s in self.shared.weight_specs()]
        return specs

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        gate, up, down = self.names
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)  # noqa: E731
        self.w_router = tensors[self.router_name].to(device=self.device, dtype=torch.float32).contiguous()
        pres = [self.expert_fmt.format(e) for e in range(self.n_experts)]
        self.w_gate_up = torch.stack([torch.cat([cast(tensors[p + gate]), cast(tensors[p + up])], 0) for p in pres]).contiguous()
        self.w_down = torch.stack([cast(tensors[p + down]) for p in pres]).contiguous()
        if self.shared is not None:
            self.shared.load_weights({s.name: tensors[self._shared_prefix + s.name] for s in self.shared.weight_specs()})

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n, top = x.shape[0], self.top
        lists = ctx.buf("moe.lists", (kernels.moe_lists_ints(n, self.n_experts, top),), torch.int32)
        score = ctx.buf("moe.score", (n * top,), torch.float32)
        act = ctx.buf("moe.act", (n * top, self.intermediate), self.dtype)
        parts = ctx.buf("ffn.out_parts", (top + (self.shared is not None), n, self.hidden), torch.float32)
        if kernels.moe_tc_supported(self.dtype, self.hidden, self.intermediate):
            # tensor cores: row tiles sized by the step's tokens, the scaled rows gathered once in list order
            tile_rows = kernels.moe_tc_tile_rows(n, self.n_experts, top)
            kernels.moe_route(x, self.w_router, top, lists, score, tile_rows)
            xs = ctx.buf("moe.rows", (n * top, self.hidden), self.dtype)
            kernels.moe_tc_gather(x, lists, score, self.n_experts, top, xs)
            kernels.moe_tc_gate_up(xs, self.w_gate_up, lists, top, tile_rows, act)
            kernels.moe_tc_down(act, self.w_down, lists, top, tile_rows, parts)
        else:
            kernels.moe_route(x, self.w_router, top, lists, score)
            kernels.moe_gate_up(x, self.w_gate_up, lists, score, top, act)
            kernels.moe_down(act, self.w_down, lists, top, parts)
        if self.shared is not None:
            self.shared.forward_into(x, ctx, parts[top])
        return parts
