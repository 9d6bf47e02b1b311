"""A feed-forward without a gate branch: ``down(act(up(x)))``, no biases.

``act`` is ``gelu_erf`` (the exact gelu, ``0.5 z (1 + erf(z / sqrt 2))``) or ``relu_squared``; the activation kernel
works in float and rounds once.  With ``scalar_gate`` (the name of a ``[1, hidden]`` tensor) the whole branch is
multiplied by ``sigmoid(w_gate . x)``, one number per token: the gate's row is stored below the up matrix, so that one
product makes the logit beside the up rows, and the activation kernel multiplies its output by the sigmoid (a constant
per row commutes with the down product).  This is the form of a shared expert that a router's layer adds for every token.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import FeedForward, WeightSpec, register_part


@register_part("ffn", "dense_act")
class DenseAct(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, dtype: torch.dtype, device: torch.device, act: str = "gelu_erf",
                 names: tuple[str, str] = ("up", "down"), scalar_gate: str | None = None) -> None:
        if act not in kernels.ACTS:
            raise ValueError(f"unknown activation {act!r}; known: {sorted(kernels.ACTS)}")
        self.hidden, self.intermediate, self.act = hidden, intermediate, act
        self.dtype, self.device = dtype, device
        self.names, self.scalar_gate = tuple(names), scalar_gate
        #: columns of the first product: the up rows, then (with a gate) the gate's row, padded to 16 bytes
        self.up_width = intermediate if scalar_gate is None else -(-(intermediate + 1) // 8) * 8
        self.w_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        up, down = self.names
        specs = [WeightSpec(up, (self.intermediate, self.hidden)), WeightSpec(down, (self.hidden, self.intermediate))]
        if self.scalar_gate is not None:
            specs.append(WeightSpec(self.scalar_gate, (1, self.hidden)))
        return specs

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        up, down = self.names
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)  # noqa: E731
        rows = [cast(tensors[up])]
        if self.scalar_gate is not None:
            rows.append(cast(tensors[self.scalar_gate]).reshape(1, self.hidden))
            rows.append(torch.zeros((self.up_width - self.intermediate - 1, self.hidden), dtype=self.dtype, device=self.device))
        self.w_up = torch.cat(rows, 0).contiguous()
        self.w_down = cast(tensors[down]).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = x.shape[0]
        n_parts = 0 if self.scalar_gate is not None else self._parts(x, ctx)
        if n_parts:      # the rows of a larger decode step: k split over the SMs, the norm after adds the parts
            y = ctx.buf("ffn.out_parts", (n_parts, n, self.hidden), torch.float32)
            kernels.linear_parts(self._act(x, ctx), self.w_down, y)
            return y
        y = ctx.buf("ffn.out", (n, self.hidden), self.dtype)
        self.forward_into(x, ctx, y)
        return y

    def _parts(self, x: torch.Tensor, ctx) -> int:
        probe = ctx.buf("ffn.act", (x.shape[0], self.intermediate), self.dtype)
        return kernels.linear_parts_count(probe, self.w_down)

    def _act(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = x.shape[0]
        up = ctx.buf("ffn.up", (n, self.up_width), self.dtype)
        kernels.linear(x, self.w_up, up)
        act = ctx.buf("ffn.act", (n, self.intermediate), self.dtype)
        kernels.act_rows(up, act, self.act, gate_col=self.intermediate if self.scalar_gate is not None else -1)
        return act

    def forward_into(self, x: torch.Tensor, ctx, y: torch.Tensor) -> None:
        """The update written to ``y``: rows of the element type or float32 (one of a sum of parts that a caller keeps)."""
        kernels.linear(self._act(x, ctx), self.w_down, y)
