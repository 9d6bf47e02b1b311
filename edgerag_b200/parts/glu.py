"""A gated feed-forward with bounded branches: ``down(act(gate(x), up(x)))`` with

    g = min(gate, limit),  u = clamp(up, -limit, limit),  act = g * sigmoid(alpha * g) * (u + shift).

``alpha``, ``shift`` and ``limit`` are constructor arguments (``limit <= 0``: unbounded; ``alpha = 1, shift = 0``
is the SwiGLU gate), as are the tensors' names.  ``act = "gelu_tanh"`` puts the tanh form of gelu,
``0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))``, in the place of ``g * sigmoid(alpha * g)``.  ``gate`` and ``up`` are stored as one matrix so that one
product feeds the activation kernel, which works in float and rounds once; for the few rows of a decode step
the product and the gate are one kernel with the same result.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import FeedForward, WeightSpec, register_part


@register_part("ffn", "glu_bounded")
class BoundedGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, dtype: torch.dtype, device: torch.device, limit: float = 0.0,
                 alpha: float = 1.0, shift: float = 0.0, names: tuple[str, str, str] = ("gate", "up", "down"),
                 act: str = "sigmoid") -> None:
        if act not in kernels.GLU_ACTS:
            raise ValueError(f"unknown gate activation {act!r}; known: {sorted(kernels.GLU_ACTS)}")
        self.act = act
        self.hidden, self.intermediate = hidden, intermediate
        self.dtype, self.device = dtype, device
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.names = tuple(names)
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        gate, up, down = self.names
        return [WeightSpec(gate, (self.intermediate, self.hidden)), WeightSpec(up, (self.intermediate, self.hidden)),
                WeightSpec(down, (self.hidden, self.intermediate))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        gate, up, down = self.names
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)  # noqa: E731
        self.w_gate_up = torch.cat([cast(tensors[gate]), cast(tensors[up])], 0).contiguous()
        self.w_down = cast(tensors[down]).contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        y = ctx.buf("ffn.out", (x.shape[0], self.hidden), self.dtype)
        self.forward_into(x, ctx, y)
        return y

    def forward_into(self, x: torch.Tensor, ctx, y: torch.Tensor) -> None:
        """The update written to ``y``: rows of the element type or float32 (one of a sum of parts that a caller keeps)."""
        n = x.shape[0]
        act = ctx.buf("ffn.act", (n, self.intermediate), self.dtype)
        if kernels.linear_glu_supported(x, self.w_gate_up):
            # a few rows: product and gate in one kernel, the same bits as the two kernels below
            kernels.linear_glu(x, self.w_gate_up, act, bounded=(self.limit, self.alpha, self.shift, self.act))
        else:
            gate_up = ctx.buf("ffn.gate_up", (n, 2 * self.intermediate), self.dtype)
            kernels.linear(x, self.w_gate_up, gate_up)
            kernels.glu_bounded(gate_up, act, self.limit, self.alpha, self.shift, self.act)
        kernels.linear(act, self.w_down, y)
