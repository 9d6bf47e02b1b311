"""RMSNorm with the residual add fused in.

The reference's formula (edgerag/core/layers.py:40-47): statistics in float32, the normalised
value cast back to the model's element type, then the weight multiply.  Here the residual stream
itself stays in float32, so the sum ``hidden + delta`` that the reference forms in 16-bit
(edgerag/core/layers.py:372-373) is exact to float32.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import Norm, NormedUpdate, ScaledUpdate, WeightSpec, register_part, settle_update


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device, weight_offset: float = 0.0,
                 exact: bool = False, tensor: str = "weight") -> None:
        """``weight_offset``: the stored tensor is the scale minus this (1.0 for weights kept around zero);
        ``exact``: the normed value is not rounded to the element type before the scale multiplies it, so the
        norm is float up to its store; ``tensor``: the tensor's name below the part's prefix."""
        self.size = size
        self.eps = float(eps)
        self.dtype = dtype
        self.device = device
        self.weight_offset = float(weight_offset)
        self.exact = bool(exact)
        self.tensor = tensor
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.size,), kind="vector32")]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        w = tensors[self.tensor].to(device=self.device, dtype=torch.float32)
        self.weight = (w + self.weight_offset if self.weight_offset else w).contiguous()

    def forward(self, hidden, out, delta=None, rows=None, write_back=True, settled=False) -> None:
        if isinstance(delta, NormedUpdate):
            post = delta.norm
            if isinstance(post, RMSNorm) and not post.weight_offset and not self.weight_offset:
                # the closing norm, the add and this norm in one kernel, all float
                kernels.rms_between(hidden, out, weight=self.weight, eps=self.eps, delta=delta.tensor, bias=delta.bias,
                                    post=(post.weight, post.eps), rows=rows, write_back=write_back)
                return
            if rows is not None or not write_back:
                raise ValueError("a pending update that another kind of norm has to close can only be added to all rows")
            settle_update(hidden, delta, self.dtype)
            delta, settled = None, False
        scale = 1.0
        if isinstance(delta, ScaledUpdate):      # the constant rides into the kernel that adds the update
            delta, scale = delta.tensor, delta.scale
        kernels.add_rmsnorm(hidden, self.weight, out, self.eps, delta=delta, rows=rows, write_back=write_back, settled=settled,
                            exact=self.exact, delta_scale=scale)

    def add_normed(self, hidden: torch.Tensor, x: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        kernels.rms_between(hidden, None, delta=x, bias=bias, post=(self._plain_weight(), self.eps), dtype=self.dtype)

    def add_normed_cast(self, hidden: torch.Tensor, x: torch.Tensor | None, out: torch.Tensor,
                        bias: torch.Tensor | None = None, write_back: bool = False) -> None:
        """``out = cast(hidden + self(x + bias))`` (``x`` None: the plain cast); ``hidden`` keeps the sum when ``write_back``."""
        kernels.rms_between(hidden, out, delta=x, bias=bias, post=None if x is None else (self._plain_weight(), self.eps),
                            write_back=write_back)

    def norm_stream(self, hidden: torch.Tensor) -> None:
        """``hidden = self(hidden)`` in place, in float (a norm that acts on the stream itself, as after an embedding)."""
        kernels.rms_between(hidden, None, own=(self._plain_weight(), self.eps), dtype=self.dtype)

    def _plain_weight(self) -> torch.Tensor:
        return self.weight        # (the offset was added when the tensor was loaded)


@register_part("norm", "pass")
class PassNorm(Norm):
    """No norm: a sublayer that reads the residual stream as it is.  ``out`` receives the stream (plus the pending
    update) rounded to the element type; a pending update that a norm has to close is closed in the same kernel
    where that norm has one (``add_normed_cast``)."""

    graph_safe = True

    def __init__(self, dtype: torch.dtype, device: torch.device, size: int | None = None, **_unused) -> None:
        self.dtype, self.device, self.size = dtype, device, size

    def forward(self, hidden, out, delta=None, rows=None, write_back=True, settled=False) -> None:
        post = bias = None
        if isinstance(delta, NormedUpdate):
            if isinstance(delta.norm, RMSNorm):
                post, bias, delta = (delta.norm.weight, delta.norm.eps), delta.bias, delta.tensor
            else:
                if rows is not None or not write_back:
                    raise ValueError("a pending update that another kind of norm has to close can only be added to all rows")
                settle_update(hidden, delta, self.dtype)
                delta = None
        kernels.rms_between(hidden, out, delta=delta, bias=bias, post=post, rows=rows, write_back=write_back)
