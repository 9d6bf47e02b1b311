"""Layer norm with weight and bias, with the residual add fused in on either side.

``y = (x - mean) / sqrt(var + eps) * w + b`` with ``var`` the mean of the squared deviations, statistics
in float32 over the float32 stream.  As the norm before a sublayer it adds the pending update while it
reads (``forward``); the update may itself be waiting for a norm (``NormedUpdate``: a block whose
sublayers end in a norm), and then the closing norm, the add and this norm are one kernel.  As the norm
that closes a sublayer it is applied to the sublayer's output and added to the stream (``add_normed``).
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import Norm, NormedUpdate, WeightSpec, register_part, settle_update


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, dtype: torch.dtype, device: torch.device, tensor: str = "weight",
                 bias_tensor: str | None = None) -> None:
        """``tensor`` / ``bias_tensor``: names below the part's prefix (the bias defaults to ``tensor + ".b"``)."""
        self.size, self.eps = size, float(eps)
        self.dtype, self.device = dtype, device
        self.tensor = tensor
        self.bias_tensor = bias_tensor or tensor + ".b"
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.size,), kind="vector32"), WeightSpec(self.bias_tensor, (self.size,), kind="vector32")]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor].to(device=self.device, dtype=torch.float32).contiguous()
        self.bias = tensors[self.bias_tensor].to(device=self.device, dtype=torch.float32).contiguous()

    def _post(self, delta):
        """(rows or partial sums, the closing norm's (weight, bias, eps) or None) of a pending update; a
        closing norm of another kind is applied by itself first."""
        if not isinstance(delta, NormedUpdate):
            return delta, None
        if isinstance(delta.norm, LayerNorm):
            return delta.tensor, (delta.norm.weight, delta.norm.bias, delta.norm.eps)
        return None, None

    def forward(self, hidden, out, delta=None, rows=None, write_back=True, settled=False) -> None:
        if isinstance(delta, NormedUpdate) and delta.bias is not None:
            raise ValueError("a layer norm has no kernel for an update that carries a bias")
        if isinstance(delta, NormedUpdate) and not isinstance(delta.norm, LayerNorm):
            if rows is not None or not write_back:
                raise ValueError("a pending update closed by another kind of norm can only be added to all rows")
            settle_update(hidden, delta, self.dtype)
            delta = None
        rows_or_parts, post = self._post(delta)
        kernels.add_layernorm(hidden, self.weight, self.bias, out, self.eps, delta=rows_or_parts, post=post, rows=rows,
                              write_back=write_back)

    def add_normed(self, hidden: torch.Tensor, x: torch.Tensor) -> None:
        kernels.add_layernorm(hidden, None, None, None, self.eps, delta=x, post=(self.weight, self.bias, self.eps))

    def add_normed_cast(self, hidden: torch.Tensor, x: torch.Tensor | None, out: torch.Tensor) -> None:
        """``out = cast(hidden + self(x))`` without touching ``hidden`` (``x`` None: the plain cast)."""
        kernels.add_layernorm(hidden, None, None, out, self.eps, delta=x,
                              post=None if x is None else (self.weight, self.bias, self.eps), write_back=False)
