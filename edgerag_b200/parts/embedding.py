"""Input and output ends of the decoder.

``TokenEmbedding``: a table lookup (times a constant where the model has one), or rows of caller-given embeddings
(edgerag/core/model.py:106-110: exactly one of ids and embeddings per token); the result is
written to the float32 residual stream.  ``LMHead``: bias-free projection to float32 logits over
the rows that were asked for (edgerag/core/model.py:150-152); where the plan names a tensor to
tie the head to, a checkpoint without a head of its own shares that tensor.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import Part, PartSpec, WeightSpec, build_part, register_part


@register_part("embedding", "table")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, dtype: torch.dtype, device: torch.device, scale: float = 1.0,
                 tensor: str = "weight", norm: PartSpec | None = None) -> None:
        """``scale`` multiplies every row as it enters the float32 stream; ``tensor`` names the table; ``norm``: a norm
        that acts on the stream right after the lookup (its tensors' names are relative to this part's prefix)."""
        self.vocab, self.hidden = vocab, hidden
        self.dtype, self.device = dtype, device
        self.scale, self.tensor = float(scale), tensor
        self.weight: torch.Tensor | None = None
        self._norm_prefix = norm.prefix if norm is not None else ""
        self.norm = build_part("norm", norm, dtype, device) if norm is not None else None
        if self.norm is not None and not hasattr(self.norm, "norm_stream"):
            raise ValueError(f"norm {norm.kind!r} cannot act on the stream in place")
        self.graph_safe = self.norm is None or bool(getattr(self.norm, "graph_safe", False))

    def weight_specs(self) -> list[WeightSpec]:
        specs = [WeightSpec(self.tensor, (self.vocab, self.hidden))]
        if self.norm is not None:
            specs += [WeightSpec(self._norm_prefix + s.name, s.shape, s.kind, s.fallback) for s in self.norm.weight_specs()]
        return specs

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor].to(device=self.device, dtype=self.dtype).contiguous()
        if self.norm is not None:
            self.norm.load_weights({s.name: tensors[self._norm_prefix + s.name] for s in self.norm.weight_specs()})

    def forward(self, ctx, hidden: torch.Tensor) -> None:
        kernels.embed_rows(hidden, self.weight, ctx.token_ids, ctx.status, embeds=ctx.embeds,
                           embed_row=ctx.embed_row if ctx.embeds is not None else None, scale=self.scale)
        if self.norm is not None:
            self.norm.norm_stream(hidden)


@register_part("head", "linear")
class LMHead(Part):
    graph_safe = True

    def __init__(self, vocab: int, hidden: int, dtype: torch.dtype, device: torch.device,
                 tied_to: str | None = None, softcap: float = 0.0, tensor: str = "weight", scale: float = 1.0) -> None:
        """``tied_to``: model-relative name of the tensor to share when the checkpoint has no head of
        its own (the plan names it; this part does not know what the model calls its embedding).
        ``softcap`` c > 0: logits <- c * tanh(logits / c), in float; ``scale``: a constant that multiplies the
        float logits (after the cap)."""
        self.scale = float(scale)
        self.vocab, self.hidden, self.tied_to = vocab, hidden, tied_to
        self.dtype, self.device = dtype, device
        self.softcap, self.tensor = float(softcap or 0.0), tensor
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.vocab, self.hidden), fallback=self.tied_to)]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor].to(device=self.device, dtype=self.dtype).contiguous()

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> None:
        kernels.linear(x, self.weight, logits)
        if self.softcap > 0.0:
            kernels.softcap(logits, self.softcap, self.dtype)
        if self.scale != 1.0:
            kernels.scale_rows(logits, self.scale, self.dtype)
