"""Block arrangements: how a layer's norms, mixer and feed-forward are wired around the residual.

``PreNormBlock`` is the reference's ``DecoderLayer`` (edgerag/core/layers.py:366-374):
``h += mixer(norm1(h)); h += ffn(norm2(h))``.  Each residual add is fused into the norm that
follows it, so a block receives the previous block's update as ``delta`` and returns its own
feed-forward output as the update that is still to be added.

``SandwichBlock`` has a norm on both sides of each sublayer: ``h += post1(mixer(norm1(h))); h += post2(ffn(norm2(h)))``.
The closing norms belong to the block (their tensors sit beside the layer's other norms).  With the ``pass`` norm in
the opening places it is the arrangement whose sublayers read the stream itself and norm only what they add.  An update leaves a
sublayer as a ``NormedUpdate``, so that the closing norm, the residual add and the norm that opens the next
sublayer run as one kernel where the norms have one.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import (Block, FeedForward, LayerCall, Mixer, Norm, NormedUpdate, PartSpec, ScaledUpdate, WeightSpec, build_part,
                   register_part)


@register_part("block", "prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None, ffn: FeedForward | None, hidden: int,
                 dtype: torch.dtype, device: torch.device, update_scale: float = 1.0) -> None:
        """``norm2`` and ``ffn`` are None for a layer that is its mixer's sublayer only.  ``update_scale`` m:
        ``h += m * mixer(norm1(h)); h += m * ffn(norm2(h))`` (the norms then have to take a ``ScaledUpdate``)."""
        self.update_scale = float(update_scale)
        if getattr(mixer, "has_update_bias", False):
            raise ValueError("a mixer whose update carries a bias needs a block that closes the update with a norm")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.hidden = hidden
        self.dtype = dtype

    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx, call: LayerCall) -> torch.Tensor:
        n = hidden.shape[0]
        x = ctx.buf("block.normed", (n, self.hidden), self.dtype)
        # A norm may read the stream while the kernel before it still runs if that kernel did not write the
        # stream: true when at least one kernel of this package has been launched since the stream's last
        # writer (`ctx.stream_written`, the launch count right after it).
        settled = lambda: kernels.launches() > getattr(ctx, "stream_written", float("inf"))   # noqa: E731
        self.norm1.forward(hidden, x, delta, settled=settled())   # hidden += delta; x = norm1(hidden)
        if delta is not None:
            ctx.stream_written = kernels.launches()
        scaled = (lambda u: ScaledUpdate(u, self.update_scale)) if self.update_scale != 1.0 else (lambda u: u)   # noqa: E731
        mixed = scaled(self.mixer.forward(x, ctx, call))
        if self.ffn is None:
            return mixed                               # added by whichever norm comes next
        self.norm2.forward(hidden, x, mixed, settled=settled())   # hidden += mixed; x = norm2(hidden)
        ctx.stream_written = kernels.launches()
        return scaled(self.ffn.forward(x, ctx))       # added by whichever norm comes next


@register_part("block", "sandwich")
class SandwichBlock(Block):
    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm | None, ffn: FeedForward | None, hidden: int,
                 dtype: torch.dtype, device: torch.device, post1: PartSpec, post2: PartSpec | None = None) -> None:
        """``post1`` / ``post2``: the norms that close the mixer's and the feed-forward's sublayer (``post2`` None
        for a layer without a feed-forward); their prefixes are relative to the layer."""
        if (ffn is None) != (post2 is None):
            raise ValueError("a closing norm of the feed-forward comes with the feed-forward or not at all")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.hidden, self.dtype = hidden, dtype
        self._post_specs = [post1] + ([post2] if post2 is not None else [])
        self.post1 = build_part("norm", post1, dtype, device)
        self.post2 = build_part("norm", post2, dtype, device) if post2 is not None else None
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in (self.post1, self.post2) if p is not None)

    def _posts(self):
        return [(spec.prefix, part) for spec, part in zip(self._post_specs, (self.post1, self.post2)) if part is not None]

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(prefix + s.name, s.shape, s.kind, s.fallback) for prefix, part in self._posts()
                for s in part.weight_specs()]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        for prefix, part in self._posts():
            part.load_weights({s.name: tensors[prefix + s.name] for s in part.weight_specs()})

    def forward(self, hidden: torch.Tensor, delta, ctx, call: LayerCall):
        n = hidden.shape[0]
        x = ctx.buf("block.normed", (n, self.hidden), self.dtype)
        self.norm1.forward(hidden, x, delta)             # hidden += (closed) delta; x = norm1(hidden)
        if delta is not None:
            ctx.stream_written = kernels.launches()
        mixed = NormedUpdate(self.mixer.forward(x, ctx, call), self.post1, self.mixer.update_bias)
        if self.ffn is None:
            return mixed                                  # closed and added by whichever norm comes next
        self.norm2.forward(hidden, x, mixed)             # hidden += post1(mixed); x = norm2(hidden)
        ctx.stream_written = kernels.launches()
        return NormedUpdate(self.ffn.forward(x, ctx), self.post2)
