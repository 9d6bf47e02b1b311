"""A mixer with a matrix state per head that is corrected towards each token's value: the gated delta rule.

One input product gives, per token, ``q | k | v | gate | b | a`` (``key_heads * key_dim`` entries for q and for k,
``heads * v_dim`` for v and for the gate, one b and one a per head).  ``q | k | v`` pass a short causal convolution per
channel (no bias) and silu.  Head ``h`` uses the queries and keys of key head ``h // (heads / key_heads)``, made unit
vectors ``x / sqrt(sum(x^2) + 1e-6)``, the query also times ``key_dim ** -0.5``.  With ``beta = sigmoid(b)`` and
``g = exp(-exp(A_log_h) * softplus(a + dt_bias_h))``, per token in this order:

    S <- g S;    u = beta (v - S^T k);    S <- S + k u^T;    o = S^T q             S: [key_dim, v_dim], float32

so the read-out sees the token's own write.  ``o`` of every head is brought to unit RMS over ``v_dim`` and scaled by
one weight vector shared by the heads, multiplied by ``silu(gate)``, and projected out.  Between steps a request keeps
two records in its state slot: the last ``conv - 1`` inputs of the convolution, and ``S`` of every head (stored with
the value index first); a new slot holds zeros, so a sequence starts from nothing and a portion of a prompt continues
exactly where the one before it stopped.  Unit vectors, ``beta``, ``g``, the state, ``o`` and its norm are float32
whatever the element type.
"""

from __future__ import annotations

import torch

from ..cache.manager import StateSpec
from ..ops import kernels
from .base import LayerCall, Mixer, WeightSpec, register_part


@register_part("mixer", "gated_delta")
class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, n_heads: int, n_key_heads: int, key_dim: int, v_dim: int, conv: int, eps: float,
                 dtype: torch.dtype, device: torch.device, names: dict[str, str] | None = None) -> None:
        if n_heads % n_key_heads or conv < 1:
            raise ValueError("gated_delta: the key heads must divide the heads; conv >= 1")
        if key_dim > kernels.DELTA_MAX_KEY_DIM:
            raise ValueError(f"gated_delta: keys of {key_dim} entries (at most {kernels.DELTA_MAX_KEY_DIM})")
        self.hidden, self.n_heads, self.n_key_heads, self.key_dim, self.v_dim = hidden, n_heads, n_key_heads, key_dim, v_dim
        self.taps, self.eps = int(conv), float(eps)
        self.dtype, self.device = dtype, device
        self.qk_width = n_key_heads * key_dim
        self.inner = n_heads * v_dim
        self.channels = 2 * self.qk_width + self.inner           # what the convolution acts on: q | k | v
        self.off_gate = self.channels
        self.off_b = self.off_gate + self.inner
        self.off_a = self.off_b + n_heads
        self.in_true = self.off_a + n_heads
        self.in_width = -(-self.in_true // 8) * 8
        self.names = {"q": "q", "k": "k", "v": "v", "gate": "g", "b": "b", "a": "a", "q_conv": "q.conv", "k_conv": "k.conv",
                      "v_conv": "v.conv", "dt_bias": "dt_bias", "A_log": "A_log", "norm": "norm", "o": "o", **(names or {})}
        self.w_in = self.w_conv = self.w_o = self.dt_bias = self.a_log = self.norm_w = None

    def cache_spec(self) -> list[StateSpec]:
        conv = [StateSpec("conv", (self.taps - 1, self.channels))] if self.taps > 1 else []
        return conv + [StateSpec("delta", (self.n_heads, self.v_dim, self.key_dim))]

    def weight_specs(self) -> list[WeightSpec]:
        nm, H, h = self.names, self.n_heads, self.hidden
        return [WeightSpec(nm["q"], (self.qk_width, h)), WeightSpec(nm["k"], (self.qk_width, h)),
                WeightSpec(nm["v"], (self.inner, h)), WeightSpec(nm["gate"], (self.inner, h)),
                WeightSpec(nm["b"], (H, h)), WeightSpec(nm["a"], (H, h)),
                WeightSpec(nm["q_conv"], (self.qk_width, self.taps)), WeightSpec(nm["k_conv"], (self.qk_width, self.taps)),
                WeightSpec(nm["v_conv"], (self.inner, self.taps)),
                WeightSpec(nm["dt_bias"], (H,), "vector32"), WeightSpec(nm["A_log"], (H,), "vector32"),
                WeightSpec(nm["norm"], (self.v_dim,), "vector32"), WeightSpec(nm["o"], (h, self.inner))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        nm = self.names
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)                   # noqa: E731
        f32 = lambda t: t.to(device=self.device, dtype=torch.float32).contiguous()   # noqa: E731
        rows = [cast(tensors[nm[key]]) for key in ("q", "k", "v", "gate", "b", "a")]
        if self.in_width > self.in_true:
            rows.append(torch.zeros((self.in_width - self.in_true, self.hidden), dtype=self.dtype, device=self.device))
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_conv = torch.cat([cast(tensors[nm[key]]) for key in ("q_conv", "k_conv", "v_conv")], 0).contiguous()
        self.dt_bias, self.a_log, self.norm_w = f32(tensors[nm["dt_bias"]]), f32(tensors[nm["A_log"]]), f32(tensors[nm["norm"]])
        self.w_o = cast(tensors[nm["o"]]).contiguous()

    def forward(self, x: torch.Tensor, ctx, call: LayerCall) -> torch.Tensor:
        n = x.shape[0]
        proj = ctx.buf("delta.proj", (n, self.in_width), self.dtype)
        kernels.linear(x, self.w_in, proj)
        qkv = ctx.buf("delta.qkv", (n, self.channels), self.dtype)
        if self.taps > 1:
            conv_state = ctx.state("conv", call.cache_layer)
            kernels.conv_silu(proj, 0, self.w_conv, None, conv_state, ctx.seq_of_token, ctx.seq_starts, ctx.state_slots, qkv)
            kernels.conv_state_update(proj, 0, conv_state, ctx.n_seqs, ctx.seq_starts, ctx.state_slots)
        else:
            kernels.conv_silu(proj, 0, self.w_conv, None, ctx.buf("delta.no_conv_state", (1, 0, self.channels), torch.float32),
                              ctx.seq_of_token, ctx.seq_starts, ctx.state_slots, qkv)
        o = ctx.buf("delta.o", (n, self.inner), torch.float32)
        kernels.delta_scan(qkv, proj, self.off_b, self.off_a, self.dt_bias, self.a_log, ctx.state("delta", call.cache_layer),
                           ctx.n_seqs, ctx.seq_starts, ctx.state_slots, o, self.n_key_heads, self.key_dim,
                           ctx.buf("delta.scratch", (kernels.delta_scratch_floats(n, self.n_heads, self.n_key_heads, self.key_dim,
                                                                                  self.v_dim),), torch.float32))
        gated = ctx.buf("delta.gated", (n, self.inner), self.dtype)
        kernels.head_norm_gate(o, proj[:, self.off_gate: self.off_gate + self.inner], self.norm_w, gated, self.n_heads, self.eps)
        n_parts = kernels.linear_parts_count(gated, self.w_o)
        if n_parts:
            y = ctx.buf("mixer.out_parts", (n_parts, n, self.hidden), torch.float32)
            kernels.linear_parts(gated, self.w_o, y)
            return y
        y = ctx.buf("mixer.out", (n, self.hidden), self.dtype)
        kernels.linear(gated, self.w_o, y)
        return y
