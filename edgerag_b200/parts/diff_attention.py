"""Differential attention over the paged cache: two softmax maps per head over the same values.

With ``H`` query heads, ``G`` key/value heads (query head ``h`` reads kv head ``h // (H / G)``), map size ``dim`` and
value size ``v_dim``, the query projection has ``H * 2 * dim`` rows and the key projection ``G * 2 * dim``, laid out head
by head as ``[map 1 | map 2]``.  Per head:

    s_m(i, j) = cap(q_m,i . k_m,j * scale),   cap(s) = softcap * tanh(s / softcap)   (no cap: s)
    a_m,i     = sum_j softmax_j(s_m(i, j)) v_j                      over the keys the mask lets i see
    o_i       = a_1,i - lambda a_2,i,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff   (one number per layer)
    out_i     = o_i / sqrt(mean(o_i^2) + eps) * (1 - diff)

then the output projection over the concatenated heads.  Before the maps are taken: an optional short causal
convolution over time on every channel of q, k and v (``conv`` taps, tensors ``<name>.conv`` of shape ``[channels,
taps]``, no bias, no activation), whose last ``conv - 1`` inputs per request live in a state record, and a rotation of
the halves of the first ``rot_dims`` entries of every map of q and k by ``position * f_i``, with frequencies that may be
stretched for long wavelengths (``parts.rope.rotary_frequencies``).  A ``window`` limits a query to its last ``window``
keys; pages behind every live window go back to the pool.

The cache holds, per token and kv head, both maps' keys side by side (``2 * dim``) and one value row (``v_dim``).
The kernels of ``csrc/diff_attention.cu`` do the work between the fused input product and the output product:
``diff_prepare`` (convolution, rotation, cache write), ``diff_attention`` (both maps in one walk over the keys; the
difference, the head norm and the constant in its epilogue; single tokens with long reaches in splits of the keys),
``diff_attention_mma`` (the same on tensor cores for prompt portions in bfloat16: both maps' weights meet one tile of
values) and, from ``csrc/ssm.cu``, the update of the convolution's state record.
"""

from __future__ import annotations

import torch

from ..cache.manager import KVGroupSpec, StateSpec
from ..ops import kernels
from .base import LayerCall, Mixer, WeightSpec, register_part
from .rope import rotary_frequencies


@register_part("mixer", "diff_attention")
class DiffAttention(Mixer):
    graph_safe = True
    #: prompt tokens of a step from which the tensor-core kernel (tiles of 64 tokens) takes the portions
    MMA_FROM_TOKENS = 32

    def __init__(self, hidden: int, n_q_heads: int, n_kv_heads: int, dim: int, v_dim: int, scale: float, diff: float,
                 eps: float, dtype: torch.dtype, device: torch.device, window: int = 0, softcap: float = 0.0, conv: int = 0,
                 rot_base: float = 10000.0, rot_dims: int = 0, rot_scaling: dict | None = None) -> None:
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} query heads are not divisible by {n_kv_heads} kv heads")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError(f"diff_attention: rot_dims {rot_dims} must be even and at most the map size {dim}")
        if v_dim > kernels.DIFF_MAX_V_DIM:
            raise ValueError(f"diff_attention: values of {v_dim} entries (at most {kernels.DIFF_MAX_V_DIM})")
        if window < 0 or conv < 0:
            raise ValueError("diff_attention: window and conv are not negative")
        self.hidden, self.n_q, self.n_kv, self.dim, self.v_dim = hidden, n_q_heads, n_kv_heads, dim, v_dim
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.window, self.softcap, self.taps = int(window), float(softcap or 0.0), int(conv or 0)
        self.rot_dims = int(rot_dims)
        self.dtype, self.device = dtype, device
        self.q_width, self.k_width, self.v_width = n_q_heads * 2 * dim, n_kv_heads * 2 * dim, n_kv_heads * v_dim
        self.channels = self.q_width + self.k_width + self.v_width
        self.in_width = -(-self.channels // 8) * 8            # rows of the fused product start 16-byte aligned
        self.inv_freq = None
        if self.rot_dims:
            self.inv_freq = rotary_frequencies(rot_base, self.rot_dims, rot_scaling).to(device=device, dtype=torch.float32).contiguous()
        self.w_in = self.w_o = self.conv_w = None
        self.lam = 0.0

    def cache_spec(self) -> list:
        """Pages for keys and values, and (with a convolution) one state record per request."""
        spec: list = [KVGroupSpec(1, self.n_kv, 2 * self.dim, self.window, v_head_dim=self.v_dim)]
        if self.taps > 1:
            spec.append(StateSpec("qkv_conv", (self.taps - 1, self.channels)))
        return spec

    def weight_specs(self) -> list[WeightSpec]:
        specs = []
        for name, rows in (("q", self.q_width), ("k", self.k_width), ("v", self.v_width)):
            specs.append(WeightSpec(name, (rows, self.hidden)))
            if self.taps:
                specs.append(WeightSpec(name + ".conv", (rows, self.taps), "vector32"))
        specs += [WeightSpec(n, (self.dim,), "vector32") for n in ("lq1", "lk1", "lq2", "lk2")]
        return specs + [WeightSpec("o", (self.hidden, self.n_q * self.v_dim))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)          # noqa: E731
        rows = [cast(tensors[n]) for n in ("q", "k", "v")]
        if self.in_width > self.channels:
            rows.append(torch.zeros((self.in_width - self.channels, self.hidden), dtype=self.dtype, device=self.device))
        self.w_in = torch.cat(rows, 0).contiguous()
        self.w_o = cast(tensors["o"]).contiguous()
        if self.taps:
            self.conv_w = torch.cat([tensors[n + ".conv"].to(device=self.device, dtype=torch.float32) for n in ("q", "k", "v")],
                                    0).contiguous()
        f64 = lambda n: tensors[n].to(dtype=torch.float64, device="cpu")     # noqa: E731
        self.lam = float(torch.exp((f64("lq1") * f64("lk1")).sum()) - torch.exp((f64("lq2") * f64("lk2")).sum()) + self.diff)

    def _decode_plan(self, ctx, n_rows: int) -> tuple[int, int]:
        """(keys per split, splits) for the single-token rows: enough blocks for two per SM, splits of a multiple of 64
        keys; a function of the row count, the window and the step's context bound alone."""
        bound = max(1, ctx.max_keys_bound())
        reach = min(bound, self.window) if self.window else bound
        blocks = -(-n_rows // 4)
        want = max(1, min(-(-2 * kernels._sms(self.device) // max(1, blocks)), -(-reach // 64), 64))
        split = -(-(-(-reach // want)) // 64) * 64
        n_splits = -(-bound // split)
        if self.window:     # a window of w keys touches at most (w - 1) // split + 2 splits, wherever it lies
            n_splits = min(n_splits, (self.window - 1) // split + 2)
        return split, n_splits

    def forward(self, x: torch.Tensor, ctx, call: LayerCall) -> torch.Tensor:
        n = x.shape[0]
        proj = ctx.buf("diff.proj", (n, self.in_width), self.dtype)
        kernels.linear(x, self.w_in, proj)
        k_pages, v_pages = ctx.pages_of(call.cache_layer)
        group = ctx.group_of(call.cache_layer)
        state = ctx.state("qkv_conv", call.cache_layer) if self.taps > 1 else None
        q = ctx.buf("diff.q", (n, self.q_width), self.dtype)
        kernels.diff_prepare(proj, q, ctx.positions, self.n_q, self.n_kv, self.dim, self.v_dim, inv_freq=self.inv_freq,
                             rot_dims=self.rot_dims, conv_w=self.conv_w, conv_state=state, seq_of_token=ctx.seq_of_token,
                             seq_starts=ctx.seq_starts, state_slots=ctx.state_slots,
                             slots=ctx.slots[group] if call.writes_cache else None, k_pages=k_pages, v_pages=v_pages,
                             page_size=ctx.page_size)
        if state is not None:     # (after the convolution has read the old record)
            kernels.conv_state_update(proj, 0, state, ctx.n_seqs, ctx.seq_starts, ctx.state_slots)
        out = ctx.buf("diff.out", (n, self.n_q * self.v_dim), self.dtype)
        tables = ctx.block_tables[group]
        nd = ctx.n_decode
        common = dict(window=self.window, softcap=self.softcap)
        mma = kernels.diff_mma_supported(self.dtype, self.dim, self.v_dim)
        rep = self.n_q // self.n_kv
        if nd:
            # single tokens: a block per (sequence, kv head, split) on tensor cores, else a warp per (token, head, split)
            split, n_splits = self._decode_plan(ctx, nd * (self.n_kv * 4 if mma else self.n_q))
            part = None
            if n_splits > 1:
                part = ctx.buf("diff.part", (nd * self.n_q * n_splits * kernels.diff_part_floats(self.v_dim),), torch.float32)
            if mma:
                rows = (kernels.DIFF_MMA_PACKED_ROWS if rep <= kernels.DIFF_MMA_PACKED_ROWS else
                        kernels.DIFF_MMA_TOKEN_ROWS if rep <= kernels.DIFF_MMA_TOKEN_ROWS else kernels.DIFF_MMA_ROWS)
                kernels.diff_attention_mma(q, k_pages, v_pages, tables, ctx.seq_starts, ctx.positions, out, self.n_q, self.scale,
                                           self.lam, self.eps, 1.0 - self.diff, 0, nd, 0, nd, nd * -(-rep // rows),
                                           split_keys=split, n_splits=n_splits, part=part, tile_rows=rows, **common)
            else:
                kernels.diff_attention(q, k_pages, v_pages, tables, ctx.seq_of_token, ctx.positions, out, self.n_q, self.scale,
                                       self.lam, self.eps, 1.0 - self.diff, 0, nd, split_keys=split, n_splits=n_splits, part=part,
                                       **common)
        if n - nd >= self.MMA_FROM_TOKENS and mma:
            # portions of prompts on tensor cores: blocks of 64 (token, head) rows of one sequence and one kv head
            kernels.diff_attention_mma(q, k_pages, v_pages, tables, ctx.seq_starts, ctx.positions, out, self.n_q, self.scale,
                                       self.lam, self.eps, 1.0 - self.diff, nd, ctx.n_seqs - nd, nd, n - nd,
                                       kernels.diff_mma_tiles(ctx.host_q_len[nd:], rep), **common)
        elif n > nd:
            kernels.diff_attention(q, k_pages, v_pages, tables, ctx.seq_of_token, ctx.positions, out, self.n_q, self.scale,
                                   self.lam, self.eps, 1.0 - self.diff, nd, n - nd, **common)
        y = ctx.buf("mixer.out", (n, self.hidden), self.dtype)
        kernels.linear(out, self.w_o, y)
        return y
