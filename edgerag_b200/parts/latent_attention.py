"""Causal attention through a low-rank latent, over the paged cache.

Per token the cache holds one row ``[c | kr]``: the normed latent ``c`` (``kv_rank`` wide) that every
head's keys and values are made from, and one rotated key part ``kr`` (``rot_dim`` wide) that all
heads share.  With per-head matrices ``Uk_h`` (``dim x kv_rank``) and ``Uv_h`` (``v_dim x kv_rank``):

    score(h, i, j) = (q_h,i[:dim] . Uk_h c_j  +  turn(q_h,i[dim:], i) . kr_j) * scale
    out_h,i        = sigmoid(g_h,i) * Uv_h  sum_j p(h, i, j) c_j

Nothing is up-projected per cached token: ``Uk_h`` is folded into the query (``Uk_h^T q``, one batched
product per step) and ``Uv_h`` is applied to the attention's result in the latent space, so the
attention kernel is multi-query attention over the cache rows, shared by all heads.  The softmax may
have a sink per head (a learnt logit that takes part in the denominator only), the queries may come
through a normed latent of their own (``q_rank``), and a layer may read the cache rows that another
layer wrote (``own_kv=False`` with a ``LayerCall`` that names that layer's cache and does not write).
With ``window`` a query sees its last ``window`` cache rows only (itself among them), the pages behind the
window go back to the pool, and ``gated=False`` leaves the sigmoid gate out.

The first product reads the mixer's input once for everything that is made from it: queries (or
their latent), the down-projection of ``[c | kr]`` and the gate logits.
"""

from __future__ import annotations

import torch

from ..cache.manager import KVGroupSpec
from ..ops import kernels
from .base import LayerCall, Mixer, WeightSpec, register_part
from .rope import rotary_frequencies


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, n_heads: int, dim: int, rot_dim: int, v_dim: int, kv_rank: int, scale: float,
                 rot_base: float, rot_dims: int, eps: float, dtype: torch.dtype, device: torch.device, q_rank: int = 0,
                 sink: bool = False, own_kv: bool = True, gated: bool = True, window: int = 0,
                 rot_scaling: dict | None = None) -> None:
        if rot_dim % 2 or rot_dims % 2 or rot_dims > rot_dim or kv_rank % 2:
            raise ValueError("latent attention: kv_rank, rot_dim and the rotated dimensions must be even, rot_dims <= rot_dim")
        self.hidden, self.n_heads, self.dim, self.rot_dim, self.v_dim = hidden, n_heads, dim, rot_dim, v_dim
        self.kv_rank, self.q_rank, self.rot_dims = kv_rank, int(q_rank or 0), rot_dims
        self.scale, self.eps = float(scale), float(eps)
        self.sink_on, self.own_kv, self.gated = bool(sink), bool(own_kv), bool(gated)
        self.window = int(window or 0)
        if self.window < 0:
            raise ValueError("latent attention: a window is positive (or 0 for none)")
        self.dtype, self.device = dtype, device
        self.q_width = n_heads * (dim + rot_dim)
        # columns of the fused first product: [queries or their latent | c and kr before norm and turn | gate logits]
        first = self.q_rank or self.q_width
        self.off_kv = first
        self.off_g = first + (kv_rank + rot_dim if own_kv else 0)
        self.in_width = _pad8(self.off_g + (n_heads if gated else 0))
        self.inv_freq = rotary_frequencies(rot_base, rot_dims, rot_scaling).to(device=device, dtype=torch.float32).contiguous()
        self.w_in = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None
        self.kv_norm = self.q_norm = self.sink = None

    def cache_spec(self) -> KVGroupSpec:
        return KVGroupSpec(1, 1, self.kv_rank + self.rot_dim, self.window, v_head_dim=0)

    def weight_specs(self) -> list[WeightSpec]:
        H, r = self.n_heads, self.kv_rank
        specs = []
        if self.q_rank:
            specs += [WeightSpec("dq", (self.q_rank, self.hidden)), WeightSpec("dq.norm", (self.q_rank,), "vector32"),
                      WeightSpec("uq", (self.q_width, self.q_rank))]
        else:
            specs.append(WeightSpec("q", (self.q_width, self.hidden)))
        if self.own_kv:
            specs += [WeightSpec("dkv", (r + self.rot_dim, self.hidden)), WeightSpec("dkv.norm", (r,), "vector32")]
        specs += [WeightSpec("uk", (H * self.dim, r)), WeightSpec("uv", (H * self.v_dim, r))]
        if self.sink_on:
            specs.append(WeightSpec("sink", (H,), "vector32"))
        if self.gated:
            specs.append(WeightSpec("g", (H, self.hidden)))
        return specs + [WeightSpec("o", (self.hidden, H * self.v_dim))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        cast = lambda t: t.to(device=self.device, dtype=self.dtype)          # noqa: E731
        f32 = lambda t: t.to(device=self.device, dtype=torch.float32).contiguous()   # noqa: E731
        H, r = self.n_heads, self.kv_rank
        rows = [cast(tensors["dq" if self.q_rank else "q"])]
        if self.own_kv:
            rows.append(cast(tensors["dkv"]))
            self.kv_norm = f32(tensors["dkv.norm"])
        if self.gated:
            rows.append(cast(tensors["g"]))
        have = sum(t.shape[0] for t in rows)
        if self.in_width > have:
            rows.append(torch.zeros((self.in_width - have, self.hidden), dtype=self.dtype, device=self.device))
        self.w_in = torch.cat(rows, 0).contiguous()
        if self.q_rank:
            self.w_uq = cast(tensors["uq"]).contiguous()
            self.q_norm = f32(tensors["dq.norm"])
        # Uk_h^T per head, [H, kv_rank, dim]: the query's unrotated part times it is the absorbed query
        self.w_uk_t = cast(tensors["uk"]).view(H, self.dim, r).transpose(1, 2).contiguous()
        self.w_uv = cast(tensors["uv"]).view(H, self.v_dim, r).contiguous()
        self.sink = f32(tensors["sink"]) if self.sink_on else None
        self.w_o = cast(tensors["o"]).contiguous()

    def _decode_plan(self, ctx, n_blocks: int, waves: int) -> tuple[int, int]:
        """(keys per split, splits) for the single-token rows: enough blocks for ``waves`` blocks per SM, splits
        of a multiple of 64 keys at multiples of their size; a function of the row count and the context bound alone."""
        bound = max(1, ctx.max_keys_bound())
        reach = min(bound, self.window) if self.window else bound        # keys a row reads
        want = max(1, min(-(-waves * kernels._sms(self.device) // max(1, n_blocks)), -(-reach // 64), kernels.LATENT_MAX_SPLITS))
        split = -(-(-(-reach // want)) // 64) * 64
        n_splits = -(-bound // split)
        if self.window:     # a window of w keys touches at most (w - 1) // split + 2 splits, wherever it lies
            n_splits = min(n_splits, (self.window - 1) // split + 2)
        return split, n_splits

    def _attend(self, ctx, q_lat, pages, tables, o_lat, gate) -> None:
        n, H, r = q_lat.shape[0], self.n_heads, self.kv_rank
        nd = ctx.n_decode
        if kernels.latent_mma_supported(self.dtype, r, self.rot_dim):
            # tensor cores: blocks of 16 or 32 (token, head) rows of one sequence; single tokens in splits
            if nd:
                mt = 1 if H <= 16 else 2
                tiles = kernels.latent_mma_tiles([1] * nd, H, mt)
                split, n_splits = self._decode_plan(ctx, tiles, 1)
                part = ctx.buf("latent.part", (kernels.latent_scratch_floats(nd, H, r, n_splits),), torch.float32) if n_splits > 1 else None
                kernels.latent_attention_mma(q_lat, pages, tables, ctx.seq_starts, ctx.positions, o_lat, self.scale, 0, nd, 0, nd,
                                             tiles, mt, gate=gate, sink=self.sink, split_keys=split, n_splits=n_splits, part=part,
                                             window=self.window)
            if n > nd:
                tiles = kernels.latent_mma_tiles(ctx.host_q_len[nd:], H, 2)
                kernels.latent_attention_mma(q_lat, pages, tables, ctx.seq_starts, ctx.positions, o_lat, self.scale, nd,
                                             ctx.n_seqs - nd, nd, n - nd, tiles, 2, gate=gate, sink=self.sink, window=self.window)
            return
        if nd:
            split, n_splits = self._decode_plan(ctx, -(-nd * H // 4), 2)
            part = ctx.buf("latent.part", (kernels.latent_scratch_floats(nd, H, r, n_splits),), torch.float32) if n_splits > 1 else None
            kernels.latent_attention(q_lat, pages, tables, ctx.seq_of_token, ctx.positions, o_lat, self.scale, 0, nd,
                                     gate=gate, sink=self.sink, split_keys=split, n_splits=n_splits, part=part, window=self.window)
        if n > nd:
            kernels.latent_attention(q_lat, pages, tables, ctx.seq_of_token, ctx.positions, o_lat, self.scale, nd, n - nd,
                                     gate=gate, sink=self.sink, window=self.window)

    def forward(self, x: torch.Tensor, ctx, call: LayerCall) -> torch.Tensor:
        n, H, r, dr = x.shape[0], self.n_heads, self.kv_rank, self.rot_dim
        proj = ctx.buf("latent.proj", (n, self.in_width), self.dtype)
        kernels.linear(x, self.w_in, proj)
        pages, _ = ctx.pages_of(call.cache_layer)
        group = ctx.group_of(call.cache_layer)
        write = call.writes_cache and self.own_kv
        q_latent = ctx.buf("latent.cq", (n, self.q_rank), self.dtype) if self.q_rank else None
        if write or self.q_rank:
            kernels.latent_store(proj, ctx.positions, self.eps, off_kv=self.off_kv if write else -1, rank=r, rot_dim=dr,
                                 kv_weight=self.kv_norm, inv_freq=self.inv_freq, rot_dims=self.rot_dims,
                                 slots=ctx.slots[group] if write else None, pages=pages if write else None, off_q=0,
                                 q_rank=self.q_rank, q_weight=self.q_norm, q_latent=q_latent)
        if self.q_rank:
            q = ctx.buf("latent.qfull", (n, self.q_width), self.dtype)
            kernels.linear(q_latent, self.w_uq, q)
        else:
            q = proj[:, : self.q_width]
        q_lat = ctx.buf("latent.q", (n, H, r + dr), torch.float32)
        kernels.latent_q_rotate(q, ctx.positions, self.inv_freq, H, self.dim, dr, r, self.rot_dims, q_lat)
        q_heads = q.as_strided((n, H, self.dim), (q.stride(0), self.dim + dr, 1))
        kernels.linear_batched(q_heads, self.w_uk_t, q_lat[:, :, :r])
        o_lat = ctx.buf("latent.o", (n, H, r), self.dtype)
        gate = proj[:, self.off_g: self.off_g + H] if self.gated else None
        self._attend(ctx, q_lat, pages, ctx.block_tables[group], o_lat, gate)
        heads = ctx.buf("latent.heads", (n, H, self.v_dim), self.dtype)
        kernels.linear_batched(o_lat, self.w_uv, heads)
        y = ctx.buf("mixer.out", (n, self.hidden), self.dtype)
        kernels.linear(heads.view(n, H * self.v_dim), self.w_o, y)
        return y
