"""Causal grouped-query attention over the paged cache: the mixer of the Llama decoder.

Formulas of the reference's ``Attention`` (edgerag/core/layers.py:278-322): bias-free q/k/v/o
projections, position encoding on q and k before the cache write, kv head ``h // (nq / nkv)``
serving query head ``h`` (edgerag/core/layers.py:117-134), scores scaled by ``head_dim ** -0.5``
(edgerag/core/layers.py:276), softmax in float32.  The three input projections are stored as one
matrix ``[Wq; Wk; Wv]`` (row concatenation leaves every output column's arithmetic unchanged), so
one product yields a row ``q heads | k heads | v heads`` per token.

Options beyond the Llama decoder's, all constructor arguments: a ``window`` with ``keep_first`` (a query sees
the last ``window`` keys and the first ``keep_first`` of its sequence, each at its true position), ``scale``,
biases on q and k (``qk_bias``), a unit-RMS norm per head on q and k before the position encoding with one
weight vector for all heads (``qk_norm_eps``), values that are the keys as projected, before norm and
encoding (``values_are_keys``: no value projection; the cache still holds keys and values), and the tensors'
names (``names``).  With any of bias, norm or shared values the step after the product is one kernel
(``kernels.qk_prepare``) that also writes the cache.

A second family of options, also one kernel after the product (``kernels.qkv_whole_norm``): biases on all four
projections (``all_bias``; the output's rides with the update to whoever adds it), a unit-RMS norm over a token's whole
query projection and whole key projection with a weight per entry (``whole_norm_eps``), values of another size than
queries and keys (``v_dim``), and a mask of chunks (``chunk``: a query sees the earlier keys of its own run of ``chunk``
positions, runs counted from the sequence's start; no key is ever out of every later query's sight, so the cache
keeps all pages).  Heads whose sizes differ or are no multiple of 8 are stored padded with zeros to one size ``D``:
scores and outputs are unchanged, and the norm's mean divides by the true count.

Single new tokens go through the split-KV decode kernels, portions of prompts through the tensor-core
kernel (bfloat16, heads of 64, with or without a window) or the row kernel; all read keys and values straight from the pages (no gather copy, unlike
edgerag/cache/paged.py:208-238).
"""

from __future__ import annotations

import torch

from ..cache.manager import KVGroupSpec
from ..ops import kernels
from .base import LayerCall, Mixer, PartSpec, WeightSpec, build_part, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, n_q_heads: int, n_kv_heads: int, head_dim: int, position: PartSpec,
                 dtype: torch.dtype, device: torch.device, window: int = 0, own_kv: bool = True,
                 scale: float | None = None, keep_first: int = 0, qk_bias: bool = False, qk_norm_eps: float | None = None,
                 values_are_keys: bool = False, names: dict[str, str] | None = None, chunk: int = 0, v_dim: int | None = None,
                 all_bias: bool = False, whole_norm_eps: float | None = None) -> None:
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} query heads are not divisible by {n_kv_heads} kv heads")
        self.chunk = int(chunk or 0)
        self.all_bias, self.whole_norm_eps = bool(all_bias), whole_norm_eps
        self.has_update_bias = self.all_bias
        #: true sizes of a query/key head and of a value head; ``head_dim`` below is the size they are stored in
        self.qk_dim = head_dim
        self.v_dim = head_dim if v_dim is None else int(v_dim)
        widest = max(self.qk_dim, self.v_dim)
        padded = -(-widest // 8) * 8 if widest <= 128 else -(-widest // 16) * 16
        #: the second family's kernel handles padded heads, a norm over the projection and the four biases
        self.whole = self.all_bias or whole_norm_eps is not None or padded != self.qk_dim or self.v_dim != self.qk_dim
        if self.whole and (qk_bias or qk_norm_eps is not None or values_are_keys):
            raise ValueError("attention: the two families of options exclude each other")
        if self.chunk < 0 or (self.chunk and window):
            raise ValueError("attention: a mask of chunks takes a positive size and excludes a window")
        head_dim = padded if self.whole else head_dim
        self.hidden, self.n_q, self.n_kv, self.head_dim = hidden, n_q_heads, n_kv_heads, head_dim
        self.window = int(window or 0)
        self.keep_first = int(keep_first or 0) if self.window > 0 else 0
        self.qk_bias, self.qk_norm_eps, self.values_are_keys = bool(qk_bias), qk_norm_eps, bool(values_are_keys)
        if (self.qk_bias or self.qk_norm_eps is not None or self.values_are_keys) and not own_kv:
            raise ValueError("biases, head norms and shared values need the layer's own keys")
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                      "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias",
                      "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", **(names or {})}
        self.q_bias = self.k_bias = self.v_bias = self.q_norm = self.k_norm = None
        self.own_kv = own_kv
        self.scale = float(head_dim ** -0.5 if scale is None else scale)
        self.dtype, self.device = dtype, device
        self.position = build_part("position", position, dtype, device)
        self.q_width = n_q_heads * head_dim
        self.kv_width = n_kv_heads * head_dim
        self.in_width = self.q_width + (1 if self.values_are_keys else 2) * self.kv_width
        if self.whole and not own_kv:
            self.in_width = self.q_width         # queries only: keys and values are another layer's
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def cache_spec(self) -> KVGroupSpec:
        return KVGroupSpec(1, self.n_kv, self.head_dim, self.window, keep_first=self.keep_first)

    def weight_specs(self) -> list[WeightSpec]:
        nm = self.names
        if self.whole:
            return self._whole_specs()
        specs = [WeightSpec(nm["q"], (self.q_width, self.hidden))]
        if self.own_kv:
            specs.append(WeightSpec(nm["k"], (self.kv_width, self.hidden)))
            if not self.values_are_keys:
                specs.append(WeightSpec(nm["v"], (self.kv_width, self.hidden)))
        if self.qk_bias:
            specs += [WeightSpec(nm["q_bias"], (self.q_width,), "vector32"), WeightSpec(nm["k_bias"], (self.kv_width,), "vector32")]
        if self.qk_norm_eps is not None:
            specs += [WeightSpec(nm["q_norm"], (self.head_dim,), "vector32"), WeightSpec(nm["k_norm"], (self.head_dim,), "vector32")]
        return specs + [WeightSpec(nm["o"], (self.hidden, self.q_width))]

    def _whole_specs(self) -> list[WeightSpec]:
        """The tensors of the second family of options, in their true (unpadded) sizes."""
        nm = self.names
        q_true, k_true, v_true = self.n_q * self.qk_dim, self.n_kv * self.qk_dim, self.n_kv * self.v_dim
        specs = [WeightSpec(nm["q"], (q_true, self.hidden))]
        if self.all_bias:
            specs.append(WeightSpec(nm["q_bias"], (q_true,), "vector32"))
        if self.whole_norm_eps is not None:
            specs.append(WeightSpec(nm["q_norm"], (q_true,), "vector32"))
        if self.own_kv:
            specs += [WeightSpec(nm["k"], (k_true, self.hidden)), WeightSpec(nm["v"], (v_true, self.hidden))]
            if self.all_bias:
                specs += [WeightSpec(nm["k_bias"], (k_true,), "vector32"), WeightSpec(nm["v_bias"], (v_true,), "vector32")]
            if self.whole_norm_eps is not None:
                specs.append(WeightSpec(nm["k_norm"], (k_true,), "vector32"))
        specs.append(WeightSpec(nm["o"], (self.hidden, self.n_q * self.v_dim)))
        if self.all_bias:
            specs.append(WeightSpec(nm["o_bias"], (self.hidden,), "vector32"))
        return specs

    def _pad_heads(self, t: torch.Tensor, heads: int, true: int, dtype: torch.dtype) -> torch.Tensor:
        """Rows (or entries) ``[heads * true, ...]`` re-laid as ``[heads * head_dim, ...]``, zeros in the padding."""
        t = t.to(device=self.device, dtype=dtype)
        if true == self.head_dim:
            return t.contiguous()
        out = torch.zeros((heads, self.head_dim) + tuple(t.shape[1:]), dtype=dtype, device=self.device)
        out[:, :true] = t.reshape((heads, true) + tuple(t.shape[1:]))
        return out.reshape((heads * self.head_dim,) + tuple(t.shape[1:])).contiguous()

    def _load_whole(self, tensors: dict[str, torch.Tensor]) -> None:
        nm, f32 = self.names, torch.float32
        parts = [self._pad_heads(tensors[nm["q"]], self.n_q, self.qk_dim, self.dtype)]
        if self.own_kv:
            parts += [self._pad_heads(tensors[nm["k"]], self.n_kv, self.qk_dim, self.dtype),
                      self._pad_heads(tensors[nm["v"]], self.n_kv, self.v_dim, self.dtype)]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        w_o = tensors[nm["o"]].to(device=self.device, dtype=self.dtype)            # [hidden, heads * v_dim]: pad the columns
        self.w_o = self._pad_heads(w_o.t(), self.n_q, self.v_dim, self.dtype).t().contiguous()
        if self.all_bias:
            self.q_bias = self._pad_heads(tensors[nm["q_bias"]], self.n_q, self.qk_dim, f32)
            self.update_bias = tensors[nm["o_bias"]].to(device=self.device, dtype=f32).contiguous()
            if self.own_kv:
                self.k_bias = self._pad_heads(tensors[nm["k_bias"]], self.n_kv, self.qk_dim, f32)
                self.v_bias = self._pad_heads(tensors[nm["v_bias"]], self.n_kv, self.v_dim, f32)
        if self.whole_norm_eps is not None:
            self.q_norm = self._pad_heads(tensors[nm["q_norm"]], self.n_q, self.qk_dim, f32)
            if self.own_kv:
                self.k_norm = self._pad_heads(tensors[nm["k_norm"]], self.n_kv, self.qk_dim, f32)

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        nm = self.names
        if self.whole:
            return self._load_whole(tensors)
        f32 = lambda t: t.to(device=self.device, dtype=torch.float32).contiguous()   # noqa: E731
        if self.own_kv:
            parts = [tensors[nm["q"]], tensors[nm["k"]]] + ([] if self.values_are_keys else [tensors[nm["v"]]])
        else:  # rows for k and v stay zero: the layer reads another layer's cache
            pad = torch.zeros((2 * self.kv_width, self.hidden), dtype=self.dtype, device=self.device)
            parts = [tensors[nm["q"]], pad]
        self.w_qkv = torch.cat([p.to(device=self.device, dtype=self.dtype) for p in parts], dim=0).contiguous()
        self.w_o = tensors[nm["o"]].to(device=self.device, dtype=self.dtype).contiguous()
        if self.qk_bias:
            self.q_bias, self.k_bias = f32(tensors[nm["q_bias"]]), f32(tensors[nm["k_bias"]])
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = f32(tensors[nm["q_norm"]]), f32(tensors[nm["k_norm"]])

    def _prepare(self, x, qkv, ctx, pages, slots) -> None:
        """The input product and everything between it and the attention: biases, head norms, positions, cache write."""
        d = self.head_dim
        if self.whole:
            pos = self.position
            if getattr(pos, "pairs", False):
                raise ValueError("attention: with these options positions turn the halves of a head's first entries")
            kernels.linear(x, self.w_qkv, qkv)
            kernels.qkv_whole_norm(qkv, ctx.positions, self.n_q, self.n_kv, d, q_count=self.n_q * self.qk_dim,
                                   k_count=self.n_kv * self.qk_dim, eps=self.whole_norm_eps or 0.0, q_bias=self.q_bias,
                                   k_bias=self.k_bias, v_bias=self.v_bias, q_norm=self.q_norm, k_norm=self.k_norm,
                                   inv_freq=getattr(pos, "inv_freq", None), rot_dim=getattr(pos, "rot_dim", 0),
                                   has_kv=self.own_kv, slots=slots, k_pages=None if pages is None else pages[0],
                                   v_pages=None if pages is None else pages[1], page_size=ctx.page_size)
            return
        if self.qk_bias or self.qk_norm_eps is not None or self.values_are_keys:
            pos = self.position
            kernels.linear(x, self.w_qkv, qkv)
            kernels.qk_prepare(qkv, ctx.positions, self.n_q, self.n_kv, d, q_bias=self.q_bias, k_bias=self.k_bias,
                               q_norm=self.q_norm, k_norm=self.k_norm, eps=self.qk_norm_eps or 0.0,
                               inv_freq=getattr(pos, "inv_freq", None), rot_dim=getattr(pos, "rot_dim", 0),
                               pairs=bool(getattr(pos, "pairs", False)), values_are_keys=self.values_are_keys, slots=slots,
                               k_pages=None if pages is None else pages[0], v_pages=None if pages is None else pages[1],
                               page_size=ctx.page_size)
            return
        if not self.position.project_apply_store(x, self.w_qkv, qkv, ctx, self.n_q, self.n_kv, d, pages, slots):
            kernels.linear(x, self.w_qkv, qkv)
            self.position.apply_and_store(qkv, ctx, self.n_q, self.n_kv, d, pages, slots)

    def forward(self, x: torch.Tensor, ctx, call: LayerCall) -> torch.Tensor:
        n = x.shape[0]
        d = self.head_dim
        qkv = ctx.buf("attn.qkv", (n, self.in_width), self.dtype)
        k_pages, v_pages = ctx.pages_of(call.cache_layer)
        group = ctx.group_of(call.cache_layer)
        write = call.writes_cache and self.own_kv
        pages, slots = ((k_pages, v_pages), ctx.slots[group]) if write else (None, None)
        self._prepare(x, qkv, ctx, pages, slots)
        out = ctx.buf("attn.out", (n, self.q_width), self.dtype)
        tables = ctx.block_tables[group]
        nd = ctx.n_decode
        reach_mask = self.window or self.chunk                  # keys a token can see under its mask (0: all before it)
        mask = kernels.mask_reach(self.window, self.chunk)      # the mask as the kernels take it
        if nd:
            # Under a window a token reads few keys, and the grouped-heads kernel takes all kv heads it can into one block:
            # with few (sequence, kv head) pairs the bulk-copy kernel's finer plan wins (8 sequences of 4 kv heads: a decode
            # step of 0.362 ms against 0.384 ms; 64 sequences of 8: 48 us against 40 us for the kernel alone).
            may_group = reach_mask <= 0 or nd * self.n_kv >= 64
            grouped = may_group and self.n_q != self.n_kv and kernels.decode_gqa_supported(
                self.dtype, d, self.window, self.n_q, self.n_kv, ctx.page_size, kernels.DECODE_SPLIT_KEYS)
            if ctx.batch_invariant:     # one plan for every batch: a sequence's sums are then added in one order
                split, heads_per_block = kernels.DECODE_SPLIT_KEYS, 0
            elif reach_mask > 0:        # a token reads its window (or chunk) and the kept keys, however long its context is
                reach = min(ctx.max_keys_bound(), -(-(reach_mask + self.keep_first) // ctx.page_size) * ctx.page_size)
                split, heads_per_block = kernels.choose_decode_plan(nd, self.n_kv, reach, ctx.page_size, d,
                                                                    grouped or self.dtype != torch.bfloat16, reach)
            else:
                split, heads_per_block = kernels.choose_decode_plan(nd, self.n_kv, ctx.max_keys_bound(), ctx.page_size, d,
                                                                    grouped or self.dtype != torch.bfloat16, ctx.keys_granule())
            max_splits = ctx.decode_splits(mask, split)
            need_acc, need_ml = kernels.decode_scratch_floats(nd, self.n_q, d, max_splits)
            part_acc = ctx.buf("attn.part_acc", (need_acc,), torch.float32)
            part_ml = ctx.buf("attn.part_ml", (need_ml,), torch.float32)
            if may_group and kernels.decode_gqa_supported(self.dtype, d, self.window, self.n_q, self.n_kv, ctx.page_size, split, max_splits):
                kernels.attention_decode_gqa(qkv[:nd], k_pages, v_pages, tables, ctx.token_of_seq[:nd], ctx.positions,
                                             out[:nd], self.n_q, self.scale, part_acc, part_ml, max_splits, ctx.status,
                                             split_keys=split, window=self.window, keep_first=self.keep_first, chunk=self.chunk)
            elif kernels.decode_bulk_supported(self.dtype, d, self.window, self.n_q, self.n_kv, max_splits):
                kernels.attention_decode_bulk(qkv[:nd], k_pages, v_pages, tables, ctx.token_of_seq[:nd], ctx.positions,
                                              out[:nd], self.n_q, self.scale, part_acc, part_ml, max_splits, ctx.status,
                                              split_keys=split, head_group=heads_per_block, window=self.window,
                                              keep_first=self.keep_first, chunk=self.chunk)
            else:
                kernels.attention_decode(qkv[:nd], k_pages, v_pages, tables, ctx.token_of_seq[:nd], ctx.positions,
                                         out[:nd], self.n_q, self.scale, part_acc, part_ml, max_splits,
                                         window=self.window, split_keys=split, keep_first=self.keep_first, chunk=self.chunk)
        if n > nd and kernels.prefill_tc_supported(self.dtype, d, self.window, ctx.page_size):
            blocks = kernels.prefill_tc_blocks(ctx.host_q_len[nd:])
            # a portion that is short against its past: its few blocks' keys are cut into ranges
            reach = ctx.max_keys_bound()
            if reach_mask > 0:          # what a block of rows can see: its rows' windows (or chunks) and the kept first keys
                reach = min(reach, reach_mask + kernels.PREFILL_TC_ROWS + self.keep_first)
            ranges = kernels.prefill_tc_key_splits(blocks, self.n_q, reach, qkv.device)
            part_o = part_ml = None
            if ranges > 1:
                need_o, need_ml = kernels.prefill_tc_scratch_floats(n, self.n_q, ranges)
                part_o = ctx.buf("attn.range_o", (need_o,), torch.float32)
                part_ml = ctx.buf("attn.range_ml", (need_ml,), torch.float32)
            kernels.attention_prefill_tc(qkv, k_pages, v_pages, tables[nd:], ctx.seq_starts[nd:], ctx.positions, out, blocks,
                                         self.n_q, self.scale, ctx.status, key_splits=ranges, first_row=nd, part_o=part_o,
                                         part_ml=part_ml, window=self.window, keep_first=self.keep_first, chunk=self.chunk)
        elif n > nd:
            kernels.attention_rows(qkv[nd:], k_pages, v_pages, tables, ctx.seq_of_token[nd:], ctx.positions[nd:],
                                   out[nd:], self.n_q, self.scale, window=self.window, keep_first=self.keep_first, chunk=self.chunk)
        return self._project_out(out, ctx)

    def _project_out(self, out: torch.Tensor, ctx) -> torch.Tensor:
        n = out.shape[0]
        n_parts = kernels.linear_parts_count(out, self.w_o)
        if n_parts:      # the rows of a larger decode step: k split over the SMs, the norm after adds the parts
            y = ctx.buf("mixer.out_parts", (n_parts, n, self.hidden), torch.float32)
            kernels.linear_parts(out, self.w_o, y)
            return y
        y = ctx.buf("mixer.out", (n, self.hidden), self.dtype)
        kernels.linear(out, self.w_o, y)
        return y
