"""A plain, slow implementation of the Lozanex decoder in float64, one function per mechanism.

It shares no code with the package: it works on whole sequences with ordinary torch arithmetic on the CPU
and exists to be compared against.  ``config`` is the dictionary of a config.json, ``tensors`` maps the
checkpoint's names to tensors.

The design, in this file's notation.  The stream ``x`` starts as ``rms(embed[token]) * w_embed_norm``.  A layer
reads the stream itself and norms what it adds: ``x += rms(mixer(x)) * w1`` and, where the layer has a
feed-forward, ``x += rms(ff(x)) * w2``.  The logits are ``head (rms(x) * w_final)``.

* mixer ``attention``: grouped-query attention with biased projections, a unit-RMS norm over the whole query
  (and key) projection of a token with a weight per entry, a rotation of pairs ``(i, i + r/2)`` of the first ``r``
  entries of every head by ``position * base**(-2i/r)``, scores times a given scale, and a mask of chunks: query
  ``i`` sees key ``j <= i`` when both lie in the same run of ``size`` positions counted from the sequence's start.
  A layer may read the keys and values of an earlier layer instead of making its own.
* mixer ``delta``: the gated delta rule.  Queries, keys and values pass a short causal convolution per channel
  and silu; queries and keys become unit vectors per head; per head a matrix ``S`` decays by ``g``, is corrected
  towards the value along the key with strength ``beta``, and is read with the query; the read-out is normed
  per head and gated.
* feed-forward ``moe``: a router's sigmoid scores choose ``top`` experts per token; a chosen expert sees the
  token's input times its score; a shared expert sees every token.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(F64)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """``x``: [tokens, heads, dim].  Entry ``i < dims/2`` of a head pairs with entry ``i + dims/2``."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    angle = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]      # [tokens, half]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def chunk_mask(n_q: int, n_k: int, first_q: int, size: int) -> torch.Tensor:
    """[n_q, n_k] of booleans: query at position ``first_q + a`` sees key at position ``b``."""
    i = torch.arange(first_q, first_q + n_q)[:, None]
    j = torch.arange(n_k)[None, :]
    seen = j <= i
    if size:
        seen &= (i // size) == (j // size)
    return seen


def attention_keys_values(h: torch.Tensor, m: dict, t: dict, pre: str, eps: float):
    """What an attention layer keeps of its input rows: keys after norm and rotation, and values."""
    n = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ t[pre + "k"].to(F64).T + t[pre + "k.b"].to(F64)
    v = h @ t[pre + "v"].to(F64).T + t[pre + "v.b"].to(F64)
    k = rms_norm(k, t[pre + "k.norm"], eps).view(n, G, d)
    rot = m.get("rot") or {}
    k = rotate_halves(k, torch.arange(n), float(rot.get("base", 1.0)), int(rot.get("dims", 0)))
    return k, v.view(n, G, dv)


def attention_mixer(h: torch.Tensor, m: dict, t: dict, pre: str, eps: float, kv) -> torch.Tensor:
    """``kv``: the (keys, values) to attend over (this layer's own or another layer's)."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ t[pre + "q"].to(F64).T + t[pre + "q.b"].to(F64)
    q = rms_norm(q, t[pre + "q.norm"], eps).view(n, H, d)
    rot = m.get("rot") or {}
    q = rotate_halves(q, torch.arange(n), float(rot.get("base", 1.0)), int(rot.get("dims", 0)))
    k, v = kv
    seen = chunk_mask(n, n, 0, int((m.get("mask") or {}).get("size", 0)))
    out = torch.zeros(n, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].T) * float(m["scale"])
        score = score.masked_fill(~seen, -math.inf)
        out[:, head] = torch.softmax(score, dim=-1) @ v[:, g]
    return out.reshape(n, H * dv) @ t[pre + "o"].to(F64).T + t[pre + "o.b"].to(F64)


def causal_conv_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x``: [tokens, channels]; ``w``: [channels, taps], the last column weighs the current token; zeros before the start."""
    n, taps = x.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F64), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y += padded[j: j + n] * w.to(F64)[:, j][None, :]
    return silu(y)


def unit_vectors(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k: [tokens, heads, dim]; v: [tokens, heads, vdim]; beta, g: [tokens, heads].  Token by token."""
    n, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(n, H, dv, dtype=F64)
    for t in range(n):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def delta_mixer(h: torch.Tensor, m: dict, t: dict, pre: str, eps: float) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ t[pre + "q"].to(F64).T, t[pre + "q.conv"]).view(n, G, d)
    k = causal_conv_silu(h @ t[pre + "k"].to(F64).T, t[pre + "k.conv"]).view(n, G, d)
    v = causal_conv_silu(h @ t[pre + "v"].to(F64).T, t[pre + "v.conv"]).view(n, H, dv)
    q = unit_vectors(q) * d ** -0.5
    k = unit_vectors(k)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ t[pre + "b"].to(F64).T)
    g = torch.exp(-torch.exp(t[pre + "A_log"].to(F64)) * softplus(h @ t[pre + "a"].to(F64).T + t[pre + "dt_bias"].to(F64)))
    o = delta_rule(q, k, v, beta, g)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * t[pre + "norm"].to(F64)
    o = o * silu(h @ t[pre + "g"].to(F64).T).view(n, H, dv)
    return o.reshape(n, H * dv) @ t[pre + "o"].to(F64).T


def expert(h: torch.Tensor, t: dict, pre: str) -> torch.Tensor:
    return (silu(h @ t[pre + "gate"].to(F64).T) * (h @ t[pre + "up"].to(F64).T)) @ t[pre + "down"].to(F64).T


def routed_choice(h: torch.Tensor, t: dict, pre: str, top: int):
    """(indices [tokens, top], scores [tokens, top]) of the experts with the largest sigmoid scores."""
    s = torch.sigmoid(h @ t[pre + "router"].to(F64).T)
    w, idx = torch.topk(s, top, dim=-1)
    return idx, w


def moe(h: torch.Tensor, mlp: dict, t: dict, pre: str, chosen: torch.Tensor | None = None) -> torch.Tensor:
    """``chosen`` [tokens, top]: experts to use instead of the router's own choice (their scores stay the router's)."""
    idx, w = routed_choice(h, t, pre, int(mlp["router"]["top"]))
    if chosen is not None:
        idx = chosen.long()
        w = torch.gather(torch.sigmoid(h @ t[pre + "router"].to(F64).T), 1, idx)
    out = torch.zeros(h.shape[0], t[pre + "e0.down"].shape[0], dtype=F64)
    for e in range(int(mlp["router"]["experts"])):
        for slot in range(idx.shape[1]):
            rows = (idx[:, slot] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += expert(h[rows] * w[rows, slot][:, None], t, f"{pre}e{e}.")
    if mlp.get("shared") is not None:
        out += expert(h, t, pre + "shared.")
    return out


def router_margins(config: dict, tensors: dict, tokens) -> torch.Tensor:
    """Per layer with a feed-forward and token: the gap between the last chosen and the first not chosen router logit."""
    gaps: list[torch.Tensor] = []
    forward(config, tensors, tokens, _gaps=gaps)
    return torch.stack(gaps) if gaps else torch.zeros(0, len(tokens), dtype=F64)


def forward(config: dict, tensors: dict, tokens, return_layers: bool = False, chosen: dict | None = None, _gaps=None):
    """Logits [tokens, vocab] of one whole sequence (float64); with ``return_layers`` also the stream after every layer.
    ``chosen``: layer -> [tokens, top] experts that the layer's feed-forward is to use whatever its router says."""
    eps = float(config["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = rms_norm(tensors["embed"].to(F64)[ids], tensors["embed.norm"], eps)
    kept: dict[int, tuple] = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}.mix."
        m = layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(x, m, tensors, pre, eps)
            y = attention_mixer(x, m, tensors, pre, eps, kept[i if src is None else src])
        elif layer["type"] == "delta":
            y = delta_mixer(x, m, tensors, pre, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, tensors[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            if _gaps is not None:
                z = torch.sort(x @ tensors[f"l{i}.mlp.router"].to(F64).T, dim=-1, descending=True).values
                top = int(layer["mlp"]["router"]["top"])
                _gaps.append(z[:, top - 1] - z[:, top] if top < z.shape[1] else torch.full_like(z[:, 0], math.inf))
            x = x + rms_norm(moe(x, layer["mlp"], tensors, f"l{i}.mlp.", None if chosen is None else chosen.get(i)),
                             tensors[f"l{i}.norm2"], eps)
        after.append(x.clone())
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].to(F64).T
    return (logits, torch.stack(after)) if return_layers else logits


# --- small configurations and random weights for tests ------------------------------------------------

def attention_layer(heads=4, kv_heads=2, dim=32, vdim=None, rot_dims=16, base=10000.0, size=24, scale=0.25, kv_from=None,
                    experts=4, top=2, ff=48, shared_ff=40) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim, "scale": scale}
    if rot_dims is not None:
        mixer["rot"] = {"base": base, "dims": rot_dims}
    if size is not None:
        mixer["mask"] = {"size": size}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": moe_mlp(experts, top, ff, shared_ff)}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=4, experts=4, top=2, ff=48, shared_ff=40) -> dict:
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": moe_mlp(experts, top, ff, shared_ff)}


def moe_mlp(experts, top, ff, shared_ff):
    if experts is None:
        return None
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff is not None:
        mlp["shared"] = {"ff": shared_ff}
    return mlp


def make_config(layers: list[dict], width=64, vocab=160, eps=1e-5) -> dict:
    import copy
    return {"architecture": "Lozanex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    w, shapes = config["width"], {}
    shapes["embed"] = (config["vocab"], w)
    shapes["embed.norm"] = (w,)
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
        shapes[f"l{i}.norm1"] = (w,)
        if layer["type"] == "attention":
            shapes.update({pre + "q": (H * d, w), pre + "q.b": (H * d,), pre + "q.norm": (H * d,),
                           pre + "o": (w, H * dv), pre + "o.b": (w,)})
            if m.get("kv_from") is None:
                shapes.update({pre + "k": (G * d, w), pre + "k.b": (G * d,), pre + "k.norm": (G * d,),
                               pre + "v": (G * dv, w), pre + "v.b": (G * dv,)})
        else:
            taps = m["conv"]
            shapes.update({pre + "q": (G * d, w), pre + "q.conv": (G * d, taps), pre + "k": (G * d, w), pre + "k.conv": (G * d, taps),
                           pre + "v": (H * dv, w), pre + "v.conv": (H * dv, taps), pre + "b": (H, w), pre + "a": (H, w),
                           pre + "A_log": (H,), pre + "dt_bias": (H,), pre + "norm": (dv,), pre + "g": (H * dv, w),
                           pre + "o": (w, H * dv)})
        mlp = layer.get("mlp")
        if mlp is not None:
            shapes[f"l{i}.norm2"] = (w,)
            f = f"l{i}.mlp."
            shapes[f + "router"] = (mlp["router"]["experts"], w)
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{f}e{e}.gate": (mlp["expert"]["ff"], w), f"{f}e{e}.up": (mlp["expert"]["ff"], w),
                               f"{f}e{e}.down": (w, mlp["expert"]["ff"])})
            if mlp.get("shared") is not None:
                shapes.update({f + "shared.gate": (mlp["shared"]["ff"], w), f + "shared.up": (mlp["shared"]["ff"], w),
                               f + "shared.down": (w, mlp["shared"]["ff"])})
    shapes["final.norm"] = (w,)
    shapes["head"] = (config["vocab"], w)
    return shapes


def random_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Seeded weights, rounded to bfloat16 (so that both number formats of the engine see the same values)."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(".conv"):
            t = torch.randn(shape, generator=gen) * 0.6
        elif last == "A_log":
            t = torch.log(0.3 + 2.0 * torch.rand(shape, generator=gen))      # decays neither all near 1 nor all near 0
        elif last == "dt_bias":
            t = torch.randn(shape, generator=gen) - 1.0
        elif last == "router":
            t = torch.randn(shape, generator=gen) * 3.0 / math.sqrt(shape[1])
        elif len(shape) == 2:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
            if ".mix." in name and last in ("q", "k"):
                t = t * 2.0                                   # sharper scores: a wrong key shows
            if last == "embed":
                t = t * math.sqrt(shape[1])
        elif last == "b":
            t = 0.2 * torch.randn(shape, generator=gen)
        else:                                                 # norm weights
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        out[name] = t.to(torch.bfloat16)
    return out
