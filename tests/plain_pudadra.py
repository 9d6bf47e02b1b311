"""A plain, slow Pudadra in float64 on the CPU: one function per mechanism, written from the design's equations.

It shares no code with the package: it reads the same config.json keys and tensor names and computes every token of
a sequence at once with dense masks.  Notation: ``x`` rows are tokens, ``W`` is stored ``[out, in]`` and applied as
``x @ W.T``; positions count from 0.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm_w(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the weight is stored around zero."""
    return rms_unit(x, eps) * (1.0 + w)


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start.  ``u``: [T, C], ``w``: [C, taps]."""
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j: j + u.shape[0]] * w[:, j]
    return y


def rot_frequencies(base: float, dims: int, scaling: dict | None = None) -> torch.Tensor:
    """f_i = base^(-2i/dims); with ``scaling`` the long wavelengths are slowed down (factor, low, high, original)."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f.tolist():
            wavelength = 2.0 * math.pi / fi
            if wavelength < orig / high:
                out.append(fi)
            elif wavelength > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=F64)
    return f


def rotate_halves(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """Entry i is paired with entry i + dims/2 among the first ``dims = 2 len(freq)`` of the last axis; x: [T, ..., D]."""
    half = freq.numel()
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    a = (pos.to(F64)[:, None] * freq[None, :]).reshape(shape)
    u, v = x[..., :half], x[..., half: 2 * half]
    return torch.cat([u * a.cos() - v * a.sin(), v * a.cos() + u * a.sin(), x[..., 2 * half:]], -1)


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """Entry 2i is paired with entry 2i + 1 among the first ``2 len(freq)`` of the last axis."""
    half = freq.numel()
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    a = (pos.to(F64)[:, None] * freq[None, :]).reshape(shape)
    out = x.clone()
    u, v = x[..., 0: 2 * half: 2], x[..., 1: 2 * half: 2]
    out[..., 0: 2 * half: 2] = u * a.cos() - v * a.sin()
    out[..., 1: 2 * half: 2] = v * a.cos() + u * a.sin()
    return out


def window_mask(n: int, size: int) -> torch.Tensor:
    """[query, key] True where 0 <= i - j < size (``size`` 0 or None: plain causal)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if size:
        seen = seen & (i - j < size)
    return seen


def softmax_masked(scores: torch.Tensor, seen: torch.Tensor) -> torch.Tensor:
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), -1)


def diff_lambda(w: dict, pre: str, diff: float) -> float:
    return float(torch.exp((w[pre + "lq1"].to(F64) * w[pre + "lk1"].to(F64)).sum())
                 - torch.exp((w[pre + "lq2"].to(F64) * w[pre + "lk2"].to(F64)).sum()) + diff)


def diff_attention_mixer(h: torch.Tensor, w: dict, pre: str, m: dict, eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values, the second taken off the first times lambda."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w[pre + n].to(F64).T for n in ("q", "k", "v"))
    if m.get("conv"):
        q, k, v = (causal_conv(t, w[pre + n + ".conv"].to(F64)) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    pos = torch.arange(T)
    q = q.view(T, H, 2, d)
    k = k.view(T, G, 2, d)
    v = v.view(T, G, dv)
    rot = m.get("rot")
    if rot:
        freq = rot_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q, k = rotate_halves(q, pos, freq), rotate_halves(k, pos, freq)
    seen = window_mask(T, (m.get("mask") or {}).get("size", 0))
    lam = diff_lambda(w, pre, m["diff"])
    cap = float(m.get("softcap") or 0.0)
    heads = []
    for hq in range(H):
        g = hq // (H // G)
        maps = []
        for s in range(2):
            score = (q[:, hq, s] @ k[:, g, s].T) * m["scale"]
            if cap > 0:
                score = cap * torch.tanh(score / cap)
            maps.append(softmax_masked(score, seen) @ v[:, g])
        o = maps[0] - lam * maps[1]
        heads.append(rms_unit(o, eps) * (1.0 - m["diff"]))
    return torch.cat(heads, -1) @ w[pre + "o"].to(F64).T


def latent_attention_mixer(h: torch.Tensor, w: dict, pre: str, m: dict, eps: float) -> torch.Tensor:
    """Keys and values of every head made from one normed latent per token, plus one rotated key part for all heads."""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    freq = rot_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    q = (h @ w[pre + "q"].to(F64).T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, freq)
    down = h @ w[pre + "dkv"].to(F64).T
    c = rms_unit(down[:, :r], eps) * w[pre + "dkv.norm"].to(F64)
    k_rot = rotate_pairs(down[:, r:], pos, freq)
    k_plain = (c @ w[pre + "uk"].to(F64).T).view(T, H, d)
    v = (c @ w[pre + "uv"].to(F64).T).view(T, H, dv)
    seen = window_mask(T, (m.get("mask") or {}).get("size", 0))
    heads = []
    for hq in range(H):
        score = (q_plain[:, hq] @ k_plain[:, hq].T + q_rot[:, hq] @ k_rot.T) * m["scale"]
        heads.append(softmax_masked(score, seen) @ v[:, hq])
    return torch.cat(heads, -1) @ w[pre + "o"].to(F64).T


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def dense_ff(h: torch.Tensor, w: dict, pre: str) -> torch.Tensor:
    return gelu_erf(h @ w[pre + "up"].to(F64).T) @ w[pre + "down"].to(F64).T


def expert_ff(h: torch.Tensor, w: dict, pre: str) -> torch.Tensor:
    return relu_squared(h @ w[pre + "up"].to(F64).T) @ w[pre + "down"].to(F64).T


def routed_choice(h: torch.Tensor, w_router: torch.Tensor, router: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """(chosen experts [T, top], their weights [T, top]): softmax scores, the best groups only, scores not renormalised."""
    s = torch.softmax(h @ w_router.to(F64).T, -1)
    T, E = s.shape
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = router.get("groups")
    if groups:
        count, keep = groups["count"], groups["keep"]
        best = s.view(T, count, E // count).max(-1).values
        kept = best.topk(keep, -1).indices
        ok = torch.zeros(T, count, dtype=torch.bool)
        ok.scatter_(1, kept, True)
        allowed = ok[:, :, None].expand(T, count, E // count).reshape(T, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(router["top"], -1).indices
    return chosen, s.gather(1, chosen)


def moe_ff(h: torch.Tensor, w: dict, pre: str, mlp: dict, chosen: torch.Tensor | None = None) -> torch.Tensor:
    """``chosen`` [T, top]: experts handed in (their weights are still this router's scores), else the router's own."""
    if chosen is None:
        chosen, weight = routed_choice(h, w[pre + "router"], mlp["router"])
    else:
        weight = torch.softmax(h @ w[pre + "router"].to(F64).T, -1).gather(1, chosen.long())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), weight[t].tolist()):
            out[t] += s * expert_ff(h[t: t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[pre + "shared.sg"].to(F64).T)             # [T, 1]
        out = out + gate * expert_ff(h, w, pre + "shared.")
    return out


def forward(w: dict, cfg: dict, tokens: list[int], layers_out: list | None = None, chosen: dict | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` receives the stream after every layer; ``chosen``: layer -> the
    experts [T, top] to use there instead of the router's choice."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"].to(F64)[torch.tensor(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = layer_norm_w(x, w[pre + "norm1"].to(F64), eps)
        mixer = diff_attention_mixer if layer["type"] == "attention" else latent_attention_mixer
        x = x + mult * mixer(h, w, pre + "mix.", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = layer_norm_w(x, w[pre + "norm2"].to(F64), eps)
            if mlp["kind"] == "dense":
                ff = dense_ff(h, w, pre + "mlp.")
            else:
                ff = moe_ff(h, w, pre + "mlp.", mlp, None if chosen is None else chosen.get(i))
            x = x + mult * ff
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm_w(x, w["final.norm"].to(F64), eps)
    return (x @ w["embed"].to(F64).T) * cfg["logit_scale"]


def greedy(w: dict, cfg: dict, prompt: list[int], n_new: int) -> list[int]:
    seq, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(forward(w, cfg, seq)[-1].argmax()))
        seq.append(out[-1])
    return out


# --- configurations and random weights for the tests --------------------------------------------------------------

def attention_layer(heads=2, kv_heads=1, dim=16, vdim=24, conv=3, diff=0.4, window=12, rot_dims=8, scale=None, softcap=15.0,
                    base=1000.0, scaling=None, mlp=None) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale or dim ** -0.5,
             "softcap": softcap, "rot": {"base": base, "dims": rot_dims}}
    if conv:
        mixer["conv"] = conv
    if window:
        mixer["mask"] = {"size": window}
    if scaling:
        mixer["rot"]["scaling"] = scaling
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent_layer(heads=3, dim=8, rot_dim=8, vdim=16, kv_rank=24, window=10, scale=None, base=500.0, mlp=None) -> dict:
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def dense_mlp(ff=48) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_mlp(ff=16, experts=6, top=2, groups=(3, 2), shared=24) -> dict:
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def make_config(layers: list[dict], width=32, vocab=97, eps=1e-5, residual_mult=0.5, logit_scale=1.5) -> dict:
    return {"architecture": "Pudadra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": residual_mult,
            "logit_scale": logit_scale, "layers": layers}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    W = cfg["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            rows = {"q": H * 2 * d, "k": G * 2 * d, "v": G * dv}
            for n, r in rows.items():
                shapes[p + "mix." + n] = (r, W)
                if m.get("conv"):
                    shapes[p + f"mix.{n}.conv"] = (r, m["conv"])
            for n in ("lq1", "lk1", "lq2", "lk2"):
                shapes[p + "mix." + n] = (d,)
            shapes[p + "mix.o"] = (W, H * dv)
        else:
            H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * (d + dr), W), p + "mix.dkv": (r + dr, W), p + "mix.dkv.norm": (r,),
                           p + "mix.uk": (H * d, r), p + "mix.uv": (H * dv, r), p + "mix.o": (W, H * dv)})
        mlp = layer.get("mlp")
        if not mlp:
            continue
        shapes[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                shapes.update({p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                shapes.update({p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf), p + "mlp.shared.sg": (1, W)})
    return shapes


def random_weights(cfg: dict, seed: int = 0, dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    """Weights of a size that keeps every sublayer's update comparable with the stream."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name == "embed":
            t = torch.randn(shape, generator=gen)
        elif leaf in ("norm1", "norm2", "norm") and not name.endswith("dkv.norm"):
            t = 0.1 * torch.randn(shape, generator=gen)
        elif name.endswith("dkv.norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        elif leaf == "conv":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * torch.randn(shape, generator=gen)
        elif leaf == "router":
            t = 2.0 * torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        else:
            t = 1.5 * torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out
