"""Lozanex: a decoder whose layers are listed one by one in config.json; every sublayer reads the residual stream
itself and an RMS norm closes what it adds: ``x += norm1(mixer(x)); x += norm2(ff(x))``.  The embedding's rows pass
an RMS norm of their own before the first layer.

config.json keys read: ``architecture``, ``width``, ``vocab``, ``norm.eps`` and ``layers``: per layer ``type``
(``attention`` | ``delta``), ``mixer`` (the mixer's sizes) and ``mlp`` (``{kind: moe, expert.ff, router.{experts, top},
shared.ff}`` or null).

* ``attention``: ``heads, kv_heads, dim, vdim, scale, rot.{base, dims}, mask.size``, optional ``kv_from: j``:
  grouped-query attention with biases on all four projections, a unit-RMS norm over a token's whole query projection
  and whole key projection (a weight per entry), the halves of the first ``rot.dims`` entries of every head turned,
  and a mask of chunks of ``mask.size`` positions.  A layer with ``kv_from`` has no key and value tensors and reads
  the cache of layer ``j``.
* ``delta``: ``heads, kv_heads, dim, vdim, conv``: the gated delta rule (``parts/delta.py``).
* ``moe``: routed experts chosen by sigmoid scores, the score multiplying the expert's input, plus a shared expert.

Tensor names: ``embed``, ``embed.norm``, ``head``, ``final.norm``, ``l<i>.{norm1, norm2}``, ``l<i>.mix.*``,
``l<i>.mlp.{router, e<j>.{gate, up, down}, shared.{gate, up, down}}``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..config.model_config import ConfigError
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec

LAYER_TYPES = ("attention", "delta")


def _need(d: Any, key: str, where: str) -> Any:
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"{where}: no '{key}'")
    return d[key]


@dataclass
class LozanexConfig:
    hidden_size: int
    vocab_size: int
    norm_eps: float
    layers: list[dict[str, Any]] = field(default_factory=list)
    architectures: list[str] = field(default_factory=lambda: ["Lozanex"])

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config") -> "LozanexConfig":
        layers = _need(raw, "layers", where)
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            at = f"{where}: layers[{i}]"
            kind = _need(layer, "type", at)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: {LAYER_TYPES}")
            m = _need(layer, "mixer", at)
            for key in ("heads", "kv_heads", "dim"):
                if int(_need(m, key, at + ".mixer")) <= 0:
                    raise ConfigError(f"{at}: mixer.{key} must be positive")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{at}: kv_heads must divide heads")
            if int(m.get("vdim") or m["dim"]) <= 0:
                raise ConfigError(f"{at}: mixer.vdim must be positive")
            if kind == "attention":
                _need(m, "scale", at + ".mixer")
                rot = m.get("rot")
                if rot is not None:
                    dims = int(_need(rot, "dims", at + ".mixer.rot"))
                    if dims % 2 or not 0 <= dims <= m["dim"]:
                        raise ConfigError(f"{at}: rot.dims must be even and at most dim")
                    if dims and not float(_need(rot, "base", at + ".mixer.rot")) > 0:
                        raise ConfigError(f"{at}: rot.base must be positive")
                mask = m.get("mask")
                if mask is not None and int(_need(mask, "size", at + ".mixer.mask")) <= 0:
                    raise ConfigError(f"{at}: mask.size must be positive")
                src = m.get("kv_from")
                if src is not None:
                    if not (isinstance(src, int) and 0 <= src < i) or layers[src].get("type") != "attention" \
                            or layers[src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{at}: kv_from must name an earlier attention layer with keys of its own")
                    theirs = layers[src]["mixer"]
                    same = ("kv_heads", "dim", "vdim", "rot")
                    if any(theirs.get(k) != m.get(k) for k in same):
                        raise ConfigError(f"{at}: kv_from layer {src} has other key/value heads or another rotation")
            else:
                if int(_need(m, "conv", at + ".mixer")) < 1:
                    raise ConfigError(f"{at}: mixer.conv must be at least 1")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"{at}: mlp.kind {mlp.get('kind')!r} is not supported (moe only)")
                _need(_need(mlp, "expert", at + ".mlp"), "ff", at + ".mlp.expert")
                router = _need(mlp, "router", at + ".mlp")
                experts, top = int(_need(router, "experts", at + ".mlp.router")), int(_need(router, "top", at + ".mlp.router"))
                if not 0 < top <= experts:
                    raise ConfigError(f"{at}: router.top must lie between 1 and router.experts")
                if mlp.get("shared") is not None:
                    _need(mlp["shared"], "ff", at + ".mlp.shared")
            out.append({"type": kind, "mixer": dict(m), "mlp": dict(mlp) if mlp is not None else None})
        return cls(hidden_size=int(_need(raw, "width", where)), vocab_size=int(_need(raw, "vocab", where)),
                   norm_eps=float(_need(_need(raw, "norm", where), "eps", where + ": norm")), layers=out)


def lozanex_plan(cfg: LozanexConfig) -> ModelPlan:
    h, eps = cfg.hidden_size, cfg.norm_eps
    norm = lambda tensor, prefix="": PartSpec("rmsnorm", {"size": h, "eps": eps, "exact": True, "tensor": tensor}, prefix)   # noqa: E731
    reads_stream = PartSpec("pass", {"size": h})
    layers, schedule = [], []
    cache_layer_of: dict[int, int] = {}
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        vdim = int(m.get("vdim") or m["dim"])
        if layer["type"] == "attention":
            rot = m.get("rot") or {}
            dims = int(rot.get("dims") or 0)
            position = PartSpec("rope_halves", {"head_dim": m["dim"], "theta": rot["base"], "rot_dim": dims, "precise": True}) \
                if dims else PartSpec("none")
            mixer = PartSpec("attention", {
                "hidden": h, "n_q_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": vdim,
                "scale": m["scale"], "chunk": int((m.get("mask") or {}).get("size") or 0), "all_bias": True,
                "whole_norm_eps": eps, "own_kv": m.get("kv_from") is None, "position": position,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                          "o_bias": "o.b", "q_norm": "q.norm", "k_norm": "k.norm"}}, "mix.")
        else:
            mixer = PartSpec("gated_delta", {"hidden": h, "n_heads": m["heads"], "n_key_heads": m["kv_heads"],
                                             "key_dim": m["dim"], "v_dim": vdim, "conv": m["conv"], "eps": eps}, "mix.")
        mlp = layer["mlp"]
        ffn = None
        if mlp is not None:
            shared = mlp.get("shared")
            ffn = PartSpec("routed_experts", {
                "hidden": h, "intermediate": mlp["expert"]["ff"], "n_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "shared": None if shared is None else PartSpec("glu_bounded", {"hidden": h, "intermediate": shared["ff"]}, "shared."),
            }, "mlp.")
        block = PartSpec("sandwich", {"post1": norm("norm1"), "post2": None if mlp is None else norm("norm2")})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, norm1=reads_stream, mixer=mixer,
                                norm2=None if mlp is None else reads_stream, ffn=ffn))
        src = m.get("kv_from") if layer["type"] == "attention" else None
        if src is None:
            cache_layer_of[i] = len(cache_layer_of)
            schedule.append(LayerCall(i, cache_layer_of[i]))
        else:
            schedule.append(LayerCall(i, cache_layer_of[src], writes_cache=False))
    return ModelPlan(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "hidden": h, "tensor": "embed", "norm": norm("embed.norm")}),
        layers=layers, schedule=schedule, final_norm=norm("norm", "final."),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "tensor": "head"}),
        name_prefixes=("",),
    )
