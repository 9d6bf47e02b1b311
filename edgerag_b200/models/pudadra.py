"""Pudadra: a decoder whose layers are listed one by one in config.json, each a pre-norm block whose two updates are
multiplied by one constant of the model, around one of two mixers and a dense or routed feed-forward.

config.json keys read: ``architecture``, ``width``, ``vocab``, ``norm.eps``, ``residual_mult``, ``logit_scale`` and
``layers``: per layer ``type`` (``attention`` | ``latent_attention``), ``mixer`` (the mixer's sizes) and ``mlp`` (or null).

* ``attention``: ``heads, kv_heads, dim, vdim, scale, diff``, optional ``softcap``, ``conv`` (taps of a causal
  convolution on q, k and v), ``mask.size`` (a window) and ``rot.{base, dims, scaling.{factor, low, high, original}}``:
  differential attention (``parts/diff_attention.py``).
* ``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale, rot.{base, dims}``, optional ``mask.size``:
  attention through a normed latent with one rotated key part for all heads, no gate (``parts/latent_attention.py``).
* ``mlp.kind = dense``: ``ff``; ``down(gelu(up x))`` with the exact gelu.
* ``mlp.kind = moe``: ``expert.ff``, ``router.{experts, top, groups.{count, keep}}``, optional ``shared.ff``: experts
  ``down(relu(up x)^2)``, softmax scores over all experts, the ``top`` best of the ``keep`` best groups, the scores
  themselves as weights of the experts' outputs, plus a shared expert of the same form times ``sigmoid(sg . x)``.

Every norm multiplies by ``1 + w`` (weights stored around zero) in float32; the head is the embedding table, and the
logits are multiplied by ``logit_scale``.  Tensor names: ``embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{q, k, v, q.conv, k.conv, v.conv, lq1, lk1, lq2, lk2, o}`` or ``l<i>.mix.{q, dkv, dkv.norm, uk, uv, o}``,
``l<i>.mlp.{up, down}`` or ``l<i>.mlp.{router, e<j>.up, e<j>.down, shared.up, shared.down, shared.sg}``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..config.model_config import ConfigError
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec

LAYER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _need(d: Any, key: str, where: str) -> Any:
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"{where}: no '{key}'")
    return d[key]


def _window(m: dict[str, Any], at: str) -> int:
    mask = m.get("mask")
    if mask is None:
        return 0
    size = int(_need(mask, "size", at + ".mixer.mask"))
    if size <= 0:
        raise ConfigError(f"{at}: mask.size must be positive")
    return size


@dataclass
class PudadraConfig:
    hidden_size: int
    vocab_size: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    layers: list[dict[str, Any]] = field(default_factory=list)
    architectures: list[str] = field(default_factory=lambda: ["Pudadra"])

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict[str, Any], where: str = "config") -> "PudadraConfig":
        layers = _need(raw, "layers", where)
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        out = []
        for i, layer in enumerate(layers):
            at = f"{where}: layers[{i}]"
            kind = _need(layer, "type", at)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: {LAYER_TYPES}")
            m = dict(_need(layer, "mixer", at))
            m["window"] = _window(m, at)
            rot = m.get("rot")
            if kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim", "scale", "diff"):
                    _need(m, key, at + ".mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{at}: kv_heads must divide heads")
                if rot is not None:
                    for key in ("base", "dims"):
                        _need(rot, key, at + ".mixer.rot")
                    if rot["dims"] % 2 or rot["dims"] > m["dim"]:
                        raise ConfigError(f"{at}: rot.dims must be even and at most dim")
                    scaling = rot.get("scaling")
                    if scaling is not None:
                        for key in ("factor", "low", "high", "original"):
                            _need(scaling, key, at + ".mixer.rot.scaling")
                        if not (float(scaling["factor"]) > 0 and float(scaling["high"]) > float(scaling["low"])):
                            raise ConfigError(f"{at}: rot.scaling needs factor > 0 and high > low")
                if int(m.get("conv") or 0) < 0:
                    raise ConfigError(f"{at}: conv must not be negative")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                    _need(m, key, at + ".mixer")
                rot = _need(m, "rot", at + ".mixer")
                for key in ("base", "dims"):
                    _need(rot, key, at + ".mixer.rot")
                if rot["dims"] % 2 or rot["dims"] > m["rot_dim"] or m["rot_dim"] % 2 or m["kv_rank"] % 2:
                    raise ConfigError(f"{at}: kv_rank, rot_dim and rot.dims must be even, rot.dims at most rot_dim")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                mkind = mlp.get("kind", "dense")
                if mkind not in MLP_KINDS:
                    raise ConfigError(f"{at}: mlp.kind {mkind!r} is not supported; known: {MLP_KINDS}")
                mlp["kind"] = mkind
                if mkind == "dense":
                    _need(mlp, "ff", at + ".mlp")
                else:
                    _need(_need(mlp, "expert", at + ".mlp"), "ff", at + ".mlp.expert")
                    router = _need(mlp, "router", at + ".mlp")
                    experts, top = int(_need(router, "experts", at + ".mlp.router")), int(_need(router, "top", at + ".mlp.router"))
                    if not 0 < top <= experts:
                        raise ConfigError(f"{at}: router.top must lie in 1..experts")
                    groups = router.get("groups")
                    if groups is not None:
                        count, keep = int(_need(groups, "count", at + ".mlp.router.groups")), int(_need(groups, "keep", at + ".mlp.router.groups"))
                        if count < 1 or experts % count or not 1 <= keep <= count or top > keep * (experts // count):
                            raise ConfigError(f"{at}: router.groups must split the experts evenly and leave at least 'top' to choose from")
                    if mlp.get("shared") is not None:
                        _need(mlp["shared"], "ff", at + ".mlp.shared")
            out.append({"type": kind, "mixer": m, "mlp": mlp})
        return cls(hidden_size=int(_need(raw, "width", where)), vocab_size=int(_need(raw, "vocab", where)),
                   norm_eps=float(_need(_need(raw, "norm", where), "eps", where + ": norm")),
                   residual_mult=float(raw.get("residual_mult", 1.0) if raw.get("residual_mult") is not None else 1.0),
                   logit_scale=float(raw.get("logit_scale", 1.0) if raw.get("logit_scale") is not None else 1.0), layers=out)


def pudadra_plan(cfg: PudadraConfig) -> ModelPlan:
    h, eps = cfg.hidden_size, cfg.norm_eps
    norm = lambda tensor, prefix="": PartSpec(      # noqa: E731
        "rmsnorm", {"size": h, "eps": eps, "weight_offset": 1.0, "exact": True, "tensor": tensor}, prefix)
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        if layer["type"] == "attention":
            rot = m.get("rot") or {}
            mixer = PartSpec("diff_attention", {
                "hidden": h, "n_q_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"], "v_dim": m["vdim"],
                "scale": m["scale"], "diff": m["diff"], "eps": eps, "window": m["window"], "softcap": float(m.get("softcap") or 0.0),
                "conv": int(m.get("conv") or 0), "rot_base": float(rot.get("base", 10000.0)), "rot_dims": int(rot.get("dims", 0)),
                "rot_scaling": rot.get("scaling")}, "mix.")
        else:
            mixer = PartSpec("latent_attention", {
                "hidden": h, "n_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "v_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "scale": m["scale"], "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"],
                "rot_scaling": m["rot"].get("scaling"), "eps": eps, "gated": False, "window": m["window"]}, "mix.")
        mlp = layer["mlp"]
        if mlp is None:
            ffn = None
        elif mlp["kind"] == "dense":
            ffn = PartSpec("dense_act", {"hidden": h, "intermediate": mlp["ff"], "act": "gelu_erf"}, "mlp.")
        else:
            router = mlp["router"]
            groups = router.get("groups")
            shared = mlp.get("shared")
            ffn = PartSpec("routed_experts", {
                "hidden": h, "intermediate": mlp["expert"]["ff"], "n_experts": router["experts"], "top": router["top"],
                "scores": "softmax", "groups": (groups["count"], groups["keep"]) if groups else None, "gated": False,
                "act": "relu_squared", "scale_input": False,
                "shared": None if shared is None else PartSpec("dense_act", {
                    "hidden": h, "intermediate": shared["ff"], "act": "relu_squared", "scalar_gate": "sg"}, "shared.")}, "mlp.")
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("prenorm", {"update_scale": cfg.residual_mult}), norm1=norm("norm1"),
                                mixer=mixer, norm2=None if mlp is None else norm("norm2"), ffn=ffn))
        schedule.append(LayerCall(i, i))
    return ModelPlan(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "hidden": h, "tensor": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("norm", "final."),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "tensor": "head", "tied_to": "embed",
                                 "scale": cfg.logit_scale}),
        name_prefixes=("",),
        # (a layer without a feed-forward has no use for a second norm: a file that stores one all the same still loads)
        ignored_prefixes=tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer["mlp"] is None),
    )
