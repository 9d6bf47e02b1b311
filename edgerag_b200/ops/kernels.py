"""Python entry points of the CUDA kernels: tensors in, one launch on the current stream each.

Every function checks what a wrong call would turn into a wrong result (device, dtype, layout,
sizes), then calls the ``extern "C"`` function of the library built for the tensors' element type.
Nothing here falls back to PyTorch arithmetic: a missing library or a refused shape raises.
"""

from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import native


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_ELEM = {torch.float32: "float32", torch.bfloat16: "bfloat16"}

_SIGNATURES = {
    "erb_embed_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                       c_void_p, c_float, c_void_p],
    "erb_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int,
                        c_float, c_void_p],
    "erb_residual_add": [c_void_p, c_void_p, c_longlong, c_float, c_void_p],
    "erb_act_rows": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "erb_scale_rows": [c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "erb_rope_cache_write": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_swiglu": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_resolve_ids": [c_void_p, c_int, c_void_p, c_int, c_void_p],
    "erb_gather_cast": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_linear": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_void_p, c_longlong, c_void_p],
    "erb_linear_skinny": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_skinny_glu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_skinny_glu_bounded": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                      c_float, c_int, c_void_p],
    "erb_linear_skinny_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "erb_linear_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_tune": [c_int],
    "erb_linear_trials": [],
    "erb_linear_tc_parts": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_tc_parts_count": [c_int, c_int],
    "erb_residual_add_parts": [c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_float, c_void_p],
    "erb_add_rmsnorm_parts": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                              c_int, c_int, c_float, c_void_p],
    "erb_linear_tc_glu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_linear_tc_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "erb_attention_rows": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "erb_attention_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                             c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_float, c_void_p],
    "erb_attention_prefill_tc": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                 c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_attention_decode_bulk": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                  c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "erb_attention_decode_gqa": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_glu_bounded": [c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p],
    "erb_add_layernorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_float,
                          c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "erb_cast_rows": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "erb_stream_set": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_qk_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_softcap": [c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "erb_linear_batched": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_longlong, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p],
    "erb_latent_store": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int,
                         c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "erb_latent_q_rotate": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
                            c_void_p],
    "erb_latent_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                             c_int, c_void_p],
    "erb_latent_attention_mma": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_float, c_int, c_void_p],
    "erb_latent_combine": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_diff_part_floats": [c_int],
    "erb_diff_prepare": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "erb_diff_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_float,
                           c_void_p],
    "erb_diff_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                               c_float, c_float, c_float, c_void_p],
    "erb_conv_silu": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p],
    "erb_conv_state_update": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "erb_ssm_scan": [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_gated_group_norm": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_float, c_void_p],
    "erb_rms_between": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p,
                        c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "erb_bias_rows": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "erb_qkv_whole_norm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                           c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                           c_void_p],
    "erb_delta_scan": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "erb_head_norm_gate": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "erb_moe_route": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "erb_moe_tc_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "erb_moe_tc_gate_up": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                           c_void_p, c_void_p],
    "erb_moe_tc_down": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                        c_void_p, c_void_p, c_void_p],
    "erb_moe_tc_up_act": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                          c_void_p, c_void_p],
    "erb_moe_product": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                        c_int, c_int, c_void_p, c_void_p, c_void_p],
    "erb_sample_rows": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
}

_functions: dict[tuple[str, str | None, str], object] = {}

#: launches issued through this module: this package's own kernels, and library products
launch_counts = {"own": 0, "library": 0}
_LAUNCHES = {"erb_diff_part_floats": 0, "erb_moe_route": 2, "erb_delta_scan": 2, "erb_linear_batched": 0, "erb_attention_decode": 2, "erb_attention_prefill_tc": 1, "erb_attention_decode_bulk": 1, "erb_attention_decode_gqa": 1, "erb_linear": 0}
SKINNY_MAX_ROWS = 16     # rows up to which the register-fed weight-streaming kernels are used
TC_MAX_ROWS = 64         # rows up to which the TMA + tcgen05 weight-streaming kernel may be used


def launches() -> int:
    """Kernels launched through this module so far (this package's own and the library's)."""
    return launch_counts["own"] + launch_counts["library"]


def _fn(library: str, elem: str | None, name: str):
    key = (library, elem, name)
    fn = _functions.get(key)
    if fn is None:
        lib = native.load(library, elem)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[name]
        fn.restype = c_int
        fn._erb_lib = lib
        fn._erb_own = _LAUNCHES.get(name, 1)
        _functions[key] = fn
    return fn


def _call(fn, *args) -> None:
    rc = fn(*args)
    if fn._erb_own:
        launch_counts["own"] += fn._erb_own
    else:
        launch_counts["library"] += 1
    if rc != 0:
        raise KernelError(fn._erb_lib.erb_last_error().decode())


def _elem(t: torch.Tensor) -> str:
    try:
        return _ELEM[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The raw handle of the current CUDA stream (the capturing stream inside a graph capture)."""
    # (the C calls directly: torch.cuda.current_device() costs a microsecond of Python per launch)
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need(t: torch.Tensor | None, name: str, dtype=None, contiguous: bool = True) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


# --- rows ------------------------------------------------------------------------------------

def embed_rows(hidden: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor,
               embeds: torch.Tensor | None = None, embed_row: torch.Tensor | None = None, scale: float = 1.0) -> None:
    """hidden[t] = scale * table[ids[t]], or scale * embeds[embed_row[t]] where embed_row[t] >= 0 (float output)."""
    n, h = hidden.shape
    _need(hidden, "hidden", torch.float32); _need(table, "table"); _need(ids, "ids", torch.int32)
    _need(status, "status", torch.int32); _need(embed_row, "embed_row", torch.int32)
    if table.shape[1] != h or ids.numel() < n:
        raise KernelError("embed_rows: shapes disagree")
    if embeds is not None:
        _need(embeds, "embeds", table.dtype)
        if embeds.shape[1] != h or embed_row is None:
            raise KernelError("embed_rows: embeds need embed_row and the hidden width")
    _call(_fn("elementwise", _elem(table), "erb_embed_rows"), hidden.data_ptr(), table.data_ptr(),
          _ptr(embeds), ids.data_ptr(), _ptr(embed_row), n, h, table.shape[0],
          0 if embeds is None else embeds.shape[0], status.data_ptr(), float(scale), _stream())


def add_rmsnorm(hidden: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
                delta: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                write_back: bool = True, settled: bool = False, exact: bool = False, delta_scale: float = 1.0) -> None:
    """out = weight * round(rmsnorm(hidden (+ delta_scale * delta))); hidden += delta_scale * delta in place when write_back.
    ``exact``: the normed value stays float until the weight has multiplied it (one rounding, at the store).
    ``delta``: rows of the element type, or float32 partial sums ``[parts, rows, width]`` (what
    ``linear_parts`` leaves) that are added in their order and rounded to the element type once, so that
    the update is what a product stored in the element type would have been.
    ``settled``: ``hidden`` was last written two or more launches ago (the launch just before this one
    wrote ``delta`` at most), so the kernel may read it while that launch is still running."""
    _need(hidden, "hidden", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    _need(rows, "rows", torch.int32)
    h = hidden.shape[1]
    n = out.shape[0]
    in_parts = delta is not None and delta.dim() == 3
    _need(delta, "delta", torch.float32 if in_parts else out.dtype)
    if out.shape[1] != h or weight.numel() != h or (delta is not None and delta.shape[-2:] != hidden.shape):
        raise KernelError("add_rmsnorm: shapes disagree")
    if rows is None and n != hidden.shape[0]:
        raise KernelError("add_rmsnorm: out rows differ from hidden rows")
    if rows is not None and rows.numel() < n:
        raise KernelError("add_rmsnorm: fewer row indices than output rows")
    if in_parts:
        _call(_fn("elementwise", _elem(out), "erb_add_rmsnorm_parts"), hidden.data_ptr(), delta.data_ptr(), delta.shape[0],
              delta.stride(0), weight.data_ptr(), out.data_ptr(), _ptr(rows), n, h, float(eps),
              int(write_back and rows is None), int(bool(settled)) | (2 if exact else 0), float(delta_scale), _stream())
        return
    _call(_fn("elementwise", _elem(out), "erb_add_rmsnorm"), hidden.data_ptr(), _ptr(delta), weight.data_ptr(),
          out.data_ptr(), _ptr(rows), n, h, float(eps), int(write_back and rows is None),
          int(bool(settled)) | (2 if exact else 0), float(delta_scale), _stream())


def residual_add(hidden: torch.Tensor, delta: torch.Tensor, dtype: torch.dtype | None = None, scale: float = 1.0) -> None:
    """hidden += scale * delta: rows of the model's element type, or float32 partial sums ``[parts, rows, width]``,
    which are added up and rounded to ``dtype`` (the model's element type) once, as ``add_rmsnorm`` does."""
    _need(hidden, "hidden", torch.float32); _need(delta, "delta")
    if delta.dim() == 3:
        _need(delta, "delta", torch.float32)
        if delta.shape[1:] != hidden.shape or dtype is None:
            raise KernelError("residual_add: partial sums need [parts, rows, width] and the element type to round to")
        _call(_fn("elementwise", _ELEM[dtype], "erb_residual_add_parts"), hidden.data_ptr(), delta.data_ptr(), delta.shape[0],
              delta.stride(0), hidden.numel(), float(scale), _stream())
        return
    if hidden.shape != delta.shape:
        raise KernelError("residual_add: shapes disagree")
    _call(_fn("elementwise", _elem(delta), "erb_residual_add"), hidden.data_ptr(), delta.data_ptr(),
          hidden.numel(), float(scale), _stream())


def add_layernorm(hidden: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None, out: torch.Tensor | None,
                  eps: float, delta: torch.Tensor | None = None, post: tuple[torch.Tensor, torch.Tensor, float] | None = None,
                  rows: torch.Tensor | None = None, write_back: bool = True) -> None:
    """The residual add between two layer norms (weight and bias, statistics in float): with ``post = (w, b, eps)``
    the update is normed first, ``d = LN(delta; w, b)`` kept in float; ``hidden += d`` in place when ``write_back``;
    ``out = LN(hidden (+ d); weight, bias)`` rounded once, or the plain cast of the sum where ``weight`` is None, or
    nothing where ``out`` is None.  ``delta``: rows of the element type or float32 partial sums ``[parts, rows,
    width]`` (added in order, rounded to the element type once).  ``out`` may be a view with unit inner stride."""
    _need(hidden, "hidden", torch.float32); _need(weight, "weight", torch.float32); _need(bias, "bias", torch.float32)
    _need(out, "out", contiguous=False); _need(rows, "rows", torch.int32)
    h = hidden.shape[1]
    in_parts = delta is not None and delta.dim() == 3
    elem = out.dtype if out is not None else (delta.dtype if delta is not None and not in_parts else None)
    if elem is None:
        raise KernelError("add_layernorm: neither an output nor rows of an update name the element type")
    _need(delta, "delta", torch.float32 if in_parts else elem)
    if delta is not None and delta.shape[-2:] != hidden.shape:
        raise KernelError("add_layernorm: delta and hidden disagree")
    if (weight is None) != (bias is None) or (weight is not None and (weight.numel() != h or bias.numel() != h)):
        raise KernelError("add_layernorm: weight and bias come together and have the row's width")
    pw = pb = None
    peps = 0.0
    if post is not None:
        pw, pb, peps = post
        _need(pw, "post weight", torch.float32); _need(pb, "post bias", torch.float32)
        if delta is None or pw.numel() != h or pb.numel() != h:
            raise KernelError("add_layernorm: a norm of the update needs the update and vectors of the row's width")
    if out is not None:
        n = out.shape[0]
        if out.shape[1] != h or out.stride(1) != 1:
            raise KernelError("add_layernorm: out must be [rows, width] with unit inner stride")
        if rows is None and n != hidden.shape[0]:
            raise KernelError("add_layernorm: out rows differ from hidden rows")
        if rows is not None and rows.numel() < n:
            raise KernelError("add_layernorm: fewer row indices than output rows")
        out_ld = out.stride(0) if n > 1 else max(h, out.stride(0))
    else:
        n, out_ld = hidden.shape[0], h
        if rows is not None:
            raise KernelError("add_layernorm: a selection of rows needs an output")
    _call(_fn("elementwise", _ELEM[elem], "erb_add_layernorm"), hidden.data_ptr(), _ptr(delta), delta.shape[0] if in_parts else 0,
          delta.stride(0) if in_parts else 0, _ptr(pw), _ptr(pb), float(peps), _ptr(weight), _ptr(bias), float(eps), _ptr(out),
          int(out_ld), _ptr(rows), n, h, int(write_back and rows is None), _stream())


def rms_between(hidden: torch.Tensor, out: torch.Tensor | None, *, weight: torch.Tensor | None = None, eps: float = 0.0,
                delta: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                post: tuple[torch.Tensor, float] | None = None, own: tuple[torch.Tensor, float] | None = None,
                rows: torch.Tensor | None = None, write_back: bool = True, dtype: torch.dtype | None = None) -> None:
    """The residual add between RMS norms, everything in float with eps inside the root.  In order: with ``own = (w,
    eps)`` the stream's rows are normed in place; the update ``delta`` (rows of the element type, or float32 partial
    sums ``[parts, rows, width]`` added in order and rounded to the element type once) gets ``bias`` added and, with
    ``post = (w, eps)``, is normed (kept float); ``hidden +=`` the update, in place when ``write_back``; ``out`` (None:
    nothing) receives the row rounded once: normed with ``weight`` and ``eps``, or as it is where ``weight`` is None.
    ``rows`` picks the rows that ``out`` gets (then nothing is written back).  ``dtype`` names the element type where
    neither ``out`` nor ``delta`` does."""
    _need(hidden, "hidden", torch.float32); _need(weight, "weight", torch.float32); _need(bias, "bias", torch.float32)
    _need(out, "out", contiguous=False); _need(rows, "rows", torch.int32)
    h = hidden.shape[1]
    in_parts = delta is not None and delta.dim() == 3
    elem = out.dtype if out is not None else (delta.dtype if delta is not None and not in_parts else dtype)
    if elem is None:
        raise KernelError("rms_between: nothing names the element type")
    _need(delta, "delta", torch.float32 if in_parts else elem)
    if delta is not None and delta.shape[-2:] != hidden.shape:
        raise KernelError("rms_between: delta and hidden disagree")
    if (bias is not None or post is not None) and delta is None:
        raise KernelError("rms_between: a bias or a closing norm needs an update")
    for pair in (post, own):
        if pair is not None:
            _need(pair[0], "norm weight", torch.float32)
            if pair[0].numel() != h:
                raise KernelError("rms_between: a norm's weight must have the row's width")
    if (weight is not None and weight.numel() != h) or (bias is not None and bias.numel() != h):
        raise KernelError("rms_between: vectors must have the row's width")
    if out is not None:
        n = out.shape[0]
        if out.shape[1] != h or out.stride(1) != 1:
            raise KernelError("rms_between: out must be [rows, width] with unit inner stride")
        if rows is None and n != hidden.shape[0]:
            raise KernelError("rms_between: out rows differ from hidden rows")
        if rows is not None and rows.numel() < n:
            raise KernelError("rms_between: fewer row indices than output rows")
        out_ld = out.stride(0) if n > 1 else max(h, out.stride(0))
    else:
        n, out_ld = hidden.shape[0], h
        if rows is not None:
            raise KernelError("rms_between: a selection of rows needs an output")
    _call(_fn("elementwise", _ELEM[elem], "erb_rms_between"), hidden.data_ptr(), _ptr(delta), delta.shape[0] if in_parts else 0,
          delta.stride(0) if in_parts else 0, _ptr(bias), _ptr(own[0]) if own else None, float(own[1]) if own else 0.0,
          _ptr(post[0]) if post else None, float(post[1]) if post else 0.0, _ptr(weight), float(eps), _ptr(out), int(out_ld),
          _ptr(rows), n, h, int(write_back and rows is None), _stream())


def qkv_whole_norm(qkv: torch.Tensor, positions: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, *,
                   q_count: int, k_count: int, eps: float, q_bias: torch.Tensor | None = None, k_bias: torch.Tensor | None = None,
                   v_bias: torch.Tensor | None = None, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                   inv_freq: torch.Tensor | None = None, rot_dim: int = 0, has_kv: bool = True, slots: torch.Tensor | None = None,
                   k_pages: torch.Tensor | None = None, v_pages: torch.Tensor | None = None, page_size: int = 16) -> None:
    """Rows ``[q heads | k heads | v heads]`` (``head_dim`` entries a head; with ``has_kv`` False the queries only) made
    ready for attention where the norm of queries and keys runs over a token's whole projection: biases added, ``q *
    rsqrt(sum(q^2) / q_count + eps) * q_norm`` (all entries of the row at once; ``q_count`` is the true number of
    entries where heads are padded with zeros), k likewise, entries ``i`` and ``i + rot_dim / 2`` of the first
    ``rot_dim`` of every q and k head turned by ``position * inv_freq[i]``; q goes back in place, k and v (plus bias)
    to the tokens' cache slots.  All in float."""
    _need(qkv, "qkv", contiguous=False); _need(positions, "positions", torch.int32)
    for name, t in (("q_bias", q_bias), ("k_bias", k_bias), ("v_bias", v_bias), ("q_norm", q_norm), ("k_norm", k_norm),
                    ("inv_freq", inv_freq)):
        _need(t, name, torch.float32)
    _need(slots, "slots", torch.int32); _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
    n = qkv.shape[0]
    qw, kw = n_q_heads * head_dim, n_kv_heads * head_dim
    if qkv.stride(1) != 1 or qkv.shape[1] < qw + (2 * kw if has_kv else 0):
        raise KernelError("qkv_whole_norm: rows too narrow")
    for t, width in ((q_bias, qw), (q_norm, qw), (k_bias, kw), (k_norm, kw), (v_bias, kw)):
        if t is not None and t.numel() != width:
            raise KernelError("qkv_whole_norm: a bias or norm weight has the wrong size")
    if rot_dim and (inv_freq is None or inv_freq.numel() < rot_dim // 2):
        raise KernelError("qkv_whole_norm: too few frequencies")
    if k_pages is not None and (tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim) or v_pages is None
                                or v_pages.shape != k_pages.shape or slots is None or slots.numel() < n):
        raise KernelError("qkv_whole_norm: pages or slots disagree with the heads")
    _call(_fn("elementwise", _elem(qkv), "erb_qkv_whole_norm"), qkv.data_ptr(), qkv.stride(0) if n > 1 else qkv.shape[1],
          _ptr(q_bias), _ptr(k_bias), _ptr(v_bias), _ptr(q_norm), _ptr(k_norm), int(q_count), int(k_count), float(eps),
          positions.data_ptr(), _ptr(inv_freq), int(rot_dim), _ptr(slots), _ptr(k_pages), _ptr(v_pages), n, n_q_heads,
          n_kv_heads, head_dim, int(page_size), int(bool(has_kv)), _stream())


def cast_rows(src: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[t, :] = src[t, :] rounded to ``dst``'s element type; ``src`` float32 rows, ``dst`` a view with unit inner stride."""
    _need(src, "src", torch.float32); _need(dst, "dst", contiguous=False)
    n, width = src.shape
    if dst.shape != (n, width) or dst.stride(1) != 1:
        raise KernelError("cast_rows: shapes disagree")
    _call(_fn("elementwise", _elem(dst), "erb_cast_rows"), src.data_ptr(), dst.data_ptr(), n, width,
          dst.stride(0) if n > 1 else max(width, dst.stride(0)), _stream())


def stream_set(hidden: torch.Tensor, y: torch.Tensor, vec: torch.Tensor | None = None) -> None:
    """hidden[t, :] = float(y[t, :]) + vec: the residual stream set anew from a product's rows and one vector."""
    _need(hidden, "hidden", torch.float32); _need(y, "y"); _need(vec, "vec", torch.float32)
    if y.shape != hidden.shape or (vec is not None and vec.numel() != hidden.shape[1]):
        raise KernelError("stream_set: shapes disagree")
    _call(_fn("elementwise", _elem(y), "erb_stream_set"), hidden.data_ptr(), y.data_ptr(), _ptr(vec), hidden.shape[0],
          hidden.shape[1], _stream())


def qk_prepare(qkv: torch.Tensor, positions: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, *,
               q_bias: torch.Tensor | None = None, k_bias: torch.Tensor | None = None, q_norm: torch.Tensor | None = None,
               k_norm: torch.Tensor | None = None, eps: float = 0.0, inv_freq: torch.Tensor | None = None, rot_dim: int = 0,
               pairs: bool = False, values_are_keys: bool = False, slots: torch.Tensor | None = None,
               k_pages: torch.Tensor | None = None, v_pages: torch.Tensor | None = None, page_size: int = 0) -> None:
    """Queries and keys made ready for attention, per head of each row ``[q heads | k heads (| v heads)]`` of ``qkv``:
    bias added, (``values_are_keys``: the result is the token's cached value), unit RMS times a weight shared by the
    heads (``q_norm`` / ``k_norm``), the first ``rot_dim`` entries turned by ``position * inv_freq[i]`` (neighbouring
    pairs ``(2i, 2i + 1)`` with ``pairs``, else ``(i, i + rot_dim / 2)``).  q is rewritten in place; k (and v) go to
    the token's cache slot (``slots``: ``page * page_size + offset``, negative: nothing is written)."""
    _need(qkv, "qkv", contiguous=False); _need(positions, "positions", torch.int32)
    for name, t in (("q_bias", q_bias), ("k_bias", k_bias), ("q_norm", q_norm), ("k_norm", k_norm), ("inv_freq", inv_freq)):
        _need(t, name, torch.float32)
    _need(slots, "slots", torch.int32); _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
    n = qkv.shape[0]
    heads = n_q_heads + n_kv_heads * (1 if values_are_keys else 2)
    if qkv.stride(1) != 1 or qkv.shape[1] < heads * head_dim or positions.numel() < n:
        raise KernelError("qk_prepare: qkv width or positions disagree with the head counts")
    if (q_bias is not None and q_bias.numel() != n_q_heads * head_dim) or (k_bias is not None and k_bias.numel() != n_kv_heads * head_dim) \
            or (q_norm is not None and q_norm.numel() != head_dim) or (k_norm is not None and k_norm.numel() != head_dim):
        raise KernelError("qk_prepare: a bias or norm weight has the wrong size")
    if rot_dim and (inv_freq is None or inv_freq.numel() != rot_dim // 2):
        raise KernelError("qk_prepare: inv_freq must hold rot_dim / 2 values")
    if k_pages is not None:
        if v_pages is None or slots is None or slots.numel() < n or page_size <= 0:
            raise KernelError("qk_prepare: a cache write needs k_pages, v_pages, slots and the page size")
        if tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelError("qk_prepare: page layout is not [pages, kv heads, page_size, head_dim]")
    _call(_fn("elementwise", _elem(qkv), "erb_qk_prepare"), qkv.data_ptr(), qkv.stride(0) if n > 1 else qkv.shape[1], _ptr(q_bias),
          _ptr(k_bias), _ptr(q_norm), _ptr(k_norm), float(eps), positions.data_ptr(), _ptr(inv_freq), int(rot_dim), int(pairs),
          _ptr(slots), _ptr(k_pages), _ptr(v_pages), n, n_q_heads, n_kv_heads, head_dim, max(1, int(page_size)),
          int(values_are_keys), _stream())


def resolve_ids(ids: torch.Tensor, fed: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> None:
    """Replace every id t < 0 of ``ids`` (int32, in place) by ``fed[-t - 1]``: tokens of the step
    before that are still on the device.  ``dtype`` only picks the library that holds the kernel
    (the engine's element type, so that nothing else has to be built)."""
    _need(ids, "ids", torch.int32); _need(fed, "fed", torch.int32)
    _call(_fn("elementwise", _ELEM[dtype], "erb_resolve_ids"), ids.data_ptr(), ids.numel(),
          fed.data_ptr(), fed.numel(), _stream())


def gather_cast(src: torch.Tensor, dst: torch.Tensor, rows: torch.Tensor | None) -> None:
    _need(src, "src", torch.float32); _need(dst, "dst"); _need(rows, "rows", torch.int32)
    _call(_fn("elementwise", _elem(dst), "erb_gather_cast"), src.data_ptr(), dst.data_ptr(), _ptr(rows),
          dst.shape[0], dst.shape[1], _stream())


def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None,
                     n_q_heads: int, n_kv_heads: int, head_dim: int, rot_dim: int,
                     slots: torch.Tensor | None = None, k_pages: torch.Tensor | None = None,
                     v_pages: torch.Tensor | None = None, page_size: int = 0) -> None:
    """Rotate q (in place) and k by the halves convention; write rotated k and v to cache slots.

    ``k_pages``/``v_pages``: one layer's pages ``[n_pages, n_kv_heads, page_size, head_dim]``.
    ``slots``: int32 per token, ``page * page_size + offset`` or negative to write nothing.
    """
    _need(qkv, "qkv"); _need(positions, "positions", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    _need(slots, "slots", torch.int32); _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q_heads + 2 * n_kv_heads) * head_dim or positions.numel() < n:
        raise KernelError("rope_cache_write: qkv width or positions disagree with the head counts")
    write = k_pages is not None
    if write:
        if v_pages is None or slots is None or slots.numel() < n:
            raise KernelError("rope_cache_write: cache write needs k_pages, v_pages and slots")
        if tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelError("rope_cache_write: page layout is not [pages, kv heads, page_size, head_dim]")
    if rot_dim and (inv_freq is None or inv_freq.numel() != rot_dim // 2):
        raise KernelError("rope_cache_write: inv_freq must hold rot_dim / 2 values")
    _call(_fn("elementwise", _elem(qkv), "erb_rope_cache_write"), qkv.data_ptr(), positions.data_ptr(),
          _ptr(inv_freq), _ptr(slots), _ptr(k_pages), _ptr(v_pages), n, n_q_heads, n_kv_heads, head_dim,
          rot_dim, page_size, int(write), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter):
        raise KernelError("swiglu: gate_up must be [tokens, 2 * intermediate]")
    _call(_fn("elementwise", _elem(out), "erb_swiglu"), gate_up.data_ptr(), out.data_ptr(), n, inter, _stream())


GLU_ACTS = {"sigmoid": 0, "gelu_tanh": 1}


def glu_bounded(gate_up: torch.Tensor, out: torch.Tensor, limit: float = 0.0, alpha: float = 1.0, shift: float = 0.0,
                act: str = "sigmoid") -> None:
    """out[t, i] = g * sigmoid(alpha * g) * (u + shift) with g = min(gate_up[t, i], limit) and
    u = clamp(gate_up[t, I + i], -limit, limit); ``limit <= 0`` bounds nothing.  ``act="gelu_tanh"``:
    ``0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))`` in the place of ``g * sigmoid(alpha * g)``."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter):
        raise KernelError("glu_bounded: gate_up must be [tokens, 2 * intermediate]")
    _call(_fn("elementwise", _elem(out), "erb_glu_bounded"), gate_up.data_ptr(), out.data_ptr(), n, inter, float(limit),
          float(alpha), float(shift), GLU_ACTS[act], _stream())


def softcap(logits: torch.Tensor, cap: float, dtype: torch.dtype) -> None:
    """logits <- cap * tanh(logits / cap) in place (float rows with unit inner stride).  ``dtype`` only
    picks the library that holds the kernel (the engine's element type)."""
    _need(logits, "logits", torch.float32, contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("softcap: logits must be rows with unit inner stride")
    n, width = logits.shape
    _call(_fn("elementwise", _ELEM[dtype], "erb_softcap"), logits.data_ptr(), n, width, logits.stride(0) if n > 1 else width,
          float(cap), _stream())


ACTS = {"gelu_erf": 0, "relu_squared": 1}


def act_rows(x: torch.Tensor, out: torch.Tensor, act: str, gate_col: int = -1) -> None:
    """out[t, i] = f(x[t, i]) for the first ``out.shape[1]`` columns of the rows ``x`` (a row-strided view allowed), in float,
    rounded once: ``gelu_erf`` the exact gelu, ``relu_squared`` the square of relu.  ``gate_col >= 0``: every row is also
    multiplied by the sigmoid of its column ``gate_col`` of ``x`` (one logit per token that scales the whole branch)."""
    _need(x, "x", contiguous=False); _need(out, "out", x.dtype)
    n, width = out.shape
    if x.shape[0] != n or x.shape[1] < width or x.stride(1) != 1 or not -1 <= gate_col < x.shape[1]:
        raise KernelError("act_rows: shapes disagree")
    if act not in ACTS:
        raise KernelError(f"act_rows: unknown activation {act!r}; known: {sorted(ACTS)}")
    _call(_fn("elementwise", _elem(x), "erb_act_rows"), x.data_ptr(), x.stride(0) if n > 1 else x.shape[1], out.data_ptr(), n, width,
          ACTS[act], int(gate_col), _stream())


def scale_rows(x: torch.Tensor, scale: float, dtype: torch.dtype) -> None:
    """Float rows times a constant, in place (``x`` may be a view whose rows are further apart than their width)."""
    _need(x, "x", torch.float32, contiguous=False)
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("scale_rows: rows with unit inner stride")
    n, width = x.shape
    _call(_fn("elementwise", _ELEM[dtype], "erb_scale_rows"), x.data_ptr(), n, width, x.stride(0) if n > 1 else width, float(scale),
          _stream())


# --- matrix products -------------------------------------------------------------------------

_workspaces: dict[int, torch.Tensor] = {}
WORKSPACE_BYTES = 64 << 20


def _workspace(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        ws = torch.empty(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _workspaces[idx] = ws
    return ws


_set_status_word = None
_status_word: torch.Tensor | None = None     # where the tensor-core weight-streaming kernel reports
_status_word_told: int | None = None         # ... and what the library was last told


def linear_status_word(status: torch.Tensor | None) -> None:
    """Name the device word (int32) to which the TMA + tcgen05 weight-streaming kernel reports a wait
    that ran out (code 4000000 + block).  Kept until named again.  The library itself is told when it
    is next used (a model that never brings 17 to 64 rows to a large product never builds it)."""
    global _status_word
    if status is not None:
        _need(status, "status", torch.int32)
    _status_word = status


def _fn_tc(name: str):
    """A function of the tensor-core weight-streaming library, which first hears of the status word if it has changed."""
    global _set_status_word, _status_word_told
    fn = _fn("linear_tc", None, name)
    told = None if _status_word is None else _status_word.data_ptr()
    if told != _status_word_told:
        if _set_status_word is None:
            _set_status_word = fn._erb_lib.erb_linear_tc_set_status_word
            _set_status_word.argtypes = [c_void_p]
            _set_status_word.restype = c_int
        _set_status_word(told)
        _status_word_told = told
    return fn


def linear_few_rows_supported(a: torch.Tensor, weight: torch.Tensor, lda: int) -> bool:
    """Whether the weight-streaming kernel takes these operands (bfloat16, at most 64 rows, 16-byte rows)."""
    k = a.shape[1]
    return (a.dtype == torch.bfloat16 and a.shape[0] <= 64 and k % 8 == 0 and lda % 8 == 0
            and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear_few_rows(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``linear`` through the weight-streaming kernel, for up to 64 rows."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", contiguous=False)
    m, k = a.shape
    n = weight.shape[0]
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_few_rows: shapes or strides disagree")
    if out.dtype not in (torch.bfloat16, torch.float32) or not linear_few_rows_supported(a, weight, lda):
        raise KernelError("linear_few_rows: operands not supported")
    _call(_fn("gemm", "bfloat16", "erb_linear_skinny"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
          lda, k, ldo, int(out.dtype == torch.float32), _stream())


def linear_tc(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``linear`` for up to 64 bfloat16 rows through the TMA + tcgen05 weight-streaming kernel."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", contiguous=False)
    m, k = a.shape
    n = weight.shape[0]
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_tc: shapes or strides disagree")
    if out.dtype not in (torch.bfloat16, torch.float32) or not linear_few_rows_supported(a, weight, lda):
        raise KernelError("linear_tc: operands not supported")
    _call(_fn_tc("erb_linear_tc"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, lda, k, ldo,
          int(out.dtype == torch.float32), _stream())


#: weights below this size stay with the library at 17 to 64 rows (measured at 64 rows: 960 x 960, 1.8 MB, 4.2 us in
#: parts against 3.4 us; 960 x 2560, 4.9 MB, 4.3 against 5.9 us; 2048 x 2048, 8.4 MB, 4.5 against 5.8 us)
PARTS_MIN_WEIGHT_ELEMENTS = 2 << 20


def linear_parts_count(a: torch.Tensor, weight: torch.Tensor) -> int:
    """How many partial results ``linear_parts`` leaves for ``a @ weight^T``, or 0 where the product is
    not taken in parts: it is for the bfloat16 rows of a decode step beyond the register kernel's
    (``SKINNY_MAX_ROWS`` < rows <= ``TC_MAX_ROWS``) against a weight with so few rows that whole tiles of
    them would leave most SMs without work (the attention output and the down projection)."""
    m, k = a.shape
    n = weight.shape[0]
    if not (SKINNY_MAX_ROWS < m <= TC_MAX_ROWS) or a.dtype != torch.bfloat16 or n % 4 or a.stride(1) != 1:
        return 0
    if not linear_few_rows_supported(a, weight, a.stride(0)) or -(-n // 128) * 2 > _sms(a.device):
        return 0
    if n * k < PARTS_MIN_WEIGHT_ELEMENTS:
        return 0
    return _parts_count(n, k)


def linear_parts_slices(weight: torch.Tensor) -> int:
    """The number of slices of k, and so of partial results, that ``linear_parts`` makes for this weight (a
    function of its shape alone)."""
    return _parts_count(weight.shape[0], weight.shape[1])


@functools.lru_cache(maxsize=256)
def _parts_count(n: int, k: int) -> int:
    return int(_fn_tc("erb_linear_tc_parts_count")(n, k))


def linear_parts(a: torch.Tensor, weight: torch.Tensor, parts: torch.Tensor) -> None:
    """``parts[s] = a[:, slice s of k] @ weight[:, slice s of k]^T`` in float32 for the
    ``linear_parts_slices`` slices of k; their sum in order is the product (``add_rmsnorm`` and
    ``residual_add`` take them as they are).  Up to ``TC_MAX_ROWS`` bfloat16 rows, n a multiple of 4."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(parts, "parts", torch.float32)
    m, k = a.shape
    n = weight.shape[0]
    if (weight.shape[1] != k or a.stride(1) != 1 or m > TC_MAX_ROWS or n % 4 or not linear_few_rows_supported(a, weight, a.stride(0))
            or tuple(parts.shape) != (linear_parts_slices(weight), m, n)):
        raise KernelError("linear_parts: shapes disagree or the operands are not supported")
    _call(_fn_tc("erb_linear_tc_parts"), a.data_ptr(), weight.data_ptr(), parts.data_ptr(), m, n, k, a.stride(0), k, n,
          _stream())


def linear_tc_glu(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``linear_glu`` through the TMA + tcgen05 kernel."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", torch.bfloat16, contiguous=False)
    m, k = a.shape
    n = weight.shape[0] // 2
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1 or not linear_glu_supported(a, weight, 64):
        raise KernelError("linear_tc_glu: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    _call(_fn_tc("erb_linear_tc_glu"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, lda, k, ldo,
          _stream())


def linear_tc_rope_store(a: torch.Tensor, weight: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                         inv_freq: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, slots: torch.Tensor,
                         k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int) -> None:
    """``linear_rope_store`` through the TMA + tcgen05 kernel (head sizes 32, 64, 128)."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32); _need(slots, "slots", torch.int32)
    _need(k_pages, "k_pages", torch.bfloat16); _need(v_pages, "v_pages", torch.bfloat16)
    m, k = a.shape
    width = (n_q_heads + 2 * n_kv_heads) * head_dim
    if (weight.shape != (width, k) or qkv.shape != (m, width) or a.stride(1) != 1 or qkv.stride(1) != 1
            or positions.numel() < m or slots.numel() < m or inv_freq.numel() != head_dim // 2
            or k_pages.shape[1:] != (n_kv_heads, page_size, head_dim) or v_pages.shape != k_pages.shape
            or head_dim not in (32, 64, 128) or not linear_rope_store_supported(a, weight, head_dim, head_dim, 64)):
        raise KernelError("linear_tc_rope_store: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = qkv.stride(0) if m > 1 else max(width, qkv.stride(0))
    _call(_fn_tc("erb_linear_tc_rope"), a.data_ptr(), weight.data_ptr(), qkv.data_ptr(), m, k, lda, k, ldo,
          n_q_heads, n_kv_heads, head_dim, positions.data_ptr(), inv_freq.data_ptr(), slots.data_ptr(),
          k_pages.data_ptr(), v_pages.data_ptr(), page_size, _stream())


def linear_glu_supported(a: torch.Tensor, weight: torch.Tensor, max_rows: int = SKINNY_MAX_ROWS) -> bool:
    """Whether the gated products take these operands: a handful of bfloat16 rows (``max_rows``: 16 where
    the register-fed kernel is the better choice, up to 64 for the kernels' own limit), 16-byte rows."""
    lda = a.stride(0) if a.shape[0] > 1 else max(a.shape[1], a.stride(0))
    return a.shape[0] <= max_rows and weight.shape[0] % 2 == 0 and linear_few_rows_supported(a, weight, lda)


def linear_glu(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, bounded: tuple | None = None) -> None:
    """out[M, N] = silu(a @ gate^T) * (a @ up^T) for ``weight = [gate; up]`` of shape [2N, K], in one
    launch; equal to ``linear`` into an [M, 2N] buffer followed by ``swiglu`` (each product is rounded
    to bfloat16 before the gate).  ``bounded = (limit, alpha, shift[, act])``: the gate of ``glu_bounded`` instead,
    equal to ``linear`` followed by ``glu_bounded``."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(out, "out", torch.bfloat16, contiguous=False)
    m, k = a.shape
    n = weight.shape[0] // 2
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1 or not linear_glu_supported(a, weight, 64):
        raise KernelError("linear_glu: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    if bounded is not None:
        limit, alpha, shift = bounded[:3]
        act = bounded[3] if len(bounded) > 3 else "sigmoid"
        _call(_fn("gemm", "bfloat16", "erb_linear_skinny_glu_bounded"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
              lda, k, ldo, float(limit), float(alpha), float(shift), GLU_ACTS[act], _stream())
        return
    _call(_fn("gemm", "bfloat16", "erb_linear_skinny_glu"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
          lda, k, ldo, _stream())


def linear_rope_store_supported(a: torch.Tensor, weight: torch.Tensor, head_dim: int, rot_dim: int,
                                max_rows: int = SKINNY_MAX_ROWS) -> bool:
    """Whether the products with the rotary epilogue take these operands: a handful of bfloat16 rows
    (``max_rows`` as for ``linear_glu_supported``), full rotation, head sizes in steps of 16."""
    lda = a.stride(0) if a.shape[0] > 1 else max(a.shape[1], a.stride(0))
    return (a.shape[0] <= max_rows and rot_dim == head_dim and head_dim % 16 == 0
            and linear_few_rows_supported(a, weight, lda))


def linear_rope_store(a: torch.Tensor, weight: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                      inv_freq: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, slots: torch.Tensor,
                      k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int) -> None:
    """``linear(a, [Wq; Wk; Wv], qkv)`` followed by ``rope_cache_write`` in one launch, for a few rows:
    rotated q lands in ``qkv``'s q columns (its k and v columns are left as they are), rotated k and
    v in the tokens' cache slots.  Same bits as the two kernels."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(weight, "weight", torch.bfloat16)
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32); _need(slots, "slots", torch.int32)
    _need(k_pages, "k_pages", torch.bfloat16); _need(v_pages, "v_pages", torch.bfloat16)
    m, k = a.shape
    width = (n_q_heads + 2 * n_kv_heads) * head_dim
    if (weight.shape != (width, k) or qkv.shape != (m, width) or a.stride(1) != 1 or qkv.stride(1) != 1
            or positions.numel() < m or slots.numel() < m or inv_freq.numel() != head_dim // 2
            or k_pages.shape[1:] != (n_kv_heads, page_size, head_dim) or v_pages.shape != k_pages.shape
            or not linear_rope_store_supported(a, weight, head_dim, head_dim, 64)):
        raise KernelError("linear_rope_store: shapes, strides or operands not supported")
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = qkv.stride(0) if m > 1 else max(width, qkv.stride(0))
    _call(_fn("gemm", "bfloat16", "erb_linear_skinny_rope"), a.data_ptr(), weight.data_ptr(), qkv.data_ptr(), m, k,
          lda, k, ldo, n_q_heads, n_kv_heads, head_dim, positions.data_ptr(), inv_freq.data_ptr(), slots.data_ptr(),
          k_pages.data_ptr(), v_pages.data_ptr(), page_size, _stream())


LINEAR_TUNE_FROM_ROWS = 1024     # rows from which the library's proposals for a shape are timed (as in csrc/gemm.cu)


def linear_tune(dtype: torch.dtype, on: bool) -> None:
    """Switch trials of the library's proposals on or off for the library products (of this element type) that
    follow: while on, a shape of ``LINEAR_TUNE_FROM_ROWS`` rows or more that has had no trial yet gets one
    (every proposal timed on the caller's operands with the weights from DRAM; the fastest stays for the
    process).  A trial costs as much as several steps: it is for a run whose shapes will be used many
    times more, such as the run before a step's layout is captured into a CUDA graph."""
    _fn("gemm", _ELEM[dtype], "erb_linear_tune")(int(bool(on)))


def linear_trials(dtype: torch.dtype) -> int:
    """How many product shapes (of this element type) have had a trial in this process."""
    return int(_fn("gemm", _ELEM[dtype], "erb_linear_trials")())


def linear(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
           library: bool = False) -> None:
    """out[M, N] (+)= a[M, K] @ weight[N, K]^T (float accumulation, no TF32).  bfloat16 rows of a
    decode step go through this package's weight-streaming kernels: up to ``SKINNY_MAX_ROWS`` rows the
    register-fed one, up to ``TC_MAX_ROWS`` rows the TMA + tcgen05 one where the product has enough
    rows of w to give every SM a block without a split over k (the output head).  Within each of the
    two a row's bits do not depend on how many other rows the step has.  Everything else, or all with
    ``library=True``, is a library product.

    ``a`` and ``out`` may be row-strided views (last dimension contiguous); ``out`` is float or the
    element type of ``a``.
    """
    _need(a, "a", contiguous=False); _need(weight, "weight", a.dtype); _need(out, "out", contiguous=False)
    m, k = a.shape
    n = weight.shape[0]
    if weight.shape[1] != k or out.shape != (m, n) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear: shapes or strides disagree")
    if out.dtype not in (a.dtype, torch.float32):
        raise KernelError("linear: out must be float32 or the input type")
    if m == 0:
        return
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    if m <= TC_MAX_ROWS and not accumulate and not library and linear_few_rows_supported(a, weight, lda):
        if m <= SKINNY_MAX_ROWS:
            # a handful of rows: this package's weight-streaming kernel instead of the library product
            _call(_fn("gemm", "bfloat16", "erb_linear_skinny"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
                  lda, k, ldo, int(out.dtype == torch.float32), _stream())
            return
        if n >= 128 * 2 * _sms(a.device):
            _call(_fn_tc("erb_linear_tc"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
                  lda, k, ldo, int(out.dtype == torch.float32), _stream())
            return
    ws = _workspace(a.device)
    _call(_fn("gemm", _elem(a), "erb_linear"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
          lda, k, ldo, int(out.dtype == torch.float32), int(accumulate), ws.data_ptr(), ws.numel(), _stream())


def linear_batched(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, b, :] = a[:, b, :] @ weight[b]^T for every b: ``a`` ``[M, B, K]``, ``weight`` ``[B, N, K]``
    contiguous, ``out`` ``[M, B, N]`` (float32 or the input type); ``a`` and ``out`` may be views with
    any row and batch strides (unit inner stride): the heads of a row against a matrix per head.
    One library call (float accumulation, no TF32)."""
    _need(a, "a", contiguous=False); _need(weight, "weight", a.dtype); _need(out, "out", contiguous=False)
    m, b, k = a.shape
    n = weight.shape[1]
    if weight.shape != (b, n, k) or out.shape != (m, b, n) or a.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("linear_batched: shapes or strides disagree")
    if out.dtype not in (a.dtype, torch.float32):
        raise KernelError("linear_batched: out must be float32 or the input type")
    if m == 0:
        return
    lda = a.stride(0) if m > 1 else max(k, a.stride(0))
    ldo = out.stride(0) if m > 1 else max(n, out.stride(0))
    ws = _workspace(a.device)
    _call(_fn("gemm", _elem(a), "erb_linear_batched"), a.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, lda, k, ldo,
          int(out.dtype == torch.float32), b, a.stride(1), n * k, out.stride(1), ws.data_ptr(), ws.numel(), _stream())


# --- attention through a latent ----------------------------------------------------------------

def latent_store(proj: torch.Tensor, positions: torch.Tensor, eps: float, *, off_kv: int = -1, rank: int = 0, rot_dim: int = 0,
                 kv_weight: torch.Tensor | None = None, inv_freq: torch.Tensor | None = None, rot_dims: int = 0,
                 slots: torch.Tensor | None = None, pages: torch.Tensor | None = None, off_q: int = 0, q_rank: int = 0,
                 q_weight: torch.Tensor | None = None, q_latent: torch.Tensor | None = None) -> None:
    """From each token's row of a fused projection: (``off_kv >= 0``) the cache row ``[unit_rms(row[off_kv :
    off_kv + rank]) * kv_weight | pairs of the next rot_dim entries turned by the position]`` written to slot
    ``slots[t]`` of ``pages`` (``[n_pages, 1, page_size, rank + rot_dim]``); (``q_rank > 0``) ``q_latent[t] =
    unit_rms(row[off_q : off_q + q_rank]) * q_weight``."""
    _need(proj, "proj", contiguous=False); _need(positions, "positions", torch.int32)
    _need(kv_weight, "kv_weight", torch.float32); _need(q_weight, "q_weight", torch.float32)
    _need(inv_freq, "inv_freq", torch.float32); _need(slots, "slots", torch.int32)
    _need(pages, "pages", proj.dtype); _need(q_latent, "q_latent", proj.dtype)
    n = proj.shape[0]
    if proj.stride(1) != 1 or positions.numel() < n:
        raise KernelError("latent_store: proj must be rows with unit inner stride, one position per row")
    if off_kv >= 0:
        if pages is None or slots is None or kv_weight is None or pages.shape[-1] != rank + rot_dim or pages.shape[1] != 1:
            raise KernelError("latent_store: pages must be [pages, 1, page_size, rank + rot_dim]")
        if off_kv + rank + rot_dim > proj.shape[1] or kv_weight.numel() != rank or slots.numel() < n:
            raise KernelError("latent_store: the down-projection lies outside the row")
        if rot_dims and (inv_freq is None or inv_freq.numel() != rot_dims // 2):
            raise KernelError("latent_store: inv_freq must hold rot_dims / 2 values")
    if q_rank and (q_weight is None or q_latent is None or q_weight.numel() != q_rank or off_q + q_rank > proj.shape[1]
                   or q_latent.shape != (n, q_rank)):
        raise KernelError("latent_store: the query latent lies outside the row or its target has another shape")
    _call(_fn("latent_attention", _elem(proj), "erb_latent_store"), proj.data_ptr(), n, proj.stride(0) if n > 1 else proj.shape[1],
          int(off_kv), int(rank), int(rot_dim), _ptr(kv_weight), float(eps), positions.data_ptr(), _ptr(inv_freq), int(rot_dims),
          _ptr(slots), _ptr(pages), int(off_q), int(q_rank), _ptr(q_weight), _ptr(q_latent), _stream())


def latent_q_rotate(q: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None, n_heads: int, dim: int,
                    rot_dim: int, rank: int, rot_dims: int, q_lat: torch.Tensor) -> None:
    """q rows hold per head ``dim`` plain then ``rot_dim`` rotated entries; the latter go, pairs turned by
    the position, to ``q_lat[t, head, rank:]`` (float ``[tokens, heads, rank + rot_dim]``)."""
    _need(q, "q", contiguous=False); _need(positions, "positions", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    _need(q_lat, "q_lat", torch.float32)
    n = q.shape[0]
    if q.stride(1) != 1 or q.shape[1] < n_heads * (dim + rot_dim) or q_lat.shape != (n, n_heads, rank + rot_dim):
        raise KernelError("latent_q_rotate: shapes disagree")
    _call(_fn("latent_attention", _elem(q), "erb_latent_q_rotate"), q.data_ptr(), n, q.stride(0) if n > 1 else q.shape[1],
          n_heads, dim, rot_dim, rank, positions.data_ptr(), _ptr(inv_freq), int(rot_dims), q_lat.data_ptr(), _stream())


def latent_scratch_floats(n_tokens: int, n_heads: int, rank: int, n_splits: int) -> int:
    return n_tokens * n_heads * n_splits * (rank + 2) if n_splits > 1 else 0


def latent_attention(q_lat: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor, seq_of_token: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, scale: float, first_token: int, n_tokens: int, *,
                     gate: torch.Tensor | None = None, sink: torch.Tensor | None = None, split_keys: int = 0,
                     n_splits: int = 1, part: torch.Tensor | None = None, window: int = 0) -> None:
    """Causal multi-query attention of tokens ``first_token .. first_token + n_tokens`` over their sequences'
    cache rows ``[c | kr]``: ``q_lat`` float ``[tokens, heads, rank + rot]`` (absorbed and rotated queries),
    ``out[t, h] = gate(t, h) * softmax_j(scale * q_lat[t, h] . row_j (+ sink_h in the denominator)) @ c_j``
    as ``[tokens, heads, rank]``.  ``gate``: ``[tokens, heads]`` logits (a view with unit inner stride) whose
    sigmoid multiplies the result.  With ``n_splits > 1`` the keys are cut at multiples of ``split_keys`` and
    ``part`` takes the splits' states."""
    _need(q_lat, "q_lat", torch.float32); _need(pages, "pages"); _need(block_tables, "block_tables", torch.int32)
    _need(seq_of_token, "seq_of_token", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", pages.dtype); _need(gate, "gate", pages.dtype, contiguous=False); _need(sink, "sink", torch.float32)
    _need(part, "part", torch.float32)
    n, heads, dk = q_lat.shape
    rank = out.shape[2]
    page_size = pages.shape[2]
    if pages.shape[1] != 1 or pages.shape[3] != dk or out.shape[:2] != (n, heads) or rank > dk:
        raise KernelError("latent_attention: q_lat, pages and out disagree")
    if first_token < 0 or first_token + n_tokens > n or seq_of_token.numel() < n or positions.numel() < n:
        raise KernelError("latent_attention: the token range lies outside the batch")
    if gate is not None and (gate.shape != (n, heads) or gate.stride(1) != 1):
        raise KernelError("latent_attention: gate must be [tokens, heads] with unit inner stride")
    if sink is not None and sink.numel() != heads:
        raise KernelError("latent_attention: one sink per head")
    if n_splits > 1 and (part is None or part.numel() < latent_scratch_floats(n_tokens, heads, rank, n_splits)):
        raise KernelError("latent_attention: the scratch for the splits is too small")
    fn = _fn("latent_attention", _elem(pages), "erb_latent_attention")
    fn._erb_own = 2 if n_splits > 1 else 1
    _call(fn, q_lat.data_ptr(), pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], seq_of_token.data_ptr(),
          positions.data_ptr(), _ptr(gate), 0 if gate is None else (gate.stride(0) if n > 1 else heads), _ptr(sink),
          out.data_ptr(), _ptr(part), int(first_token), int(n_tokens), heads, rank, dk - rank, page_size, int(split_keys),
          int(n_splits), float(scale), int(window), _stream())


LATENT_MMA_KEYS = 64       # keys per tile of the tensor-core form: splits are multiples of it
LATENT_MAX_SPLITS = 64     # splits a row's keys are cut into at most (the merge kernel takes up to 128)


def latent_mma_supported(dtype: torch.dtype, rank: int, rot_dim: int) -> bool:
    """Whether the tensor-core form of the latent attention takes these sizes: bfloat16, cache rows and latents
    of a multiple of 8 entries (16-byte copies, whole column tiles), a latent of at most 512, and two stages
    of 64 rows beside 32 query rows within an SM's shared memory."""
    dk = rank + rot_dim
    d16 = -(-dk // 16) * 16 + 8
    smem = 2 * (32 * d16 + 2 * 64 * d16 + 32 * 72) + 4 * (2 * 8 * 32 + 2 * 32)
    return dtype == torch.bfloat16 and rank % 8 == 0 and dk % 8 == 0 and 0 < rank <= 512 and smem <= 227 * 1024


def latent_mma_tiles(q_lens, n_heads: int, row_tiles: int) -> int:
    """Blocks of ``16 * row_tiles`` (token, head) rows that sequences of these many new tokens need."""
    m = 16 * row_tiles
    return sum(-(-int(n) * n_heads // m) for n in q_lens)


def latent_attention_mma(q_lat: torch.Tensor, pages: torch.Tensor, block_tables: torch.Tensor, seq_starts: torch.Tensor,
                         positions: torch.Tensor, out: torch.Tensor, scale: float, first_seq: int, n_seqs: int, first_token: int,
                         n_tokens: int, n_tiles: int, row_tiles: int, *, gate: torch.Tensor | None = None,
                         sink: torch.Tensor | None = None, split_keys: int = 0, n_splits: int = 1,
                         part: torch.Tensor | None = None, window: int = 0) -> None:
    """``latent_attention`` on tensor cores for sequences ``first_seq .. first_seq + n_seqs`` of the batch (their
    tokens are rows ``first_token .. first_token + n_tokens``, sequence ``s`` owning ``seq_starts[s] ..
    seq_starts[s + 1]`` and row ``s`` of ``block_tables``).  ``n_tiles = latent_mma_tiles(new tokens per sequence,
    heads, row_tiles)``; ``split_keys`` a multiple of ``LATENT_MMA_KEYS``.  ``window`` > 0: a query sees its last ``window``
    keys only; the splits are then counted from the one that holds a row's first visible key."""
    _need(q_lat, "q_lat", torch.float32); _need(pages, "pages", torch.bfloat16); _need(block_tables, "block_tables", torch.int32)
    _need(seq_starts, "seq_starts", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", torch.bfloat16); _need(gate, "gate", torch.bfloat16, contiguous=False); _need(sink, "sink", torch.float32)
    _need(part, "part", torch.float32)
    n, heads, dk = q_lat.shape
    rank = out.shape[2]
    if pages.shape[1] != 1 or pages.shape[3] != dk or out.shape[:2] != (n, heads) or not latent_mma_supported(pages.dtype, rank, dk - rank):
        raise KernelError("latent_attention_mma: q_lat, pages and out disagree, or the sizes are not supported")
    if first_seq < 0 or first_seq + n_seqs > block_tables.shape[0] or seq_starts.numel() < first_seq + n_seqs + 1 or \
            first_token < 0 or first_token + n_tokens > n or positions.numel() < n:
        raise KernelError("latent_attention_mma: the sequence or token range lies outside the batch")
    if gate is not None and (gate.shape != (n, heads) or gate.stride(1) != 1):
        raise KernelError("latent_attention_mma: gate must be [tokens, heads] with unit inner stride")
    if sink is not None and sink.numel() != heads:
        raise KernelError("latent_attention_mma: one sink per head")
    if n_splits > 1 and (part is None or split_keys % LATENT_MMA_KEYS or
                         part.numel() < latent_scratch_floats(n_tokens, heads, rank, n_splits)):
        raise KernelError("latent_attention_mma: splits need scratch and a split size that is a multiple of the key tile")
    gate_ld = 0 if gate is None else (gate.stride(0) if n > 1 else heads)
    _call(_fn("latent_attention", "bfloat16", "erb_latent_attention_mma"), q_lat.data_ptr(), pages.data_ptr(),
          block_tables.data_ptr(), block_tables.shape[1], seq_starts.data_ptr(), positions.data_ptr(), _ptr(gate), gate_ld,
          _ptr(sink), out.data_ptr(), _ptr(part), int(first_token), int(first_seq), int(n_seqs), int(n_tiles), int(row_tiles),
          heads, rank, dk - rank, pages.shape[2], int(split_keys), int(n_splits), float(scale), int(window), _stream())
    if n_splits > 1:
        _call(_fn("latent_attention", "bfloat16", "erb_latent_combine"), part.data_ptr(), _ptr(gate), gate_ld, _ptr(sink),
              out.data_ptr(), int(first_token), int(n_tokens), heads, rank, int(n_splits), _stream())


# --- differential attention ----------------------------------------------------------------------

DIFF_MAX_V_DIM = 256       # entries of a value row the differential-attention kernel keeps per warp


def diff_part_floats(v_dim: int) -> int:
    """Floats of scratch that one (token, head, split) of ``diff_attention`` takes for value rows of ``v_dim`` entries."""
    return 4 + 2 * 64 * (1 if v_dim <= 64 else 2 if v_dim <= 128 else 4)


def diff_prepare(proj: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, n_heads: int, n_kv_heads: int, dim: int,
                 v_dim: int, *, inv_freq: torch.Tensor | None = None, rot_dims: int = 0, conv_w: torch.Tensor | None = None,
                 conv_state: torch.Tensor | None = None, seq_of_token: torch.Tensor | None = None,
                 seq_starts: torch.Tensor | None = None, state_slots: torch.Tensor | None = None,
                 slots: torch.Tensor | None = None, k_pages: torch.Tensor | None = None, v_pages: torch.Tensor | None = None,
                 page_size: int = 1) -> None:
    """What lies between the fused q/k/v product and a differential attention.  A row of ``proj`` holds ``n_heads``
    query heads of two maps (``dim`` entries each), ``n_kv_heads`` key heads of two maps and ``n_kv_heads`` value heads
    (``v_dim``).  ``conv_w`` (float ``[channels, taps]``): a causal convolution over time on every channel, whose inputs
    before a portion's first token come from the request's record in ``conv_state`` (float ``[slots, taps - 1,
    channels]``, oldest first); the halves of the first ``rot_dims`` entries of every map of q and k are turned by
    ``position * inv_freq``; q goes to ``q_out`` ``[tokens, n_heads * 2 * dim]``, k and v to the tokens' cache slots
    (``k_pages`` ``[pages, kv heads, page_size, 2 * dim]``, ``v_pages`` ``[..., v_dim]``; a negative slot writes nothing)."""
    _need(proj, "proj", contiguous=False); _need(q_out, "q_out", proj.dtype); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32); _need(conv_w, "conv_w", torch.float32); _need(conv_state, "conv_state", torch.float32)
    for name, t in (("seq_of_token", seq_of_token), ("seq_starts", seq_starts), ("state_slots", state_slots), ("slots", slots)):
        _need(t, name, torch.int32)
    _need(k_pages, "k_pages", proj.dtype); _need(v_pages, "v_pages", proj.dtype)
    n = proj.shape[0]
    channels = (n_heads + n_kv_heads) * 2 * dim + n_kv_heads * v_dim
    taps = 1 if conv_w is None else conv_w.shape[1]
    if proj.stride(1) != 1 or proj.shape[1] < channels or q_out.shape != (n, n_heads * 2 * dim) or positions.numel() < n:
        raise KernelError("diff_prepare: shapes disagree")
    if rot_dims and (inv_freq is None or inv_freq.numel() != rot_dims // 2):
        raise KernelError("diff_prepare: inv_freq must hold rot_dims / 2 values")
    if conv_w is not None and conv_w.shape[0] != channels:
        raise KernelError("diff_prepare: one row of taps per channel")
    if taps > 1 and (conv_state is None or tuple(conv_state.shape[1:]) != (taps - 1, channels) or seq_of_token is None
                     or seq_starts is None or state_slots is None):
        raise KernelError("diff_prepare: a convolution needs its state [slots, taps - 1, channels] and the step's sequences")
    if slots is not None:
        if k_pages is None or v_pages is None or tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, 2 * dim) or \
                tuple(v_pages.shape[1:]) != (n_kv_heads, page_size, v_dim) or slots.numel() < n:
            raise KernelError("diff_prepare: pages must be [pages, kv heads, page_size, 2 dim] and [..., v_dim]")
    _call(_fn("diff_attention", _elem(proj), "erb_diff_prepare"), proj.data_ptr(), n, proj.stride(0) if n > 1 else proj.shape[1],
          _ptr(conv_w), int(taps), _ptr(conv_state), _ptr(seq_of_token), _ptr(seq_starts), _ptr(state_slots), positions.data_ptr(),
          _ptr(inv_freq), int(rot_dims), int(n_heads), int(n_kv_heads), int(dim), int(v_dim), q_out.data_ptr(), _ptr(slots),
          _ptr(k_pages), _ptr(v_pages), int(page_size), _stream())


def diff_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                   seq_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float,
                   lam: float, eps: float, out_scale: float, first_token: int, n_tokens: int, *, window: int = 0,
                   softcap: float = 0.0, split_keys: int = 0, n_splits: int = 1, part: torch.Tensor | None = None) -> None:
    """Differential attention for rows ``first_token .. first_token + n_tokens`` of the batch: per head two softmax maps
    over the same values, ``o = map1 - lam * map2``, then ``o * rsqrt(mean(o^2) + eps) * out_scale``.  ``q`` ``[tokens,
    n_heads * 2 * dim]`` (both maps of a head side by side), ``k_pages`` ``[pages, kv heads, page_size, 2 * dim]``,
    ``v_pages`` ``[pages, kv heads, page_size, v_dim]``, ``out`` ``[tokens, n_heads * v_dim]``.  Scores are ``q . k *
    scale``, then ``softcap * tanh(score / softcap)`` where a cap is given; a query sees its last ``window`` keys (0: all).
    With ``n_splits > 1`` the keys are cut at multiples of ``split_keys``, counted from the split that holds a row's first
    visible key, and ``part`` takes the splits' states."""
    _need(q, "q"); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype); _need(out, "out", q.dtype)
    _need(block_tables, "block_tables", torch.int32); _need(seq_of_token, "seq_of_token", torch.int32)
    _need(positions, "positions", torch.int32); _need(part, "part", torch.float32)
    n = q.shape[0]
    n_kv, page_size, two_dim = k_pages.shape[1:]
    v_dim = v_pages.shape[3]
    if two_dim % 2 or q.shape[1] != n_heads * two_dim or out.shape != (n, n_heads * v_dim) or n_heads % n_kv or \
            tuple(v_pages.shape[1:3]) != (n_kv, page_size) or v_dim > DIFF_MAX_V_DIM:
        raise KernelError("diff_attention: q, pages and out disagree")
    if first_token < 0 or first_token + n_tokens > n or seq_of_token.numel() < n or positions.numel() < n:
        raise KernelError("diff_attention: the token range lies outside the batch")
    if n_splits > 1 and (part is None or split_keys <= 0 or part.numel() < n_tokens * n_heads * n_splits * diff_part_floats(v_dim)):
        raise KernelError("diff_attention: the scratch for the splits is too small")
    fn = _fn("diff_attention", _elem(q), "erb_diff_attention")
    fn._erb_own = 2 if n_splits > 1 else 1
    _call(fn, q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
          seq_of_token.data_ptr(), positions.data_ptr(), out.data_ptr(), _ptr(part), int(first_token), int(n_tokens), int(n_heads),
          int(n_kv), two_dim // 2, v_dim, page_size, int(window), int(split_keys), int(n_splits), float(scale), float(softcap),
          float(lam), float(eps), float(out_scale), _stream())


DIFF_MMA_ROWS = 64         # (token, head) rows of one sequence and kv head that a block of the tensor-core form owns
DIFF_MMA_TOKEN_ROWS = 16   # the same for single tokens: the block's warps share out the keys instead of the rows
DIFF_MMA_PACKED_ROWS = 8   # single tokens with at most 8 heads a kv head: both maps of a head in one tile of 16 rows


def diff_mma_supported(dtype: torch.dtype, dim: int, v_dim: int) -> bool:
    """Whether the tensor-core form of the differential attention takes these sizes: bfloat16, maps of a multiple of 16
    entries, value rows of a multiple of 8 entries up to 128, and its three tiles within an SM's shared memory."""
    vt = 2 if v_dim <= 32 else 4 if v_dim <= 64 else 6 if v_dim <= 96 else 8
    smem = 2 * ((64 + 2 * 64) * (2 * dim + 8) + 2 * 64 * (16 * vt + 8))
    return dtype == torch.bfloat16 and dim % 16 == 0 and v_dim % 8 == 0 and 0 < v_dim <= 128 and smem <= 227 * 1024


def diff_mma_tiles(q_lens, heads_per_kv: int, tile_rows: int = DIFF_MMA_ROWS) -> int:
    """Blocks of ``tile_rows`` (token, head) rows per kv head that sequences of these many new tokens need."""
    return sum(-(-int(n) * heads_per_kv // tile_rows) for n in q_lens)


def diff_attention_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                       seq_starts: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float,
                       lam: float, eps: float, out_scale: float, first_seq: int, n_seqs: int, first_token: int, n_tokens: int,
                       n_tiles: int, *, window: int = 0, softcap: float = 0.0, split_keys: int = 0, n_splits: int = 1,
                       part: torch.Tensor | None = None, tile_rows: int = DIFF_MMA_ROWS) -> None:
    """``diff_attention`` on tensor cores for sequences ``first_seq .. first_seq + n_seqs`` of the batch (their tokens are
    rows ``first_token .. first_token + n_tokens``, sequence ``s`` owning ``seq_starts[s] .. seq_starts[s + 1]`` and row
    ``s`` of ``block_tables``); ``n_tiles = diff_mma_tiles(new tokens per sequence, heads per kv head, tile_rows)``.
    ``tile_rows`` 64: a block's warps share out the rows (portions); 16: they share out the keys (single tokens with at
    most 16 heads per kv head); 8: single tokens, one a sequence, with at most 8 heads per kv head, whose two maps share
    one tile of 16 rows (half the arithmetic of the form before).  Splits as for ``diff_attention`` (single tokens)."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", torch.bfloat16); _need(v_pages, "v_pages", torch.bfloat16)
    _need(out, "out", torch.bfloat16); _need(block_tables, "block_tables", torch.int32); _need(seq_starts, "seq_starts", torch.int32)
    _need(positions, "positions", torch.int32)
    n = q.shape[0]
    n_kv, page_size, two_dim = k_pages.shape[1:]
    v_dim = v_pages.shape[3]
    if two_dim % 2 or q.shape[1] != n_heads * two_dim or out.shape != (n, n_heads * v_dim) or n_heads % n_kv or \
            tuple(v_pages.shape[1:3]) != (n_kv, page_size) or not diff_mma_supported(q.dtype, two_dim // 2, v_dim):
        raise KernelError("diff_attention_mma: q, pages and out disagree, or the sizes are not supported")
    if first_seq < 0 or first_seq + n_seqs > block_tables.shape[0] or seq_starts.numel() < first_seq + n_seqs + 1 or \
            first_token < 0 or first_token + n_tokens > n or positions.numel() < n:
        raise KernelError("diff_attention_mma: the sequence or token range lies outside the batch")
    _need(part, "part", torch.float32)
    if n_splits > 1 and (part is None or split_keys <= 0 or part.numel() < n_tokens * n_heads * n_splits * diff_part_floats(v_dim)):
        raise KernelError("diff_attention_mma: the scratch for the splits is too small")
    fn = _fn("diff_attention", "bfloat16", "erb_diff_attention_mma")
    fn._erb_own = 2 if n_splits > 1 else 1
    _call(fn, q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
          seq_starts.data_ptr(), positions.data_ptr(), out.data_ptr(), _ptr(part), int(first_token), int(n_tokens), int(first_seq),
          int(n_seqs), int(n_tiles), int(tile_rows), int(n_heads), int(n_kv), two_dim // 2, v_dim, page_size, int(window),
          int(split_keys), int(n_splits), float(scale), float(softcap), float(lam), float(eps), float(out_scale), _stream())


# --- state-space mixer -------------------------------------------------------------------------

def conv_silu(proj: torch.Tensor, off: int, weight: torch.Tensor, bias: torch.Tensor | None, conv_state: torch.Tensor,
              seq_of_token: torch.Tensor, seq_starts: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, ch] = silu(bias[ch] + sum_j weight[ch, j] * input(t - (taps - 1 - j), ch)) over columns ``off ..
    off + channels`` of ``proj``; inputs before the portion's first token come from the request's record in
    ``conv_state`` (float ``[slots, taps - 1, channels]``, oldest first; zeros for a new request)."""
    _need(proj, "proj", contiguous=False); _need(weight, "weight", proj.dtype); _need(bias, "bias", proj.dtype)
    _need(conv_state, "conv_state", torch.float32); _need(out, "out", proj.dtype)
    for name, t in (("seq_of_token", seq_of_token), ("seq_starts", seq_starts), ("state_slots", state_slots)):
        _need(t, name, torch.int32)
    n = proj.shape[0]
    channels, taps = weight.shape
    if proj.stride(1) != 1 or off + channels > proj.shape[1] or out.shape != (n, channels) or \
            tuple(conv_state.shape[1:]) != (taps - 1, channels):
        raise KernelError("conv_silu: shapes disagree")
    _call(_fn("ssm", _elem(proj), "erb_conv_silu"), proj.data_ptr(), n, proj.stride(0) if n > 1 else proj.shape[1], int(off),
          channels, taps, weight.data_ptr(), _ptr(bias), conv_state.data_ptr(), seq_of_token.data_ptr(), seq_starts.data_ptr(),
          state_slots.data_ptr(), out.data_ptr(), _stream())


def conv_state_update(proj: torch.Tensor, off: int, conv_state: torch.Tensor, n_seqs: int, seq_starts: torch.Tensor,
                      state_slots: torch.Tensor) -> None:
    """Every request's record in ``conv_state`` becomes the last ``taps - 1`` inputs of (record, then the step's rows)."""
    _need(proj, "proj", contiguous=False); _need(conv_state, "conv_state", torch.float32)
    _need(seq_starts, "seq_starts", torch.int32); _need(state_slots, "state_slots", torch.int32)
    n = proj.shape[0]
    _, keep, channels = conv_state.shape
    if off + channels > proj.shape[1] or seq_starts.numel() < n_seqs + 1 or state_slots.numel() < n_seqs:
        raise KernelError("conv_state_update: shapes disagree")
    _call(_fn("ssm", _elem(proj), "erb_conv_state_update"), proj.data_ptr(), int(n_seqs), proj.stride(0) if n > 1 else proj.shape[1],
          int(off), channels, keep + 1, conv_state.data_ptr(), seq_starts.data_ptr(), state_slots.data_ptr(), _stream())


def ssm_scan(xbc: torch.Tensor, proj: torch.Tensor, off_dt: int, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
             state: torch.Tensor, n_seqs: int, seq_starts: torch.Tensor, state_slots: torch.Tensor, y: torch.Tensor,
             n_groups: int) -> None:
    """The recurrence of the state-space mixer over every request's rows, from and to its record in ``state``
    (float ``[slots, heads, N, P]``): ``xbc`` rows ``[x (heads * P) | B (groups * N) | C (groups * N)]``, raw
    step sizes in columns ``off_dt .. off_dt + heads`` of ``proj``; ``y`` float ``[tokens, heads * P]``."""
    _need(xbc, "xbc"); _need(proj, "proj", xbc.dtype, contiguous=False); _need(state, "state", torch.float32)
    _need(y, "y", torch.float32)
    for name, t in (("dt_bias", dt_bias), ("a_log", a_log), ("d_skip", d_skip)):
        _need(t, name, torch.float32)
    _need(seq_starts, "seq_starts", torch.int32); _need(state_slots, "state_slots", torch.int32)
    n = xbc.shape[0]
    _, heads, n_state, p = state.shape
    if xbc.shape[1] != heads * p + 2 * n_groups * n_state or y.shape != (n, heads * p) or off_dt + heads > proj.shape[1] or \
            dt_bias.numel() != heads or a_log.numel() != heads or d_skip.numel() != heads or proj.shape[0] != n:
        raise KernelError("ssm_scan: shapes disagree")
    _call(_fn("ssm", _elem(xbc), "erb_ssm_scan"), xbc.data_ptr(), xbc.shape[1], proj.data_ptr(),
          proj.stride(0) if n > 1 else proj.shape[1], int(off_dt), dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(),
          state.data_ptr(), seq_starts.data_ptr(), state_slots.data_ptr(), y.data_ptr(), int(n_seqs), n, heads, p, n_state,
          int(n_groups), _stream())


def gated_group_norm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, parts: int = 1,
                     gate: torch.Tensor | None = None) -> None:
    """out = unit_rms(x * silu(gate)) * weight, the mean square taken over each of ``parts`` equal pieces of a
    row; ``x`` float32 or the element type, ``gate`` (optional) and ``out`` the element type; row-strided views allowed."""
    _need(x, "x", contiguous=False); _need(weight, "weight", torch.float32); _need(out, "out", contiguous=False)
    _need(gate, "gate", out.dtype, contiguous=False)
    n, width = out.shape
    if x.shape != (n, width) or weight.numel() != width or x.dtype not in (torch.float32, out.dtype) or \
            x.stride(1) != 1 or out.stride(1) != 1 or (gate is not None and (gate.shape != (n, width) or gate.stride(1) != 1)):
        raise KernelError("gated_group_norm: shapes or types disagree")
    ld = lambda t: t.stride(0) if n > 1 else width   # noqa: E731
    _call(_fn("ssm", _elem(out), "erb_gated_group_norm"), x.data_ptr(), int(x.dtype == torch.float32), ld(x), _ptr(gate), 0 if gate is None else ld(gate), weight.data_ptr(), out.data_ptr(), ld(out), n, width, int(parts),
          float(eps), _stream())


# --- the gated delta rule ------------------------------------------------------------------------

DELTA_MAX_KEY_DIM = 512      # entries of a key the scan kernel holds per column (32 lanes of 16)


def delta_scratch_floats(n_tokens: int, n_heads: int, n_key_heads: int, key_dim: int, v_dim: int) -> int:
    """Floats of the scratch ``delta_scan`` fills for a step of ``n_tokens`` tokens: per token the unit queries and keys of
    every key head, three scalars per head and the values, rows padded to 16 bytes."""
    pad = lambda v: (v + 3) & ~3   # noqa: E731
    return n_tokens * (n_key_heads * 2 * pad(key_dim) + n_heads * 4 + n_heads * pad(v_dim))


def delta_scan(qkv: torch.Tensor, proj: torch.Tensor, off_b: int, off_a: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
               state: torch.Tensor, n_seqs: int, seq_starts: torch.Tensor, state_slots: torch.Tensor, out: torch.Tensor,
               n_key_heads: int, key_dim: int, scratch: torch.Tensor | None = None) -> None:
    """The gated delta rule over every request's rows, from and to its record in ``state`` (float ``[slots, heads,
    vdim, key_dim]``, the matrix of a head stored with the value index first).  ``qkv``: convolved and activated rows
    ``[q (key heads * key_dim) | k (the same) | v (heads * vdim)]``; the raw write strengths and decay inputs are
    columns ``off_b .. off_b + heads`` and ``off_a .. off_a + heads`` of ``proj``.  Per token and head: q and k are
    made unit vectors (q also times ``key_dim ** -0.5``), ``beta = sigmoid(b)``, ``g = exp(-exp(a_log) * softplus(a +
    dt_bias))``, ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q``.  ``out`` float ``[tokens, heads * vdim]``.
    ``scratch``: float, ``delta_scratch_floats`` entries (None: allocated here), where a first kernel leaves every token's
    unit vectors, scalars and values for the walk along the tokens."""
    _need(qkv, "qkv"); _need(proj, "proj", qkv.dtype, contiguous=False); _need(state, "state", torch.float32)
    _need(out, "out", torch.float32); _need(dt_bias, "dt_bias", torch.float32); _need(a_log, "a_log", torch.float32)
    _need(seq_starts, "seq_starts", torch.int32); _need(state_slots, "state_slots", torch.int32)
    n = qkv.shape[0]
    _, heads, vdim, d = state.shape
    if d != key_dim or qkv.shape[1] != 2 * n_key_heads * d + heads * vdim or out.shape != (n, heads * vdim) or \
            proj.shape[0] != n or max(off_b, off_a) + heads > proj.shape[1] or dt_bias.numel() != heads or \
            a_log.numel() != heads or heads % n_key_heads or seq_starts.numel() < n_seqs + 1 or state_slots.numel() < n_seqs:
        raise KernelError("delta_scan: shapes disagree")
    need = delta_scratch_floats(n, heads, n_key_heads, d, vdim)
    if scratch is None:
        scratch = torch.empty(max(need, 4), dtype=torch.float32, device=qkv.device)
    _need(scratch, "scratch", torch.float32)
    if scratch.numel() < need:
        raise KernelError("delta_scan: the scratch is too small")
    _call(_fn("delta", _elem(qkv), "erb_delta_scan"), qkv.data_ptr(), qkv.shape[1], proj.data_ptr(),
          proj.stride(0) if n > 1 else proj.shape[1], int(off_b), int(off_a), dt_bias.data_ptr(), a_log.data_ptr(),
          state.data_ptr(), seq_starts.data_ptr(), state_slots.data_ptr(), out.data_ptr(), scratch.data_ptr(), int(n_seqs), n, heads,
          int(n_key_heads), d, vdim, _stream())


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n_heads: int, eps: float) -> None:
    """out = o / sqrt(mean(o^2) + eps) * weight * silu(gate), the mean taken over every head's ``vdim`` entries, one
    weight vector of ``vdim`` entries for all heads.  ``o`` float ``[tokens, heads * vdim]``; ``gate`` a view with unit
    inner stride and ``out`` of the element type."""
    _need(o, "o", torch.float32); _need(gate, "gate", out.dtype, contiguous=False); _need(weight, "weight", torch.float32)
    _need(out, "out")
    n, width = o.shape
    if width % n_heads or weight.numel() != width // n_heads or out.shape != (n, width) or gate.shape != (n, width) or \
            gate.stride(1) != 1:
        raise KernelError("head_norm_gate: shapes disagree")
    _call(_fn("delta", _elem(out), "erb_head_norm_gate"), o.data_ptr(), gate.data_ptr(), gate.stride(0) if n > 1 else width,
          weight.data_ptr(), out.data_ptr(), n, int(n_heads), width // n_heads, float(eps), _stream())


# --- routed experts ------------------------------------------------------------------------------

def moe_tile_rows() -> int:
    """Rows of one tile of the experts' products: an expert's list of rows is walked in tiles of this many."""
    return int(_fn("moe", "float32", "erb_moe_tile_rows")())


def moe_lists_ints(n_tokens: int, n_experts: int, top: int) -> int:
    """int32 entries of the scratch ``moe_route`` fills: choices and order per pair, counts, offsets, tile offsets."""
    return 2 * n_tokens * top + 3 * (n_experts + 1)


def _moe_lists(lists: torch.Tensor, n_tokens: int, n_experts: int, top: int):
    pairs = n_tokens * top
    if lists.numel() < moe_lists_ints(n_tokens, n_experts, top):
        raise KernelError("moe: the scratch of lists is too small")
    e1 = n_experts + 1
    choice, order = lists[:pairs], lists[pairs: 2 * pairs]
    counts, offsets, tiles = (lists[2 * pairs + i * e1: 2 * pairs + (i + 1) * e1] for i in range(3))
    return choice, order, counts, offsets, tiles


MOE_SCORES = {"sigmoid": 0, "softmax": 1}


def moe_route(x: torch.Tensor, w_router: torch.Tensor, top: int, lists: torch.Tensor, score: torch.Tensor,
              tile_rows: int = 0, scores: str = "sigmoid", groups: tuple[int, int] | None = None) -> None:
    """Route every row of ``x`` (element type, row-strided view allowed): logits ``w_router x`` in float (``w_router``
    float ``[experts, width]``), the ``top`` largest chosen (the lower index wins a tie), ``score`` float ``[tokens *
    top]`` their sigmoids; ``lists`` (int32, ``moe_lists_ints`` entries) receives the choices and, per expert, the list
    of its (token, choice) pairs in rising order with offsets, all made on the device.  ``tile_rows``: the rows of a tile
    that the lists' tile offsets count (0: those of ``moe_gate_up`` and ``moe_down``; ``moe_tc_tile_rows`` for the
    tensor-core products).  ``scores``: ``sigmoid`` of the logit, or ``softmax`` over all experts' logits.  ``groups =
    (count, keep)``: the experts form ``count`` equal groups of neighbours, a group counts as much as its best expert, and
    only experts of the ``keep`` best groups can be chosen."""
    _need(x, "x", contiguous=False); _need(w_router, "w_router", torch.float32); _need(lists, "lists", torch.int32)
    n_groups, keep = groups if groups else (1, 1)
    _need(score, "score", torch.float32)
    n, width = x.shape
    n_experts = w_router.shape[0]
    if w_router.shape[1] != width or x.stride(1) != 1 or score.numel() < n * top:
        raise KernelError("moe_route: shapes disagree")
    choice, order, counts, offsets, tiles = _moe_lists(lists, n, n_experts, top)
    _call(_fn("moe", _elem(x), "erb_moe_route"), x.data_ptr(), x.stride(0) if n > 1 else width, w_router.data_ptr(), n, width,
          n_experts, int(top), choice.data_ptr(), score.data_ptr(), counts.data_ptr(), offsets.data_ptr(), tiles.data_ptr(),
          order.data_ptr(), int(tile_rows), MOE_SCORES[scores], int(n_groups), int(keep), _stream())


def moe_tc_supported(dtype: torch.dtype, width: int, ff: int) -> bool:
    """Shapes the tensor-core products of the routed experts take: bfloat16, rows of whole 16-byte pieces."""
    return dtype == torch.bfloat16 and width % 8 == 0 and ff % 8 == 0


def moe_tc_tile_rows(n_tokens: int, n_experts: int, top: int) -> int:
    """Rows of a tile of the tensor-core products for this many tokens: 16 to 128, the smallest that holds an expert's
    even share of the (token, choice) pairs, so that few rows cost few columns of the accumulator and many rows re-read
    the weight seldom."""
    share = -(-n_tokens * top // max(1, n_experts))
    return 16 if share <= 16 else 32 if share <= 32 else 64 if share <= 64 else 128


def moe_tc_gather(x: torch.Tensor, lists: torch.Tensor, score: torch.Tensor | None, n_experts: int, top: int, xs: torch.Tensor) -> None:
    """xs[list row] = round(score * x[token]) for every (token, choice) pair, in the order of the experts' lists
    (``score`` None: the rows as they are)."""
    _need(x, "x", torch.bfloat16, contiguous=False); _need(xs, "xs", torch.bfloat16); _need(score, "score", torch.float32)
    n, width = x.shape
    if xs.shape != (n * top, width) or x.stride(1) != 1:
        raise KernelError("moe_tc_gather: shapes disagree")
    _, order, _, _, _ = _moe_lists(lists, n, n_experts, top)
    _call(_fn("moe_tc", None, "erb_moe_tc_gather"), x.data_ptr(), x.stride(0) if n > 1 else width, order.data_ptr(), _ptr(score),
          int(top), n, width, xs.data_ptr(), _stream())


def moe_tc_gate_up(xs: torch.Tensor, w_gate_up: torch.Tensor, lists: torch.Tensor, top: int, tile_rows: int, act: torch.Tensor) -> None:
    """``moe_gate_up`` on tensor cores, from the gathered and scaled rows ``xs`` of ``moe_tc_gather``; the lists must have
    been made with ``tile_rows`` rows a tile."""
    _need(xs, "xs", torch.bfloat16); _need(w_gate_up, "w_gate_up", torch.bfloat16); _need(act, "act", torch.bfloat16)
    pairs, width = xs.shape
    n_experts, two_ff, k = w_gate_up.shape
    if k != width or two_ff % 2 or pairs % top or act.shape != (pairs, two_ff // 2):
        raise KernelError("moe_tc_gate_up: shapes disagree")
    _, order, _, offsets, tiles = _moe_lists(lists, pairs // top, n_experts, top)
    _call(_fn("moe_tc", None, "erb_moe_tc_gate_up"), xs.data_ptr(), w_gate_up.data_ptr(), offsets.data_ptr(), tiles.data_ptr(),
          order.data_ptr(), n_experts, int(top), pairs // top, two_ff // 2, width, int(tile_rows), act.data_ptr(), _ptr(_status_word),
          _stream())


def moe_tc_up_act(xs: torch.Tensor, w_up: torch.Tensor, lists: torch.Tensor, top: int, tile_rows: int, act: torch.Tensor) -> None:
    """``moe_up_act`` on tensor cores, from the gathered rows ``xs``: act[list row] = relu(W_up r)^2; ``w_up`` ``[experts, ff, width]``."""
    _need(xs, "xs", torch.bfloat16); _need(w_up, "w_up", torch.bfloat16); _need(act, "act", torch.bfloat16)
    pairs, width = xs.shape
    n_experts, ff, k = w_up.shape
    if k != width or pairs % top or act.shape != (pairs, ff):
        raise KernelError("moe_tc_up_act: shapes disagree")
    _, order, _, offsets, tiles = _moe_lists(lists, pairs // top, n_experts, top)
    _call(_fn("moe_tc", None, "erb_moe_tc_up_act"), xs.data_ptr(), w_up.data_ptr(), offsets.data_ptr(), tiles.data_ptr(),
          order.data_ptr(), n_experts, int(top), pairs // top, ff, width, int(tile_rows), act.data_ptr(), _ptr(_status_word),
          _stream())


def moe_tc_down(act: torch.Tensor, w_down: torch.Tensor, lists: torch.Tensor, top: int, tile_rows: int, parts: torch.Tensor,
                out_score: torch.Tensor | None = None) -> None:
    """``moe_down`` on tensor cores; the lists must have been made with ``tile_rows`` rows a tile."""
    _need(act, "act", torch.bfloat16); _need(w_down, "w_down", torch.bfloat16); _need(parts, "parts", torch.float32)
    _need(out_score, "out_score", torch.float32)
    n_experts, width, ff = w_down.shape
    n = act.shape[0] // top
    if act.shape != (n * top, ff) or parts.dim() != 3 or parts.shape[0] < top or parts.shape[1:] != (n, width):
        raise KernelError("moe_tc_down: shapes disagree")
    _, order, _, offsets, tiles = _moe_lists(lists, n, n_experts, top)
    _call(_fn("moe_tc", None, "erb_moe_tc_down"), act.data_ptr(), w_down.data_ptr(), offsets.data_ptr(), tiles.data_ptr(),
          order.data_ptr(), n_experts, int(top), n, width, ff, int(tile_rows), parts.data_ptr(), _ptr(out_score), _ptr(_status_word),
          _stream())


def moe_gate_up(x: torch.Tensor, w_gate_up: torch.Tensor, lists: torch.Tensor, score: torch.Tensor, top: int,
                act: torch.Tensor) -> None:
    """act[list row] = silu(W_gate r) * (W_up r) with ``r = round(score * x[token])`` for every (token, choice) pair,
    in the order of the experts' lists.  ``w_gate_up`` ``[experts, 2 * ff, width]`` (gate rows, then up rows)."""
    _need(x, "x", contiguous=False); _need(w_gate_up, "w_gate_up", x.dtype); _need(act, "act", x.dtype)
    n, width = x.shape
    n_experts, two_ff, k = w_gate_up.shape
    if k != width or two_ff % 2 or act.shape != (n * top, two_ff // 2) or x.stride(1) != 1:
        raise KernelError("moe_gate_up: shapes disagree")
    _, order, _, offsets, tiles = _moe_lists(lists, n, n_experts, top)
    _call(_fn("moe", _elem(x), "erb_moe_product"), x.data_ptr(), x.stride(0) if n > 1 else width, w_gate_up.data_ptr(),
          offsets.data_ptr(), tiles.data_ptr(), order.data_ptr(), score.data_ptr(), n_experts, int(top), n, two_ff // 2, width,
          1, act.data_ptr(), None, _stream())


def moe_up_act(x: torch.Tensor, w_up: torch.Tensor, lists: torch.Tensor, top: int, act: torch.Tensor) -> None:
    """act[list row] = relu(W_up x[token])^2 for every (token, choice) pair, in the order of the experts' lists: experts
    without a gate branch.  ``w_up`` ``[experts, ff, width]``."""
    _need(x, "x", contiguous=False); _need(w_up, "w_up", x.dtype); _need(act, "act", x.dtype)
    n, width = x.shape
    n_experts, ff, k = w_up.shape
    if k != width or act.shape != (n * top, ff) or x.stride(1) != 1:
        raise KernelError("moe_up_act: shapes disagree")
    _, order, _, offsets, tiles = _moe_lists(lists, n, n_experts, top)
    _call(_fn("moe", _elem(x), "erb_moe_product"), x.data_ptr(), x.stride(0) if n > 1 else width, w_up.data_ptr(),
          offsets.data_ptr(), tiles.data_ptr(), order.data_ptr(), None, n_experts, int(top), n, ff, width,
          2, act.data_ptr(), None, _stream())


def moe_down(act: torch.Tensor, w_down: torch.Tensor, lists: torch.Tensor, top: int, parts: torch.Tensor,
             out_score: torch.Tensor | None = None) -> None:
    """parts[choice, token] = W_down[expert] act[list row]: float ``[>= top, tokens, width]`` partial sums of the
    tokens' updates, one per choice (times the pair's ``out_score`` where given).  ``w_down`` ``[experts, width, ff]``."""
    _need(act, "act"); _need(w_down, "w_down", act.dtype); _need(parts, "parts", torch.float32)
    _need(out_score, "out_score", torch.float32)
    n_experts, width, ff = w_down.shape
    n = act.shape[0] // top
    if act.shape != (n * top, ff) or parts.dim() != 3 or parts.shape[0] < top or parts.shape[1:] != (n, width):
        raise KernelError("moe_down: shapes disagree")
    _, order, _, offsets, tiles = _moe_lists(lists, n, n_experts, top)
    _call(_fn("moe", _elem(act), "erb_moe_product"), act.data_ptr(), ff, w_down.data_ptr(), offsets.data_ptr(),
          tiles.data_ptr(), order.data_ptr(), _ptr(out_score), n_experts, int(top), n, width, ff, 0, None, parts.data_ptr(), _stream())


# --- attention -------------------------------------------------------------------------------

DECODE_SPLIT_KEYS = 512


def mask_reach(window: int, chunk: int) -> int:
    """The one integer in which the attention kernels take their mask: a window as it is, a mask of chunks as
    the negative of the chunk's size, 0 for plain causal attention."""
    if window and chunk:
        raise KernelError("attention: a window and a mask of chunks exclude each other")
    if window < 0 or chunk < 0:
        raise KernelError("attention: window and chunk must not be negative")
    return int(window) if window else -int(chunk)


def attention_rows(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                   seq_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                   scale: float, window: int = 0, keep_first: int = 0, chunk: int = 0) -> None:
    """Causal attention of every token over its sequence's pages (general kernel, any portion sizes).
    ``window`` > 0: a query sees the last ``window`` keys (its own included) and the first ``keep_first`` of the sequence.
    ``chunk`` > 0 (instead of a window): a query sees the earlier keys of its own run of ``chunk`` positions, runs
    counted from position 0 of the sequence.

    ``q``: ``[tokens, >= n_q_heads * D]`` view with unit inner stride (the q part of a qkv buffer);
    ``out``: ``[tokens, n_q_heads * D]``; pages ``[n_pages, n_kv_heads, page_size, D]``;
    ``block_tables`` int32 ``[sequences, max_pages]``.
    """
    _need(q, "q", contiguous=False); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    _need(block_tables, "block_tables", torch.int32); _need(seq_of_token, "seq_of_token", torch.int32)
    _need(positions, "positions", torch.int32); _need(out, "out", q.dtype, contiguous=False)
    n = q.shape[0]
    _, nkv, page_size, d = k_pages.shape
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] < n_q_heads * d or out.shape[1] < n_q_heads * d:
        raise KernelError("attention_rows: q/out layout disagrees with the head counts")
    _call(_fn("attention", _elem(q), "erb_attention_rows"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], seq_of_token.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), n, n_q_heads, nkv, d, page_size, mask_reach(window, chunk),
          int(keep_first), float(scale), _stream())


_sm_counts: dict[int, int] = {}


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch._C._cuda_getDevice()
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def choose_decode_split(n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int = 64) -> int:
    """Keys per split for the decode kernels (see ``_choose_decode_split``; answers are remembered)."""
    return _choose_decode_split(torch._C._cuda_getDevice(), n_seqs, n_kv_heads, max_keys, page_size, head_dim)


@functools.lru_cache(maxsize=4096)
def _choose_decode_split(device: int, n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int) -> int:
    """Keys per split for the decode kernels, from 128 to 2048.

    The bulk kernel runs one block per (sequence, group of neighbouring kv heads, split), two blocks per SM.
    Measured on the decode step (24 layers, contexts of 8,192, batches of 1 to 16): best is the
    largest split that still fills most of one wave of blocks; a little more than one wave is worst
    (the few blocks of the second wave stream alone, far below the memory's bandwidth); from about
    two waves on, the largest such split, but no more than 1024 keys once there are many waves.  A function of the batch's size and of a power-of-two
    bound on its longest context only, so an eager step and a captured one make the same choice.
    """
    sms = _sm_counts.get(device)
    if sms is None:
        sms = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    slots = 2 * sms
    if head_dim in (32, 64, 128):    # the sizes of the bulk-copy kernels: blocks per sequence and split as they group heads
        groups = native.load("attention_tc", None).erb_attention_decode_bulk_groups(n_kv_heads, head_dim, page_size, 512)
    else:                            # the general kernel (and no need to build the other library for it)
        groups = n_kv_heads
    fits = [s for s in (2048, 1024, 512, 256, 128) if s % page_size == 0 or page_size % s == 0]
    if not fits:
        return DECODE_SPLIT_KEYS
    blocks = {s: n_seqs * groups * -(-max_keys // s) for s in fits}
    for s in fits:                       # most of one wave
        if 0.6 * slots <= blocks[s] <= slots:
            return s
    for s in fits:                       # well beyond one wave: splits of 2048 only up to two waves (measured)
        if blocks[s] >= 1.7 * slots and (s <= 1024 or blocks[s] <= 2 * slots):
            return s
    return fits[-1] if blocks[fits[-1]] < slots else min(fits, key=lambda s: abs(blocks[s] - slots))


def context_bound(pages: int) -> tuple[int, int]:
    """(bound, granule) in pages for a batch whose longest context has ``pages`` pages: the bound is
    ``pages`` rounded up to a multiple of the granule, a quarter of the power-of-two bucket it lies in
    (at least 4 pages).  Steps that share a bound share launch shapes (and a captured graph); the
    longest context then lies within one granule below the bound."""
    bucket = max(4, 1 << (max(1, pages) - 1).bit_length())
    granule = max(1, bucket // 4)
    return -(-max(1, pages) // granule) * granule, granule


def choose_decode_plan(n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int = 64,
                       grouped: bool = False, granule: int = 0) -> tuple[int, int]:
    """(keys per split, kv heads per block) for a decode step whose longest context lies in
    (``max_keys`` - ``granule``, ``max_keys``]; heads per block 0 means the kernel's own choice.
    ``grouped``: the kernel for several query heads per kv head runs, which groups by itself."""
    if grouped or head_dim not in (32, 64, 128):
        return choose_decode_split(n_seqs, n_kv_heads, max_keys, page_size, head_dim), 0
    return _choose_decode_plan(torch._C._cuda_getDevice(), n_seqs, n_kv_heads, max_keys, page_size, head_dim,
                               granule if granule > 0 else max_keys)


@functools.lru_cache(maxsize=4096)
def _choose_decode_plan(device: int, n_seqs: int, n_kv_heads: int, max_keys: int, page_size: int, head_dim: int,
                        granule: int) -> tuple[int, int]:
    """The bulk kernel runs one block per (sequence, group of kv heads, split), two blocks per SM.  By
    default it groups as many neighbouring heads as make a page's copy about 8 KB, which long contexts
    and large batches need for bandwidth; a small batch or a short context then gives far fewer blocks
    than SMs, each walking through many stages one after the other.  Measured with caches read from
    DRAM (batches of 1 to 64, contexts of 640 to 8,192): best is the plan with the fewest heads per
    block (from 2) and then the longest splits whose blocks fill most of one wave, e.g. 16 sequences
    of 640 tokens 15 us with 2 heads per block and no split against 23 us with 8 heads and splits of
    256; where no such plan exists the rule of ``_choose_decode_split`` with the default grouping
    stands (it is as good for 8 sequences of 8,192 tokens and better beyond).  Splits are either at
    most a granule long or hold the whole context: a split between the two leaves the longest
    context with one full split and a short rest, and the step waits for the full one (8 sequences
    of 640 tokens: 1.53 ms a step with splits of 512, 1.46 ms with splits of 256).  A function of the
    batch's size and of the bound on the longest context only."""
    split = _choose_decode_split(device, n_seqs, n_kv_heads, max_keys, page_size, head_dim)
    lib = native.load("attention_tc", None)
    default = lib.erb_attention_decode_bulk_head_group(n_kv_heads, head_dim, page_size, 512, 0)
    slots = 2 * _sm_counts[device]
    sizes = [s for s in (2048, 1024, 512, 256, 128, 64)
             if s % page_size == 0 and -(-max_keys // s) <= 64 and (s <= granule or s >= max_keys)]
    finest = None
    for hg in (2, 4, 8):
        if hg > default:
            break
        for s in sizes:
            if lib.erb_attention_decode_bulk_head_group(n_kv_heads, head_dim, page_size, s, hg) != hg:
                continue
            blocks = n_seqs * -(-n_kv_heads // hg) * -(-max_keys // s)
            if 0.6 * slots <= blocks <= slots:
                return s, hg
            if hg == 2:
                finest = (s, hg, blocks)
    if finest is not None and finest[2] < 0.6 * slots:       # even the finest plan leaves SMs idle: take it
        return finest[0], finest[1]
    return split, 0


def decode_scratch_floats(n_seqs: int, n_q_heads: int, head_dim: int, max_splits: int) -> tuple[int, int]:
    return n_seqs * n_q_heads * max_splits * head_dim, n_seqs * n_q_heads * max_splits * 2


def attention_decode(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                     token_of_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                     scale: float, part_acc: torch.Tensor, part_ml: torch.Tensor, max_splits: int,
                     window: int = 0, split_keys: int = DECODE_SPLIT_KEYS, keep_first: int = 0, chunk: int = 0) -> None:
    """Attention of one new token per sequence, keys cut into splits of ``split_keys`` (split-KV).
    With a window the first ``keep_first`` keys stay visible; the first split of the window takes them along.
    ``chunk`` > 0 (instead of a window): the mask of chunks of ``attention_rows``.

    ``token_of_seq`` int32 ``[sequences]`` gives each sequence's row in q/out/positions.  Scratch:
    ``part_acc`` float ``[sequences * heads * max_splits * D]``, ``part_ml`` twice
    ``sequences * heads * max_splits``.
    """
    _need(q, "q", contiguous=False); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    _need(block_tables, "block_tables", torch.int32); _need(token_of_seq, "token_of_seq", torch.int32)
    _need(positions, "positions", torch.int32); _need(out, "out", q.dtype, contiguous=False)
    _need(part_acc, "part_acc", torch.float32); _need(part_ml, "part_ml", torch.float32)
    n_seqs = token_of_seq.numel()
    _, nkv, page_size, d = k_pages.shape
    need_acc, need_ml = decode_scratch_floats(n_seqs, n_q_heads, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError("attention_decode: scratch too small")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode: q/out inner stride must be 1")
    _call(_fn("attention", _elem(q), "erb_attention_decode"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], token_of_seq.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), part_acc.data_ptr(), part_ml.data_ptr(),
          max_splits, n_seqs, n_q_heads, nkv, d, page_size, mask_reach(window, chunk), int(keep_first), int(split_keys),
          float(scale), _stream())


def decode_bulk_supported(dtype: torch.dtype, head_dim: int, window: int, n_q_heads: int, n_kv_heads: int,
                          max_splits: int = 1) -> bool:
    """Shapes the bulk-copy decode kernel takes (with or without a window); everything else goes to the general
    decode kernel."""
    return (dtype == torch.bfloat16 and head_dim in (32, 64, 128)
            and n_q_heads // n_kv_heads <= 8 and max_splits <= 64)


_split_counters: dict[torch.device, torch.Tensor] = {}


def split_counters(device: torch.device, n: int) -> torch.Tensor:
    """The counters by which the split decode kernels find the block that finishes last for each
    (sequence, group of kv heads): one zeroed int32 array per device, shared by all calls (calls on
    one stream follow each other; the kernels leave every counter at zero).  It keeps its address, so
    that captured graphs stay valid."""
    buf = _split_counters.get(device)
    if buf is None:
        buf = _split_counters[device] = torch.zeros(1 << 18, dtype=torch.int32, device=device)
    if n > buf.numel():
        raise KernelError(f"decode attention: {n} (sequence, head group) pairs, at most {buf.numel()}")
    return buf


def reset_split_counters() -> None:
    """Zeroes the counters again: needed after a kernel gave up on a wait (a flagged status), since
    its block did not count."""
    for buf in _split_counters.values():
        buf.zero_()


def attention_decode_bulk(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                          token_of_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                          scale: float, part_acc: torch.Tensor, part_ml: torch.Tensor, max_splits: int,
                          status: torch.Tensor, split_keys: int = DECODE_SPLIT_KEYS, head_group: int = 0, window: int = 0,
                          keep_first: int = 0, chunk: int = 0) -> None:
    """``attention_decode`` for bfloat16 with keys and values streamed by bulk asynchronous copies.
    ``chunk`` > 0 (instead of a window): the mask of chunks of ``attention_rows``.
    ``window`` > 0: the last ``window`` keys and the first ``keep_first``; the splits are counted from the one
    that holds the window's first key, and the first of them also walks the kept keys.
    The splits of a sequence are merged by the block that finishes last (``split_counters``), so
    this is one launch.  ``head_group``: kv heads per block (a power of two; 0: as many as make a
    page's copy about 8 KB)."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16); _need(block_tables, "block_tables", torch.int32)
    _need(token_of_seq, "token_of_seq", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", torch.bfloat16, contiguous=False); _need(part_acc, "part_acc", torch.float32)
    _need(part_ml, "part_ml", torch.float32); _need(status, "status", torch.int32)
    n_seqs = token_of_seq.numel()
    _, nkv, page_size, d = k_pages.shape
    need_acc, need_ml = decode_scratch_floats(n_seqs, n_q_heads, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError("attention_decode_bulk: scratch too small")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode_bulk: q/out inner stride must be 1")
    _call(_fn("attention_tc", None, "erb_attention_decode_bulk"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], token_of_seq.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), part_acc.data_ptr(), part_ml.data_ptr(), max_splits,
          n_seqs, n_q_heads, nkv, d, page_size, int(split_keys), float(scale), status.data_ptr(),
          split_counters(q.device, n_seqs * nkv).data_ptr(), int(head_group), mask_reach(window, chunk), int(keep_first), _stream())


@functools.lru_cache(maxsize=4096)
def decode_gqa_supported(dtype: torch.dtype, head_dim: int, window: int, n_q_heads: int, n_kv_heads: int,
                         page_size: int, split_keys: int, max_splits: int = 1) -> bool:
    """Shapes the tensor-core decode kernel for grouped query heads takes: bfloat16, head size 64,
    2 to 8 query heads per kv head, pages of a multiple of 8 tokens, with or without a window."""
    if dtype != torch.bfloat16 or max_splits > 64 or head_dim != 64 or n_q_heads == n_kv_heads:
        return False        # (answered here so that other models need not build the tensor-core library)
    return bool(native.load("attention_tc", None).erb_attention_decode_gqa_supported(
        n_q_heads, n_kv_heads, head_dim, page_size, int(split_keys)))


def attention_decode_gqa(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                         token_of_seq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_q_heads: int,
                         scale: float, part_acc: torch.Tensor, part_ml: torch.Tensor, max_splits: int,
                         status: torch.Tensor, split_keys: int = DECODE_SPLIT_KEYS, window: int = 0, keep_first: int = 0,
                         chunk: int = 0) -> None:
    """``attention_decode`` for several query heads per kv head on tensor cores (``window`` and ``keep_first`` as in
    ``attention_decode_bulk``): the query heads of a
    kv head are the rows of one matrix tile, pages arrive by TMA tensor copies."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16); _need(block_tables, "block_tables", torch.int32)
    _need(token_of_seq, "token_of_seq", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", torch.bfloat16, contiguous=False); _need(part_acc, "part_acc", torch.float32)
    _need(part_ml, "part_ml", torch.float32); _need(status, "status", torch.int32)
    n_seqs = token_of_seq.numel()
    n_pages, nkv, page_size, d = k_pages.shape
    need_acc, need_ml = decode_scratch_floats(n_seqs, n_q_heads, d, max_splits)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml or v_pages.shape != k_pages.shape:
        raise KernelError("attention_decode_gqa: scratch too small or pools disagree")
    if q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_decode_gqa: q/out inner stride must be 1")
    _call(_fn("attention_tc", None, "erb_attention_decode_gqa"), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), n_pages, block_tables.data_ptr(), block_tables.shape[1], token_of_seq.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), part_acc.data_ptr(), part_ml.data_ptr(), max_splits,
          n_seqs, n_q_heads, nkv, d, page_size, int(split_keys), float(scale), status.data_ptr(),
          split_counters(q.device, n_seqs * nkv).data_ptr(), mask_reach(window, chunk), int(keep_first), _stream())


#: query rows of one (sequence, head) that a block of the tensor-core prefill kernel takes
PREFILL_TC_ROWS = 256


def prefill_tc_supported(dtype: torch.dtype, head_dim: int, window: int, page_size: int = 16) -> bool:
    """Shapes the tensor-core prefill kernel takes (bfloat16, head size 64, with or without a window, pages
    of 8 to 128 tokens, a power of two); everything else goes to the general row kernel."""
    return (dtype == torch.bfloat16 and head_dim == 64
            and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0)


def prefill_tc_blocks(q_lens) -> int:
    """Blocks per head the tensor-core prefill kernel needs for portions of these lengths."""
    return sum(-(-int(n) // PREFILL_TC_ROWS) for n in q_lens)


def prefill_tc_key_splits(n_blocks: int, n_q_heads: int, max_keys: int, device: torch.device) -> int:
    """Ranges to cut every block's keys into: 1 unless the portions give far fewer blocks than the GPU has
    SMs and the walk over the keys is long (512 new tokens after 7,000 cached ones: 30 to 64 blocks of
    59 key tiles each take 131 us whatever their number; cut so that the blocks fill one wave, 4 tiles
    a range at least).  ``max_keys``: a bound on the longest context that steps of one layout share."""
    sms = _sms(device)
    blocks = n_blocks * n_q_heads
    tiles = -(-max_keys // 128)
    if blocks * 2 > sms or tiles < 8:
        return 1
    return max(1, min(sms // blocks, tiles // 4, 16))


def prefill_tc_scratch_floats(n_rows: int, n_q_heads: int, key_splits: int) -> tuple[int, int]:
    """Floats of ``part_o`` and ``part_ml`` for ``attention_prefill_tc`` with key splits over the first ``n_rows`` rows of the batch."""
    return n_rows * n_q_heads * key_splits * 64, n_rows * n_q_heads * key_splits * 2


def attention_prefill_tc(qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                         seq_starts: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, n_blocks: int,
                         n_q_heads: int, scale: float, status: torch.Tensor, key_splits: int = 1, first_row: int = 0,
                         part_o: torch.Tensor | None = None, part_ml: torch.Tensor | None = None, window: int = 0,
                         keep_first: int = 0, chunk: int = 0) -> None:
    """Causal attention of prompt portions on tcgen05 tensor cores (bfloat16, head_dim 64).  ``window`` > 0: a
    query sees the last ``window`` keys (its own included) and the first ``keep_first`` of its sequence.
    ``chunk`` > 0 (instead of a window): the mask of chunks of ``attention_rows``.

    ``qkv`` / ``out``: row t is token t of the batch (the q heads lead each qkv row);
    ``seq_starts`` int32 ``[n + 1]``: token offsets of the n sequences to process, whose block tables
    are the n rows of ``block_tables``; ``n_blocks``: ``prefill_tc_blocks`` of their lengths (an upper
    bound is fine).  ``key_splits`` > 1 (``prefill_tc_key_splits``): every block's keys are cut into
    that many ranges, each a block of its own, and a second kernel merges them; the sequences'
    tokens are then rows ``first_row`` to the end of ``qkv``, and ``part_o`` / ``part_ml`` are float
    scratch of ``prefill_tc_scratch_floats(qkv rows, heads, key_splits)``.
    """
    _need(qkv, "qkv", torch.bfloat16, contiguous=False); _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16); _need(block_tables, "block_tables", torch.int32)
    _need(seq_starts, "seq_starts", torch.int32); _need(positions, "positions", torch.int32)
    _need(out, "out", torch.bfloat16, contiguous=False); _need(status, "status", torch.int32)
    n_pages, nkv, page_size, d = k_pages.shape
    n_seqs = seq_starts.numel() - 1
    if qkv.stride(1) != 1 or out.stride(1) != 1 or block_tables.shape[0] < n_seqs or v_pages.shape != k_pages.shape:
        raise KernelError("attention_prefill_tc: layout disagrees")
    if key_splits > 1:
        _need(part_o, "part_o", torch.float32); _need(part_ml, "part_ml", torch.float32)
        need_o, need_ml = prefill_tc_scratch_floats(qkv.shape[0], n_q_heads, key_splits)
        if part_o is None or part_ml is None or part_o.numel() < need_o or part_ml.numel() < need_ml or not 0 <= first_row < qkv.shape[0]:
            raise KernelError("attention_prefill_tc: scratch for the key ranges is missing or too small")
    _call(_fn("attention_prefill", None, "erb_attention_prefill_tc"), qkv.data_ptr(), qkv.stride(0), k_pages.data_ptr(),
          v_pages.data_ptr(), n_pages, block_tables.data_ptr(), block_tables.shape[1], seq_starts.data_ptr(),
          positions.data_ptr(), out.data_ptr(), out.stride(0), n_seqs, int(n_blocks), n_q_heads, nkv, d, page_size,
          float(scale), status.data_ptr(), int(key_splits), int(first_row), qkv.shape[0] - int(first_row), _ptr(part_o), _ptr(part_ml),
          mask_reach(window, chunk), int(keep_first), _stream())
    if key_splits > 1:
        launch_counts["own"] += 1          # the merge of the ranges


# --- sampling --------------------------------------------------------------------------------

def sample_rows(logits: torch.Tensor, tokens: torch.Tensor, temperature: torch.Tensor | None = None,
                rng_state: torch.Tensor | None = None) -> None:
    """tokens[r] = argmax(logits[r]) where temperature[r] <= 0, else an inverse-CDF draw."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(tokens, "tokens", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(rng_state, "rng_state", torch.int64)
    if logits.stride(1) != 1 or tokens.numel() < logits.shape[0]:
        raise KernelError("sample_rows: layout disagrees")
    _call(_fn("sampling", None, "erb_sample_rows"), logits.data_ptr(), logits.stride(0) if logits.shape[0] > 1 else max(logits.stride(0), logits.shape[1]),
          logits.shape[0], logits.shape[1], _ptr(temperature), _ptr(rng_state), tokens.data_ptr(), _stream())


def uniform_from_state(state: int) -> float:
    """The uniform in [0, 1) that the sampling kernel derives from a 64-bit state (host copy)."""
    z = (state + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    z ^= z >> 31
    return (z >> 40) / 16777216.0
