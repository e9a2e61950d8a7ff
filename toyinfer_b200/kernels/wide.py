"""A float32 residual stream beside activations of the engine's type (csrc/wide_residual.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Optional, Sequence, Tuple, Union

import torch

from . import KernelError, _call, _code, _i32, _need_cuda, _ptr, _stream
from .lib import declare

_fns = {}


def _fn(name, argtypes):
    f = _fns.get(name)
    if f is None:
        f = _fns[name] = declare(name, argtypes)
    return f


P, I, F = c_void_p, c_int, c_float
Pending = Union[None, torch.Tensor, Tuple[Optional[torch.Tensor], ...]]


def pending_terms(delta: Pending) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
    """(d0, d1, d2) of a pending sum: the stream becomes ((d0 + d1) + h) + d2."""
    if delta is None:
        return None, None, None
    if isinstance(delta, torch.Tensor):
        return delta, None, None
    terms = tuple(delta) + (None,) * (3 - len(delta))
    if len(terms) != 3:
        raise KernelError(f"a pending sum has at most three terms, got {len(delta)}")
    return terms


def embed_wide(table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0, copies: int = 1) -> torch.Tensor:
    """float32 out[m] = table[ids[m]] * scale, ``copies`` times side by side ([M, copies * H])."""
    _need_cuda(table, ids, what="embed_wide")
    _i32(ids, "embed_wide ids")
    V, H = table.shape
    out = torch.empty((ids.numel(), int(copies) * H), dtype=torch.float32, device=table.device)
    _call(_fn("ti_embed_wide", [P, P, P, I, I, I, F, I, I, P]), _ptr(table), _ptr(ids), _ptr(out), ids.numel(), H, V,
          float(scale), int(copies), _code(table, "embed_wide"), _stream())
    return out


def add_norm_wide(h: torch.Tensor, delta: Pending, weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                  rows: Optional[torch.Tensor] = None, want_out: bool = True) -> Optional[torch.Tensor]:
    """h (float32 [M, H]) takes the pending terms in place (without ``rows``); returns
    rmsnorm(h) * weight in ``out_dtype`` (the rounded sum itself when ``weight`` is None).  With
    ``rows`` only those rows are summed and normed and h is left as it is."""
    d0, d1, d2 = pending_terms(delta)
    _need_cuda(h, d0, d1, d2, weight, rows, what="add_norm_wide")
    if h.dtype != torch.float32 or h.dim() != 2 or not h.is_contiguous():
        raise KernelError("add_norm_wide: the stream must be a dense float32 [tokens, width] tensor")
    M, H = h.shape
    for d in (d0, d1, d2):
        if d is not None and (d.shape != h.shape or d.dtype != out_dtype or not d.is_contiguous()):
            raise KernelError(f"add_norm_wide: a pending term must be dense {out_dtype} of the stream's shape")
    w_f32 = 0
    if weight is not None:
        if weight.shape != (H,) or not weight.is_contiguous() or weight.dtype not in (out_dtype, torch.float32):
            raise KernelError(f"add_norm_wide: weight {tuple(weight.shape)} {weight.dtype} does not fit rows of {H}")
        w_f32 = 1 if weight.dtype == torch.float32 else 0
    R = M
    if rows is not None:
        _i32(rows, "add_norm_wide rows")
        R = rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=h.device) if want_out else None
    code = 0 if out_dtype == torch.float32 else 1
    _call(_fn("ti_add_norm_wide", [P, P, P, P, P, P, I, P, P, I, I, I, F, I, I, P]),
          _ptr(h), _ptr(d0), _ptr(d1), _ptr(d2), _ptr(rows), _ptr(weight), w_f32, _ptr(out), None, R, H, M, float(eps),
          0 if rows is not None else 1, code, _stream())
    return out
