"""Several float32 residual streams per token and the norm that reads them (csrc/hyper.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

from . import KernelError, _call, _i32, _need_cuda, _ptr, _stream
from .wide import _fn

P, I, F = c_void_p, c_int, c_float


@dataclass
class StreamUpdate:
    """What a sublayer left pending on the streams X [M, S, H]: X_t <- sum_s carry[s, t] X_s + write[t] * (gain * y).
    ``carry`` None is the identity, ``write`` None ones, ``gain`` None no scale."""

    y: torch.Tensor                          # [M, H], the engine's type
    gain: Optional[torch.Tensor] = None      # float32 [H]
    carry: Optional[torch.Tensor] = None     # float32 [S, S], indexed [from, to]
    write: Optional[torch.Tensor] = None     # float32 [S]


def _f32(t: Optional[torch.Tensor], shape, what: str) -> None:
    if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != tuple(shape) or not t.is_contiguous()):
        raise KernelError(f"hyper_norm: {what} must be dense float32 {tuple(shape)}, got {t.dtype} {tuple(t.shape)}")


def hyper_norm(X: torch.Tensor, pending: Optional[StreamUpdate], read: Optional[torch.Tensor], weight: Optional[torch.Tensor],
               eps: float, out_dtype: torch.dtype, streams: int, rows: Optional[torch.Tensor] = None,
               want_sum: bool = False):
    """X (float32 [M, streams * H]) takes the pending update in place (without ``rows``); returns
    rmsnorm(sum_s read[s] X_s) * weight in ``out_dtype`` (``read`` None: ones; ``weight`` None: the rounded sum itself).
    With ``rows`` only those rows are worked on and X is left as it is.  ``want_sum``: also the float32 sum
    (returns a pair)."""
    y = pending.y if pending is not None else None
    gain = pending.gain if pending is not None else None
    carry = pending.carry if pending is not None else None
    write = pending.write if pending is not None else None
    _need_cuda(X, y, gain, carry, write, read, weight, rows, what="hyper_norm")
    S = int(streams)
    if X.dtype != torch.float32 or X.dim() != 2 or not X.is_contiguous() or X.shape[1] % S:
        raise KernelError("hyper_norm: the streams must be a dense float32 [tokens, streams * width] tensor")
    M, H = X.shape[0], X.shape[1] // S
    if y is not None and (tuple(y.shape) != (M, H) or y.dtype != out_dtype or not y.is_contiguous()):
        raise KernelError(f"hyper_norm: the pending output must be dense {out_dtype} [{M}, {H}]")
    _f32(gain, (H,), "the scale")
    _f32(carry, (S, S), "the carry matrix")
    _f32(write, (S,), "the write vector")
    _f32(read, (S,), "the read vector")
    _f32(weight, (H,), "the norm weight")
    R = M
    if rows is not None:
        _i32(rows, "hyper_norm rows")
        R = rows.numel()
    out = torch.empty((R, H), dtype=out_dtype, device=X.device)
    total = torch.empty((R, H), dtype=torch.float32, device=X.device) if want_sum else None
    _call(_fn("ti_hyper_norm", [P, P, P, P, P, P, P, P, P, P, I, I, I, I, F, I, I, P]),
          _ptr(X), _ptr(y), _ptr(gain), _ptr(carry), _ptr(write), _ptr(read), _ptr(weight), _ptr(rows), _ptr(out), _ptr(total),
          R, H, M, S, float(eps), 0 if rows is not None else 1, 0 if out_dtype == torch.float32 else 1, _stream())
    return (out, total) if want_sum else out
