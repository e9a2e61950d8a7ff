"""Mixture-of-experts feed-forward with tokens grouped by expert, and the squared-ReLU activation
(csrc/moe_grouped.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import KernelError, _call, _code, _i32, _need_cuda, _ptr, _stream
from .wide import _fn

P, I, L, F = c_void_p, c_int, c_longlong, c_float


def relu2(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2, elementwise."""
    _need_cuda(x, what="relu2")
    if not x.is_contiguous():
        raise KernelError("relu2: expected a dense tensor")
    out = torch.empty_like(x)
    _call(_fn("ti_relu2", [P, P, L, I, P]), _ptr(x), _ptr(out), x.numel(), _code(x, "relu2"), _stream())
    return out


def route_by_table(ids: torch.Tensor, table: torch.Tensor, n_experts: int):
    """ids int32 [M], table int32 [vocab, top] -> (perm int32 [M * top], off int32 [experts + 1]): the (token, choice)
    pairs grouped by expert."""
    _need_cuda(ids, table, what="moe_route_table")
    _i32(ids, "moe ids")
    _i32(table, "moe table")
    M = ids.numel()
    vocab, top = table.shape
    perm = torch.empty(M * top, dtype=torch.int32, device=ids.device)
    off = torch.empty(n_experts + 1, dtype=torch.int32, device=ids.device)
    scratch = torch.empty(M * top, dtype=torch.int32, device=ids.device)
    _call(_fn("ti_moe_route_table", [P, P, I, I, I, I, P, P, P, P]), _ptr(ids), _ptr(table), vocab, top, n_experts, M,
          _ptr(perm), _ptr(off), _ptr(scratch), _stream())
    return perm, off


def experts_ffn(x: torch.Tensor, perm: torch.Tensor, off: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                w_down: torch.Tensor, top: int, limit: float, alpha: float, weight: float) -> torch.Tensor:
    """x[M, H]; w_gate, w_up [experts, ff, H]; w_down [experts, H, ff].  Every pair's expert output times ``weight``,
    summed per token in the order of its choices -> [M, H]."""
    _need_cuda(x, perm, off, w_gate, w_up, w_down, what="moe")
    M, H = x.shape
    E, ff, H2 = w_gate.shape
    if H2 != H or w_up.shape != w_gate.shape or w_down.shape != (E, H, ff) or x.stride(1) != 1:
        raise KernelError("moe: the experts' matrices do not fit the tokens")
    for t in (w_gate, w_up, w_down):
        if t.dtype != x.dtype or not t.is_contiguous():
            raise KernelError("moe: the experts' matrices must be dense and of the tokens' dtype")
    Pn = M * top
    code = _code(x, "moe")
    fn = _fn("ti_moe_grouped", [P, L, P, P, P, L, P, P, I, I, I, I, I, I, I, I, F, F, F, I, P])
    y = torch.empty((Pn, ff), dtype=x.dtype, device=x.device)
    _call(fn, _ptr(x), x.stride(0), _ptr(w_gate), _ptr(w_up), _ptr(y), ff, _ptr(perm), _ptr(off), E, Pn, ff, H, top, 1, 0, 1,
          1.0, float(limit), float(alpha), code, _stream())
    z = torch.empty((Pn, H), dtype=x.dtype, device=x.device)
    _call(fn, _ptr(y), ff, _ptr(w_down), None, _ptr(z), H, _ptr(perm), _ptr(off), E, Pn, H, ff, top, 0, 1, 0,
          float(weight), 0.0, 0.0, code, _stream())
    if top == 1:
        return z
    out = torch.empty((M, H), dtype=x.dtype, device=x.device)
    _call(_fn("ti_moe_combine", [P, P, I, I, I, I, P]), _ptr(z), _ptr(out), M, H, top, code, _stream())
    return out
