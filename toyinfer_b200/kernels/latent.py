"""Attention over a shared low-rank latent (csrc/attn_latent.cu): the rows that the cache keeps,
the query carried into the latent space, the attention with a window and sinks, and the way out."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import KernelError, _call, _code, _need_cuda, _ptr, _stream
from .wide import _fn

P, I, L, F = c_void_p, c_int, c_longlong, c_float


def _pages(mem):
    if mem is None:
        return (None, None, 0, 0, 0, 0)
    pt = mem.page_table
    return (_ptr(mem.k_pages), _ptr(pt), pt.shape[1], mem.page_size, mem.ring_rows, mem.k_pages.shape[0])


def _check_mem(mem, W: int, dtype, what: str) -> None:
    if mem.n_kv_heads != 1 or mem.head_dim != W or mem.k_pages.dtype != dtype or not mem.k_pages.is_contiguous():
        raise KernelError(f"{what}: the cache does not hold rows of {W} {dtype} elements")


def prep(d: torch.Tensor, q: Optional[torch.Tensor], rank: int, rot: int, norm_w: torch.Tensor, eps: float, tables,
         batch, mem=None) -> torch.Tensor:
    """d[M, rank + rot] (dense rows, any row stride): returns the step's rows [norm(d[:rank]) | rotate(d[rank:])],
    stores them to ``mem``'s pages when given, and rotates q[M, heads, plain + rot]'s rotated part in place."""
    _need_cuda(d, q, norm_w, what="latent_prep")
    M, W = d.shape
    if W != rank + rot or d.stride(1) != 1:
        raise KernelError("latent_prep: the down-projection's rows do not fit rank + rot")
    if norm_w.dtype != torch.float32 or norm_w.shape != (rank,) or not norm_w.is_contiguous():
        raise KernelError("latent_prep: the norm weight must be float32 [rank]")
    cos = sin = None
    max_pos = 0
    if rot:
        cos, sin, dim = tables
        if dim != rot or cos.dtype != torch.float32 or cos.shape != sin.shape or cos.shape[1] * 2 != rot:
            raise KernelError("latent_prep: rotary tables must be float32 [positions, rot / 2]")
        max_pos = cos.shape[0]
        if batch.max_pos_after > max_pos:
            raise KernelError(f"latent_prep: position {batch.max_pos_after - 1} is beyond the rotary tables' {max_pos}")
    nh = plain = 0
    qs = 0
    if q is not None:
        if q.dim() != 3 or q.shape[0] != M or q.stride(2) != 1 or q.stride(1) != q.shape[2] or q.dtype != d.dtype:
            raise KernelError("latent_prep: q must be [M, heads, plain + rot] with dense heads")
        nh, plain, qs = q.shape[1], q.shape[2] - rot, q.stride(0)
    if mem is not None:
        _check_mem(mem, W, d.dtype, "latent_prep")
    lat = torch.empty((M, W), dtype=d.dtype, device=d.device)
    _call(_fn("ti_latent_prep", [P, L, P, L, I, I, I, I, P, F, P, P, I, P, P, P, P, P, P, P, I, I, I, I, I, I, P]),
          _ptr(d), d.stride(0), _ptr(q), qs, nh, plain, rank, rot, _ptr(norm_w), float(eps), _ptr(cos), _ptr(sin), max_pos,
          _ptr(batch.tok_pos), _ptr(batch.tok_seq), _ptr(batch.seq_slot), _ptr(batch.seq_len), _ptr(lat), *_pages(mem), M,
          _code(d, "latent_prep"),
          _stream())
    return lat


def store(lat: torch.Tensor, batch, mem) -> None:
    """The step's rows to the cache."""
    M, W = lat.shape
    _check_mem(mem, W, lat.dtype, "latent_store")
    _call(_fn("ti_latent_store", [P, I, P, P, P, P, P, P, I, I, I, I, I, I, P]), _ptr(lat), W, _ptr(batch.tok_pos),
          _ptr(batch.tok_seq), _ptr(batch.seq_slot), _ptr(batch.seq_len), *_pages(mem), M, _code(lat, "latent_store"), _stream())


def heads_per_block(n_heads: int, one_token_each: bool) -> int:
    """Heads that share a block's key tiles: as many as fit its 32 rows when every sequence brings one query, else 8
    (4 consecutive queries read nearly the same keys)."""
    cap = 32 if one_token_each else 8
    hb = 1
    while hb < min(n_heads, cap):
        hb <<= 1
    return hb


def decode_splits(n_seq: int, n_heads: int, hb: int, span: int, sms: int) -> int:
    """Blocks that share a sequence's keys when every sequence brings one query: about one block per SM in all (every
    split costs the merging kernel a row of partial sums), a tile of 32 keys each at least, 64 at most."""
    tiles = span // 32 + 2
    groups = (n_heads + hb - 1) // hb
    return max(1, min(sms // max(1, n_seq * groups), tiles, 64))


def plan(n_seq: int, n_heads: int, window: int, plan_len: int, device) -> int:
    """The splits of a step of single tokens planned for ``plan_len`` positions (what of its launches depends on the length)."""
    from .gemm import sm_count
    span = plan_len if window <= 0 else min(plan_len, window)
    return decode_splits(n_seq, n_heads, heads_per_block(n_heads, True), span, sm_count(device))


def prompt_heads(plain: int, rot: int, vdim: int) -> int:
    """The head size (64 or 128) at which a step of whole prompts runs as plain multi-head attention on the tensor cores,
    or 0 when the heads do not fit."""
    need = max(plain + rot, vdim)
    return 64 if need <= 64 else 128 if need <= 128 else 0


def attention_prompt(q: torch.Tensor, lat: torch.Tensor, w_ukv: torch.Tensor, vdim: int, rank: int, rot: int, scale: float,
                     window: int, sink: Optional[torch.Tensor], batch, D: int) -> torch.Tensor:
    """Every sequence starts at position 0, bfloat16: keys and values per head are formed from the step's rows by one product
    with w_ukv = [Wuk; Wuv], packed beside the queries into heads of D elements, and a multi-head attention over the step's own
    tokens runs on the tensor cores.  Returns [M, heads * D]: head h's value in its first ``vdim`` elements, zeros after."""
    from . import linear
    from .lib import library
    M, nh, hd = q.shape
    plain = hd - rot
    ku = linear(lat[:, :rank], w_ukv)                    # [M, heads * plain + heads * vdim]
    Qp = torch.empty((M, nh, D), dtype=q.dtype, device=q.device)
    Kp, Vp, out = torch.empty_like(Qp), torch.empty_like(Qp), torch.empty_like(Qp)
    _call(_fn("ti_latent_pack", [P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, P]), _ptr(q), q.stride(0), _ptr(ku), _ptr(lat),
          _ptr(Qp), _ptr(Kp), _ptr(Vp), M, nh, plain, rot, vdim, rank, D, _code(q, "latent_pack"), _stream())
    _call(_fn("ti_attn_prefill_tc_sink", [P, P, P, P, L, L, L, L, P, I, I, I, I, I, I, F, I, P, P]),
          _ptr(Qp), _ptr(Kp), _ptr(Vp), _ptr(out), nh * D, nh * D, nh * D, nh * D, _ptr(batch.cu_new), batch.n_seq, batch.max_new,
          M, nh, nh, D, float(scale), int(window), _ptr(sink), _stream())
    return out.view(M, nh * D)


def prompt_eligible(q: torch.Tensor, lat: torch.Tensor, rank: int, rot: int, vdim: int, batch) -> int:
    """The head size for attention_prompt, or 0: bfloat16, every sequence at its start, heads that fit, and rows the
    tensor-core product takes (16-byte pieces)."""
    if q.dtype != torch.bfloat16 or batch.mode != "start":
        return 0
    if rank % 8 or (rank + rot) % 8 or lat.data_ptr() % 16:
        return 0
    return prompt_heads(q.shape[2] - rot, rot, vdim)


def single_eligible(q: torch.Tensor, rank: int, rot: int, batch, mem) -> bool:
    """Whether attention_single takes this step: every sequence one token, bfloat16, sizes the tensor-core kernel takes."""
    return (batch.mode == "extend" and q.dtype == torch.bfloat16 and (rank + rot) % 16 == 0 and rank % 8 == 0 and rank <= 512
            and mem.k_pages.dtype == torch.bfloat16 and mem.k_pages.data_ptr() % 16 == 0)


def attention_single(d: torch.Tensor, q: torch.Tensor, rank: int, rot: int, norm_w: torch.Tensor, eps: float, tables,
                     uk: torch.Tensor, uv: torch.Tensor, vdim: int, scale: float, window: int, sink: Optional[torch.Tensor],
                     batch, mem) -> torch.Tensor:
    """A step in which every sequence brings one token, bfloat16, in three launches: the token's row (normed, rotated, stored)
    together with its queries' way into the latent space; the attention over the cached rows on the tensor cores, a
    sequence's keys split over blocks; the splits' merge together with the way out through uv.  d[M, rank + rot] and
    q[M, heads, plain + rot] are the projection's output as it is -> [M, heads * vdim]."""
    _need_cuda(d, q, norm_w, uk, uv, sink, what="latent_attention")
    M, nh, hd = q.shape
    plain, W = hd - rot, rank + rot
    _check_mem(mem, W, q.dtype, "latent_attention")
    cos = sin = None
    max_pos = 0
    if rot:
        cos, sin, dim = tables
        max_pos = cos.shape[0]
        if dim != rot or batch.max_pos_after > max_pos:
            raise KernelError(f"latent_attention: position {batch.max_pos_after - 1} is beyond the rotary tables' {max_pos}")
    lat = torch.empty((M, W), dtype=q.dtype, device=q.device)
    qa = torch.empty((M, nh, W), dtype=torch.float32, device=q.device)
    _call(_fn("ti_latent_prep_absorb", [P, L, P, L, I, I, I, I, P, F, P, P, I, P, P, P, P, P, P, P, I, I, I, I, P, P, I, I, P]),
          _ptr(d), d.stride(0), _ptr(q), q.stride(0), nh, plain, rank, rot, _ptr(norm_w), float(eps), _ptr(cos), _ptr(sin), max_pos,
          _ptr(batch.tok_pos), _ptr(batch.tok_seq), _ptr(batch.seq_slot), _ptr(batch.seq_len), _ptr(lat), *_pages(mem), _ptr(uk),
          _ptr(qa), M, _code(q, "latent_attention"), _stream())
    splits = plan(batch.n_seq, nh, window, batch.plan_len, q.device)
    part_o = torch.empty((M, nh, splits, rank), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((M, nh, splits, 2), dtype=torch.float32, device=q.device)
    o = torch.empty((M, nh * vdim), dtype=q.dtype, device=q.device)
    _call(_fn("ti_latent_decode", [P, P, P, P, P, I, I, I, I, F, I, P, P, P, I, I, I, I, I, P, P, P, P, L, I, P]),
          _ptr(qa), _ptr(lat), _ptr(batch.cu_new), _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seq, nh, rank, rot,
          float(scale), int(window), _ptr(sink), *_pages(mem), splits, _ptr(part_o), _ptr(part_ml), _ptr(uv), _ptr(o), o.stride(0),
          vdim, _stream(), launches=2)
    return o


def attention(q: torch.Tensor, lat: torch.Tensor, uk: torch.Tensor, uv: torch.Tensor, vdim: int, rank: int, rot: int,
              scale: float, window: int, sink: Optional[torch.Tensor], batch, mem) -> torch.Tensor:
    """q[M, heads, plain + rot] (rotated part already rotated), the step's rows lat[M, rank + rot], uk[heads * plain, rank],
    uv[heads * vdim, rank] -> [M, heads * vdim].  Keys at positions below a sequence's start come from ``mem``."""
    _need_cuda(q, lat, uk, uv, sink, what="latent_attention")
    M, nh, hd = q.shape
    plain, W = hd - rot, rank + rot
    if lat.shape != (M, W) or not lat.is_contiguous() or lat.dtype != q.dtype:
        raise KernelError("latent_attention: the step's rows do not fit the queries")
    if uk.shape != (nh * plain, rank) or uv.shape != (nh * vdim, rank) or not uk.is_contiguous() or not uv.is_contiguous() \
            or uk.dtype != q.dtype or uv.dtype != q.dtype:
        raise KernelError("latent_attention: the up-projections do not fit")
    if sink is not None and (sink.dtype != torch.float32 or sink.shape != (nh,) or not sink.is_contiguous()):
        raise KernelError("latent_attention: sinks must be float32 [heads]")
    _check_mem(mem, W, q.dtype, "latent_attention")
    code = _code(q, "latent_attention")
    qa = torch.empty((M, nh, W), dtype=torch.float32, device=q.device)
    _call(_fn("ti_latent_absorb", [P, L, P, P, I, I, I, I, I, I, P]), _ptr(q), q.stride(0), _ptr(uk), _ptr(qa), M, nh, plain,
          rank, rot, code, _stream())
    ol = torch.empty((M, nh, rank), dtype=torch.float32, device=q.device)
    hb = heads_per_block(nh, batch.mode == "extend")
    splits, part_o, part_ml = 1, None, None
    if batch.mode == "extend":
        splits = plan(batch.n_seq, nh, window, batch.plan_len, q.device)
        if splits > 1:
            part_o = torch.empty((M, nh, splits, rank), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((M, nh, splits, 2), dtype=torch.float32, device=q.device)
    _call(_fn("ti_latent_attn", [P, P, P, P, P, P, I, I, I, I, I, I, F, I, P, P, P, I, I, I, I, I, P, P, I, I, P]),
          _ptr(qa), _ptr(lat), _ptr(ol), _ptr(batch.cu_new), _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seq,
          batch.max_new, nh, hb, rank, rot, float(scale), int(window), _ptr(sink), *_pages(mem), splits, _ptr(part_o),
          _ptr(part_ml), M, code, _stream(), launches=2 if splits > 1 else 1)
    o = torch.empty((M, nh * vdim), dtype=q.dtype, device=q.device)
    _call(_fn("ti_latent_expand", [P, P, P, L, I, I, I, I, I, P]), _ptr(ol), _ptr(uv), _ptr(o), o.stride(0), M, nh, vdim, rank,
          code, _stream())
    return o
