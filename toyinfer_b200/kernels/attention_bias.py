"""Attention with a soft cap and a bias by distance, keys and values of different sizes (csrc/attn_bias.cu)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import KernelError, _call, _code, _need_cuda, _ptr, _stream
from .gemm import sm_count
from .wide import _fn

P, I, L, F = c_void_p, c_int, c_longlong, c_float


def _pages(mem, dtype, n_kv: int, dim: int, vdim: int, what: str):
    kp, vp, pt = mem.k_pages, mem.v_pages, mem.page_table
    if vp is None or mem.ring_rows:
        raise KernelError(f"{what}: needs keys and values of all positions (no ring, a value array)")
    if kp.dtype != dtype or vp.dtype != dtype or tuple(kp.shape[1:]) != (n_kv, mem.page_size, dim) \
            or tuple(vp.shape[1:]) != (n_kv, mem.page_size, vdim) or not kp.is_contiguous() or not vp.is_contiguous():
        raise KernelError(f"{what}: the cache pages do not fit {n_kv} kv heads of {dim} and {vdim} elements in {dtype}")
    return _ptr(kp), _ptr(vp), _ptr(pt), pt.shape[1], mem.page_size, kp.shape[0]


def prepare(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
            n_heads: int, n_kv: int, dim: int, vdim: int, mem, batch) -> None:
    """qkv [M, heads * dim + kv_heads * (dim + vdim)], one projection's rows: adds ``bias`` (float32, a row long), norms the
    query and key heads (weights float32 [dim] or None), leaves the queries in place and stores keys and values in ``mem``."""
    _need_cuda(qkv, bias, q_w, k_w, what="attention_bias.prepare")
    M, N = qkv.shape
    if N != n_heads * dim + n_kv * (dim + vdim) or qkv.stride(1) != 1:
        raise KernelError("attention_bias.prepare: the projection's rows do not fit the heads")
    for t, n in ((bias, N), (q_w, dim), (k_w, dim)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
            raise KernelError("attention_bias.prepare: biases and norm weights must be dense float32")
    _call(_fn("ti_attn_bias_prepare", [P, L, P, P, P, F, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P]),
          _ptr(qkv), qkv.stride(0), _ptr(bias), _ptr(q_w), _ptr(k_w), float(eps), _ptr(batch.tok_pos), _ptr(batch.tok_seq),
          _ptr(batch.seq_slot), *_pages(mem, qkv.dtype, n_kv, dim, vdim, "attention_bias.prepare"), M, n_heads, n_kv, dim, vdim,
          _code(qkv, "attention_bias"), _stream())


def decode_splits(n_seq: int, n_heads: int, n_kv_heads: int, plan_len: int, sms: int) -> int:
    """Ranges that a single query's keys are cut into, so that the step has about four blocks per SM but no range
    shorter than 128 keys: depends only on the batch's padded size and the length the step was planned for.  (A block
    takes up to four query heads of a kv head: csrc/attn_bias.cu.)"""
    group = n_heads // n_kv_heads
    per_block = 4 if group % 4 == 0 else 2 if group % 2 == 0 else 1
    want = max(1, (4 * sms) // max(1, n_seq * n_heads // per_block))
    return max(1, min(want, (plan_len + 127) // 128, 64))


tensor_cores = True          # tests clear this to run prompts and pieces on the CUDA-core kernel whatever their sizes


def attend(q: torch.Tensor, vdim: int, mem, scale: float, cap: float, dist_bias: Optional[torch.Tensor], batch,
           k: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [M, heads, dim] (normed) over the keys and values that ``mem`` holds, the step's own included -> [M, heads * vdim].
    dist_bias: float32 [heads, far + 1], the bias of every distance up to ``far`` (all further ones share the last).
    k, v: the step's own keys [M, kv_heads, dim] and values [M, kv_heads, vdim] as they were stored, for the
    tensor-core kernel (bfloat16, heads of 64 or 128 elements for keys and values alike)."""
    _need_cuda(q, dist_bias, what="attention_bias")
    M, H, dim = q.shape
    if q.stride(2) != 1 or q.stride(1) != dim:
        raise KernelError("attention_bias: heads of a token must be dense")
    far = 0
    if dist_bias is not None:
        if dist_bias.dtype != torch.float32 or dist_bias.dim() != 2 or dist_bias.shape[0] != H or not dist_bias.is_contiguous():
            raise KernelError("attention_bias: the distance table must be dense float32 [heads, far + 1]")
        far = dist_bias.shape[1] - 1
    pages = _pages(mem, q.dtype, mem.n_kv_heads, dim, vdim, "attention_bias")
    out = torch.zeros((M, H * vdim), dtype=q.dtype, device=q.device)
    code = _code(q, "attention_bias")
    if batch.mode == "extend":
        splits = decode_splits(M, H, mem.n_kv_heads, batch.plan_len, sm_count(q.device))
        part_o = part_ml = None
        if splits > 1:
            part_o = torch.empty((M, H, splits, vdim), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((M, H, splits, 2), dtype=torch.float32, device=q.device)
        _call(_fn("ti_attn_bias_decode", [P, L, P, L, P, P, I, P, P, P, I, I, I, P, I, I, I, I, I, F, F, I, P, P, I, P]),
              _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(batch.seq_len), _ptr(batch.seq_slot), M, *pages, _ptr(dist_bias),
              far, H, mem.n_kv_heads, dim, vdim, float(scale), float(cap), splits, _ptr(part_o), _ptr(part_ml), code, _stream(),
              launches=2 if splits > 1 else 1)
        return out
    G = mem.n_kv_heads
    if tensor_cores and q.dtype == torch.bfloat16 and dim == vdim and dim in (64, 128) and k is not None and mem.page_size == 64 \
            and all(t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 for t in (q, k, v, out)) and scale > 0:
        # whole prompts and pieces on tcgen05: the kernel of the other attention mixers, told of cap and table
        # (csrc/attn_prefill_tc.cu); it reads the step's own keys and values beside the pages
        if batch.mode == "start":
            _call(_fn("ti_attn_prefill_tc_bias", [P, P, P, P, L, L, L, L, P, I, I, I, I, I, I, F, F, P, I, P]),
                  _ptr(q), _ptr(k), _ptr(v), _ptr(out), q.stride(0), k.stride(0), v.stride(0), out.stride(0), _ptr(batch.cu_new),
                  batch.n_seq, batch.max_new, M, H, G, dim, float(scale), float(cap), _ptr(dist_bias), far, _stream())
        else:
            _call(_fn("ti_attn_chunk_tc_bias", [P, P, P, P, L, L, L, L, P, P, P, I, I, I, I, I, I, F, P, P, P, I, I, I, F, P, I, P]),
                  _ptr(q), _ptr(k), _ptr(v), _ptr(out), q.stride(0), k.stride(0), v.stride(0), out.stride(0), _ptr(batch.cu_new),
                  _ptr(batch.seq_start), _ptr(batch.seq_slot), batch.n_seq, batch.max_new, M, H, G, dim, float(scale), *pages,
                  float(cap), _ptr(dist_bias), far, _stream())
        return out
    _call(_fn("ti_attn_bias", [P, L, P, L, P, P, P, I, I, P, P, P, I, I, I, P, I, I, I, I, I, F, F, I, P]),
          _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(batch.cu_new), _ptr(batch.seq_start), _ptr(batch.seq_slot),
          batch.n_seq, batch.max_new, *pages, _ptr(dist_bias), far, H, mem.n_kv_heads, dim, vdim, float(scale), float(cap), code,
          _stream())
    return out
