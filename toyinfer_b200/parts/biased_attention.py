"""Grouped-query attention without rotation: positions enter through a learned bias by distance.

For each token x: q = Wq x + bq [heads, dim], k = Wk x + bk [kv_heads, dim], v = Wv x + bv [kv_heads, vdim]; q and k
normed per head over dim (plain weight [dim] shared by the heads); query head h reads kv head h // (heads / kv_heads);

    s_ij = (q_i . k_j) * scale;   s_ij <- softcap * tanh(s_ij / softcap);   s_ij <- s_ij + table[bucket(i - j), h]

over the keys j <= i, ordinary softmax, weighted sum of v, then o = Wo a + bo.  The table has B rows; with
half = B // 2 and ``bias_max`` = D:  bucket(n) = n below half, else min(B - 1, half + floor(ln(n / half) / ln(D / half)
* (B - half))): exact for near keys, logarithmic steps further out, one row for everything from about D on.  The
bucket of every distance up to D is looked up once when the weights are bound ([heads, D + 1], float32); the
kernels index it with min(i - j, D).  Soft cap, table and biases are each optional.

Keys and values of all positions live in the cache (``KVRequest`` with a value size of its own); a step first
stores its own, then attends over the pages, whatever mix of new and cached tokens it brings (kernels/attention_bias.py).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import kernels as K
from ..kernels import attention_bias as KA
from ..kernels.gemm import sm_count
from ..tracing import ranged
from .base import BuildContext, KVRequest, Mixer, ParamSpec, register_part


def distance_buckets(n_rows: int, far: float) -> torch.Tensor:
    """int64 [ceil(far) + 1]: the table row of every distance 0 .. ceil(far)."""
    half = n_rows // 2
    last = max(int(math.ceil(far)), half, 1)
    out = []
    for n in range(last + 1):
        if n < half or half == 0:
            out.append(min(n, n_rows - 1))
        else:
            out.append(min(n_rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (n_rows - half)))))
    return torch.tensor(out, dtype=torch.int64)


class BiasedAttention(Mixer):
    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, softcap: float = 0.0, bias_rows: int = 0, bias_max: float = 0.0, qk_norm: bool = True,
                 biases: bool = True, names: Optional[Dict[str, str]] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads evenly")
        self.ctx, self.hidden = ctx, ctx.hidden_size
        self.n_heads, self.n_kv, self.dim, self.vdim = int(n_heads), int(n_kv_heads), int(dim), int(vdim)
        self.scale, self.eps, self.softcap = float(scale), float(eps), float(softcap)
        self.bias_rows, self.bias_max = int(bias_rows), float(bias_max)
        if self.bias_rows and not self.bias_max > max(self.bias_rows // 2, 1):
            raise ValueError(f"attention at {prefix!r}: a table of {self.bias_rows} rows needs bias_max above {self.bias_rows // 2}")
        self.qk_norm, self.biases = bool(qk_norm), bool(biases)
        n = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "table": "rel", "bias": ".b"}
        n.update(names or {})
        self.n, self.prefix = n, prefix
        self.w_qkv = self.w_o = self.b_qkv = self.b_o = self.q_w = self.k_w = self.dist_bias = None

    def _name(self, k: str, bias: bool = False) -> str:
        return self.prefix + self.n[k] + (self.n["bias"] if bias else "")

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, G, d, vd = self.n_heads, self.n_kv, self.dim, self.vdim
        s = {self._name("q"): ParamSpec((H * d, self.hidden), std=0.05), self._name("k"): ParamSpec((G * d, self.hidden), std=0.05),
             self._name("v"): ParamSpec((G * vd, self.hidden), std=0.05), self._name("o"): ParamSpec((self.hidden, H * vd), std=0.05)}
        if self.biases:
            for k, rows in (("q", H * d), ("k", G * d), ("v", G * vd), ("o", self.hidden)):
                s[self._name(k, True)] = ParamSpec((rows,), role="norm", init="normal", std=0.1)
        if self.qk_norm:
            s[self._name("q_norm")] = ParamSpec((d,), role="norm", init="one_plus_normal", std=0.1)
            s[self._name("k_norm")] = ParamSpec((d,), role="norm", init="one_plus_normal", std=0.1)
        if self.bias_rows:
            # (how many rows the table has is the checkpoint's matter)
            s[self._name("table")] = ParamSpec((self.bias_rows, H), role="norm", init="normal", std=1.0, free=(0,))
        return s

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = lambda name: tensors.pop(name)
        f32 = lambda name: t(name).to(torch.float32).contiguous()
        self.w_qkv = torch.cat([t(self._name(k)) for k in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = t(self._name("o")).contiguous()
        if self.biases:
            self.b_qkv = torch.cat([f32(self._name(k, True)) for k in ("q", "k", "v")]).contiguous()
            self.b_o = f32(self._name("o", True))
        if self.qk_norm:
            self.q_w, self.k_w = f32(self._name("q_norm")), f32(self._name("k_norm"))
        if self.bias_rows:
            table = f32(self._name("table"))                                     # [rows, heads]
            self.bias_rows = table.shape[0]
            if not self.bias_max > max(self.bias_rows // 2, 1):
                raise ValueError(f"attention at {self.prefix!r}: a table of {self.bias_rows} rows needs bias_max above {self.bias_rows // 2}")
            rows = distance_buckets(self.bias_rows, self.bias_max).to(table.device)
            self.dist_bias = table[rows].T.contiguous()                          # [heads, far + 1]

    def check_kernels(self, dtype) -> None:
        if max(self.dim, self.vdim) > 256:
            raise K.KernelError(f"attention: heads of {self.dim} and {self.vdim} elements are not supported (up to 256)")

    def memory_request(self):
        return KVRequest(self.n_kv, self.dim, 0, True, self.vdim if self.vdim != self.dim else 0)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return ("biased", KA.decode_splits(n_seq, self.n_heads, self.n_kv, plan_len, sm_count(device)))

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if mem is None or not hasattr(mem, "k_pages"):
            raise RuntimeError("attention needs key/value memory; the schedule gave it none")
        H, d = self.n_heads, self.dim
        with ranged(batch, "mixer.qkv"):
            qkv = K.linear(x, self.w_qkv)
        M = qkv.shape[0]
        with ranged(batch, "mixer.attention"):
            KA.prepare(qkv, self.b_qkv, self.q_w, self.k_w, self.eps, H, self.n_kv, d, self.vdim, mem, batch)
            G, vd = self.n_kv, self.vdim
            a = KA.attend(qkv[:, :H * d].view(M, H, d), vd, mem, self.scale, self.softcap, self.dist_bias, batch,
                          k=qkv[:, H * d:(H + G) * d].view(M, G, d), v=qkv[:, (H + G) * d:].view(M, G, vd))
        with ranged(batch, "mixer.out"):
            return K.linear_bias(a, self.w_o, self.b_o)


register_part("mixer", "biased_attention", BiasedAttention)
