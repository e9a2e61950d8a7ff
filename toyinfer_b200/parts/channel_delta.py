"""Linear attention by the gated delta rule with a decay per key channel, short convolutions and a gated output.

Per token x: q = silu(conv(Wq x)), k = silu(conv(Wk x)) [qk_heads, dim], v = silu(conv(Wv x)) [heads, vdim], each through a
causal convolution over time per channel (no bias); q and k are made unit vectors per head, q also times dim^-1/2;
beta = sigmoid(Wb x) per head; g = exp(-exp(A_h) softplus(Wa2 Wa1 x + dt)) per head and key channel.  Per head, with a
state S [dim, vdim] carried from token to token in float32 (zero when the sequence starts), in this order:

    S <- diag(g) S;   e = beta (v - S^T k);   S <- S + k e^T;   o = S^T q

(value head h with query/key head h // (heads / qk_heads)); then o / rms(o) per head times a weight [vdim] shared by the
heads, times sigmoid(Wg2 Wg1 x), and Wo.

What a sequence carries, one float32 row per slot (``StateRequest``): the convolutions' last ``conv - 1`` inputs over all
of q, k and v's channels, then S [heads, dim, vdim].  q, k, v, the two low-rank projections' first halves and beta come
from one product (every part's rows start at a multiple of 8, so that the later products read aligned rows).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..kernels import recurrent as KR
from ..tracing import ranged
from .base import BuildContext, Mixer, ParamSpec, StateRequest, register_part


def _up8(n: int) -> int:
    return (n + 7) // 8 * 8


class ChannelDeltaAttention(Mixer):
    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_heads: int, n_qk_heads: int, dim: int, vdim: int, conv: int, eps: float,
                 decay_rank: int = 0, gate_rank: int = 0, names: Optional[Dict[str, str]] = None):
        if n_heads % n_qk_heads:
            raise ValueError(f"{n_heads} value heads cannot share {n_qk_heads} query/key heads evenly")
        self.ctx, self.hidden = ctx, ctx.hidden_size
        self.n_heads, self.n_qk, self.dim, self.vdim, self.taps = int(n_heads), int(n_qk_heads), int(dim), int(vdim), int(conv)
        self.eps = float(eps)
        n = {"q": "q", "k": "k", "v": "v", "conv": ".conv", "beta": "b", "rate": "A_log", "norm": "norm", "decay_in": "a1",
             "decay_out": "a2", "decay_bias": "dt_bias", "gate_in": "g1", "gate_out": "g2", "o": "o"}
        n.update(names or {})
        self.n, self.prefix = n, prefix
        self.channels = 2 * self.n_qk * self.dim + self.n_heads * self.vdim
        self.state_conv = 0
        self.state_s = (self.taps - 1) * self.channels
        # the low ranks come with the checkpoint's shapes; these are the ones random weights are drawn with
        self.rank_a = int(decay_rank) or max(8, self.dim // 2)
        self.rank_g = int(gate_rank) or max(8, self.dim // 2)

    def _name(self, k: str) -> str:
        return self.prefix + self.n[k]

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, G, d, vd, hid = self.n_heads, self.n_qk, self.dim, self.vdim, self.hidden
        ra, rg = self.rank_a, self.rank_g
        small = lambda shape, **kw: ParamSpec(shape, role="norm", init="normal", **kw)
        conv = self.n["conv"]
        return {
            self._name("q"): ParamSpec((G * d, hid), std=0.1), self._name("q") + conv: small((G * d, self.taps), std=0.5),
            self._name("k"): ParamSpec((G * d, hid), std=0.1), self._name("k") + conv: small((G * d, self.taps), std=0.5),
            self._name("v"): ParamSpec((H * vd, hid), std=0.1), self._name("v") + conv: small((H * vd, self.taps), std=0.5),
            self._name("beta"): ParamSpec((H, hid), std=0.1), self._name("rate"): small((H,), std=0.5),
            self._name("norm"): ParamSpec((vd,), role="norm", init="one_plus_normal", std=0.1),
            self._name("decay_in"): ParamSpec((ra, hid), std=0.1, free=(0,)),
            self._name("decay_out"): ParamSpec((H * d, ra), std=0.3, free=(1,)),
            self._name("decay_bias"): small((H * d,), std=1.0),
            self._name("gate_in"): ParamSpec((rg, hid), std=0.1, free=(0,)),
            self._name("gate_out"): ParamSpec((H * vd, rg), std=0.3, free=(1,)),
            self._name("o"): ParamSpec((hid, H * vd), std=0.05),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = lambda k: tensors.pop(self._name(k))
        f32 = lambda name: tensors.pop(name).to(torch.float32).contiguous()
        conv = self.n["conv"]
        self.conv_w = torch.cat([f32(self._name(k) + conv) for k in ("q", "k", "v")], dim=0).contiguous()
        parts = [torch.cat([t("q"), t("k"), t("v")], dim=0), t("decay_in"), t("gate_in"), t("beta")]
        self.rank_a, self.rank_g = parts[1].shape[0], parts[2].shape[0]
        rows, self.cols = [], []
        at = 0
        for p in parts:                      # every part starts at a multiple of 8 rows
            pad = _up8(at) - at
            if pad:
                rows.append(torch.zeros((pad, self.hidden), dtype=p.dtype, device=p.device))
            at += pad
            self.cols.append(at)
            rows.append(p)
            at += p.shape[0]
        if _up8(at) > at:                    # ... and a token's row of results is a multiple of 8 long
            rows.append(torch.zeros((_up8(at) - at, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_decay = t("decay_out").contiguous()
        self.w_gate = t("gate_out").contiguous()
        if self.w_decay.shape[1] != self.rank_a or self.w_gate.shape[1] != self.rank_g:
            raise ValueError(f"delta rule at {self.prefix!r}: the two halves of a low-rank projection differ in rank")
        self.dt_bias = f32(self._name("decay_bias"))
        self.rate = torch.exp(f32(self._name("rate"))).contiguous()
        self.norm_w = f32(self._name("norm"))
        self.w_o = t("o").contiguous()

    def check_kernels(self, dtype) -> None:
        if self.dim > 128:
            raise K.KernelError(f"delta rule: heads of {self.dim} query/key elements are not supported (up to 128)")
        if self.taps > 8:
            raise K.KernelError(f"short convolution: {self.taps} taps are not supported (up to 8)")

    def memory_request(self):
        return StateRequest((self.state_s + self.n_heads * self.dim * self.vdim,), torch.float32)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return ("delta",)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if mem is None or not hasattr(mem, "state"):
            raise RuntimeError("a delta-rule mixer needs a state; the schedule gave it none")
        H, G, d, vd = self.n_heads, self.n_qk, self.dim, self.vdim
        c_qkv, c_a, c_g, c_b = self.cols
        with ranged(batch, "mixer.qkv"):
            y = K.linear(x, self.w_in)
            M = y.shape[0]
            u = KR.short_conv(y[:, c_qkv:c_qkv + self.channels], self.conv_w, mem.state, self.state_conv, batch, act="silu")
            decay_logit = K.linear(y[:, c_a:c_a + self.rank_a], self.w_decay, out_dtype=torch.float32)
            gate_logit = K.linear(y[:, c_g:c_g + self.rank_g], self.w_gate)
        q = u[:, :G * d].view(M, G, d)
        k = u[:, G * d:2 * G * d].view(M, G, d)
        v = u[:, 2 * G * d:].view(M, H, vd)
        with ranged(batch, "mixer.attention"):
            o = KR.delta_rule(q, k, v, decay_logit, self.dt_bias, self.rate, y[:, c_b:c_b + H], mem.state, self.state_s, batch)
            a = KR.head_gated_rmsnorm(o, gate_logit, self.norm_w, H, self.eps)
        with ranged(batch, "mixer.out"):
            return K.linear(a, self.w_o)


register_part("mixer", "channel_delta", ChannelDeltaAttention)
