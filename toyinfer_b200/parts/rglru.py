"""The recurrent block of Griffin (De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for
Efficient Language Models"): two branches of ``width`` channels around a real-gated linear recurrent unit.

Per token x:  z = gelu_tanh(Wy x + by);  c = conv(Wx x + bx), a short causal convolution per channel with a bias;
the channels are cut into ``blocks`` parts, each with two square gate matrices of its own:
r = sigmoid(Ra c + ra), i = sigmoid(Ri c + ri);  a = exp(-8 softplus(lam) r);
S <- a S + sqrt(1 - a^2) (i c)   (float32, zero when the sequence starts);  y = Wo (S z).

What a sequence carries, one float32 row per slot (``StateRequest``): the convolution's last ``conv - 1`` inputs
[conv - 1, width], then S [width].  Both branches come from one product; each gate block's two matrices are one
product with float32 logits; the convolution, and the recurrence with both activations, are a kernel each
(kernels/recurrent.py).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from ..kernels import recurrent as KR
from ..tracing import ranged
from .base import BuildContext, Mixer, ParamSpec, StateRequest, register_part


class RGLRUBlock(Mixer):
    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, width: int, blocks: int, conv: int, rate_scale: float = 8.0,
                 names: Optional[Dict[str, str]] = None):
        self.ctx, self.hidden = ctx, ctx.hidden_size
        self.width, self.blocks, self.taps = int(width), int(blocks), int(conv)
        self.rate_scale = float(rate_scale)
        if self.blocks < 1 or self.width % self.blocks:
            raise ValueError(f"rglru at {prefix!r}: {self.width} channels do not cut into {self.blocks} equal gate blocks")
        if self.taps < 1:
            raise ValueError(f"rglru at {prefix!r}: a convolution of {self.taps} taps")
        n = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b", "gate_r": "ra",
             "gate_r_bias": "ra.b", "gate_i": "ri", "gate_i_bias": "ri.b", "lam": "lam", "o": "o"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.state_conv = 0
        self.state_s = (self.taps - 1) * self.width

    def param_specs(self) -> Dict[str, ParamSpec]:
        C, nb, bs = self.width, self.blocks, self.width // self.blocks
        small = lambda shape, **kw: ParamSpec(shape, role="norm", init="normal", **kw)
        return {
            self.names["y"]: ParamSpec((C, self.hidden), std=0.05), self.names["y_bias"]: small((C,), std=0.1),
            self.names["x"]: ParamSpec((C, self.hidden), std=0.05), self.names["x_bias"]: small((C,), std=0.1),
            self.names["conv"]: small((C, self.taps), std=0.4), self.names["conv_bias"]: small((C,), std=0.1),
            self.names["gate_r"]: ParamSpec((nb, bs, bs), std=0.2), self.names["gate_r_bias"]: small((nb, bs), std=0.3),
            self.names["gate_i"]: ParamSpec((nb, bs, bs), std=0.2), self.names["gate_i_bias"]: small((nb, bs), std=0.3),
            self.names["lam"]: small((C,), std=1.0, mean=-1.0),
            self.names["o"]: ParamSpec((self.hidden, C), std=0.05),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        t = lambda k: tensors.pop(self.names[k])
        f32 = lambda k: t(k).to(torch.float32).contiguous()
        self.w_in = torch.cat([t("x"), t("y")], dim=0).contiguous()                    # rows: conv branch, then gelu branch
        self.b_x, self.b_y = f32("x_bias"), f32("y_bias")
        self.conv_w, self.conv_b = f32("conv"), f32("conv_bias")
        # a gate block's two matrices as one [2 bs, bs] matrix: recurrence gate's rows, then the input gate's
        self.w_gates = torch.cat([t("gate_r"), t("gate_i")], dim=1).contiguous()
        self.b_r, self.b_i = f32("gate_r_bias").reshape(-1), f32("gate_i_bias").reshape(-1)
        self.rate = (self.rate_scale * torch.nn.functional.softplus(f32("lam"))).contiguous()
        self.w_o = t("o").contiguous()

    def memory_request(self):
        return StateRequest((self.taps * self.width,), torch.float32)

    def launch_plan(self, n_seq: int, plan_len: int, dtype, device, n_live=None):
        return ("rglru",)

    def forward(self, x, batch, mem, shared) -> torch.Tensor:
        if mem is None or not hasattr(mem, "state"):
            raise RuntimeError("a recurrent block needs a state; the schedule gave it none")
        C, bs = self.width, self.width // self.blocks
        with ranged(batch, "mixer.qkv"):
            xy = K.linear(x, self.w_in)
            u = KR.short_conv(xy[:, :C], self.conv_w, mem.state, self.state_conv, batch, in_bias=self.b_x, out_bias=self.conv_b)
            gates = KR.block_diag_linear(u, self.w_gates)
        with ranged(batch, "mixer.attention"):
            s = KR.rglru_scan(gates, u, xy[:, C:], self.b_r, self.b_i, self.b_y, self.rate, bs, mem.state, self.state_s, batch)
        with ranged(batch, "mixer.out"):
            return K.linear(s, self.w_o)


register_part("mixer", "rglru", RGLRUBlock)
