"""A layer whose mixer and feed-forward read the same normed input.

n = norm(h);  h <- h + (mixer(n) + ffn(n)).  One norm per layer; the two outputs stay pending
as a pair and the next norm (the next layer's, or the head's) forms the sum, so that the
stream is read and written once per layer.  The feed-forward may be absent.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Block, BuildContext, ParamSpec, PartSpec, build_part, register_part


class ParallelBlock(Block):
    def __init__(self, ctx: BuildContext, prefix: str, norm: PartSpec, mixer: PartSpec,
                 feed_forward: Optional[PartSpec] = None, names: Optional[Dict[str, str]] = None):
        n = {"norm": "", "mixer": "mix.", "feed_forward": "mlp."}
        n.update(names or {})
        self.norm = build_part("norm", norm, ctx, prefix + n["norm"])
        self.mixer = build_part("mixer", mixer, ctx, prefix + n["mixer"])
        self.feed_forward = build_part("feed_forward", feed_forward, ctx, prefix + n["feed_forward"]) \
            if feed_forward is not None else None
        self._children = tuple(c for c in (self.norm, self.mixer, self.feed_forward) if c is not None)

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for c in self._children:
            out.update(c.param_specs())
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for c in self._children:
            c.bind(tensors)

    def check_kernels(self, dtype) -> None:
        for c in self._children:
            c.check_kernels(dtype)

    @property
    def captures_start(self) -> bool:
        return bool(self.mixer.captures_start and (self.feed_forward is None or self.feed_forward.captures_start))

    def forward(self, h, delta, batch, mem, shared):
        trace = getattr(batch, "trace", None)
        x = self.norm.add_forward(h, delta)
        if trace is not None and trace.active:
            with trace.range("layer.attn_block"):
                a = self.mixer.forward(x, batch, mem, shared)
            with trace.range("layer.mlp_block"):
                m = self.feed_forward.forward(x, batch) if self.feed_forward is not None else None
        else:
            a = self.mixer.forward(x, batch, mem, shared)
            m = self.feed_forward.forward(x, batch) if self.feed_forward is not None else None
        return h, (a if m is None else (a, m))


register_part("block", "parallel", ParallelBlock)
