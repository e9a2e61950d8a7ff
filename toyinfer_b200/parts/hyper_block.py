"""A pre-norm layer over several residual streams ("hyper-connections") with a scale per channel on each sublayer.

A token's hidden state is X [streams, width], float32.  Each of the two sublayers (mixer, then feed-forward; the
second may be absent) has three small tensors: ``in`` [streams], ``mix`` [streams, streams] indexed [from, to] and
``out`` [streams], and a scale ``ls`` [width]:

    u = sum_s in[s] X_s;   y = ls * sublayer(norm(u));   X_t <- sum_s mix[s, t] X_s + out[t] y    (all t from the old X)

With ``connections=False`` there are no such tensors and one stream: X <- X + ls * sublayer(norm(X)).  The update a
sublayer leaves is not applied at once: it stays pending (kernels.hyper.StreamUpdate) and the norm that reads the
streams next (this layer's second, the next layer's first, the head's) applies it in the same kernel, so that the
streams are read and written once per sublayer.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels.hyper import StreamUpdate
from .base import Block, BuildContext, ParamSpec, PartSpec, build_part, register_part


class HyperBlock(Block):
    def __init__(self, ctx: BuildContext, prefix: str, norm: PartSpec, mixer: PartSpec, feed_forward: Optional[PartSpec] = None,
                 streams: int = 1, connections: bool = True, layer_scale: bool = True, names: Optional[Dict[str, str]] = None):
        n = {"norm1": "norm1", "norm2": "norm2", "mixer": "mix.", "feed_forward": "mlp.", "scale1": "ls1", "scale2": "ls2",
             "conn1": "hc1.", "conn2": "hc2."}
        n.update(names or {})
        self.hidden, self.streams = ctx.hidden_size, int(streams)
        self.connections, self.layer_scale = bool(connections), bool(layer_scale)
        if not self.connections and self.streams != 1:
            raise ValueError(f"layer at {prefix!r}: {self.streams} streams need connection tensors")

        def norm_spec(name):
            p = dict(norm.params)
            p.update(name=name, streams=self.streams)
            return PartSpec(norm.kind, p)

        self.norm1 = build_part("norm", norm_spec(n["norm1"]), ctx, prefix)
        self.mixer = build_part("mixer", mixer, ctx, prefix + n["mixer"])
        self.feed_forward = self.norm2 = None
        if feed_forward is not None:
            self.norm2 = build_part("norm", norm_spec(n["norm2"]), ctx, prefix)
            self.feed_forward = build_part("feed_forward", feed_forward, ctx, prefix + n["feed_forward"])
        self._children = tuple(c for c in (self.norm1, self.norm2, self.mixer, self.feed_forward) if c is not None)
        self.prefix, self.n = prefix, n
        self.consts: Dict[str, Optional[torch.Tensor]] = {}

    def _sublayers(self):
        return (1, 2) if self.feed_forward is not None else (1,)

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for c in self._children:
            out.update(c.param_specs())
        S = self.streams
        for q in self._sublayers():
            if self.layer_scale:
                out[self.prefix + self.n[f"scale{q}"]] = ParamSpec((self.hidden,), role="norm", init="normal", mean=0.5, std=0.1)
            if self.connections:
                c = self.prefix + self.n[f"conn{q}"]
                # (drawn near a plain residual sum: streams that are carried as they are, read evenly, written alike)
                out[c + "in"] = ParamSpec((S,), role="norm", init="normal", mean=1.0 / S, std=0.1 / S)
                out[c + "out"] = ParamSpec((S,), role="norm", init="normal", mean=1.0, std=0.2)
                out[c + "mix"] = ParamSpec((S, S), role="norm", init="eye_plus_normal", std=0.1)
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for c in self._children:
            c.bind(tensors)
        f32 = lambda name: tensors.pop(name).to(torch.float32).contiguous()
        for q in self._sublayers():
            self.consts[f"gain{q}"] = f32(self.prefix + self.n[f"scale{q}"]) if self.layer_scale else None
            c = self.prefix + self.n[f"conn{q}"]
            for k in ("in", "out", "mix"):
                self.consts[f"{k}{q}"] = f32(c + k) if self.connections else None

    def check_kernels(self, dtype) -> None:
        from .. import kernels as K
        if not 1 <= self.streams <= 8:
            raise K.KernelError(f"{self.streams} residual streams are not supported (1 to 8)")
        for c in self._children:
            c.check_kernels(dtype)

    @property
    def captures_start(self) -> bool:
        return bool(self.mixer.captures_start and (self.feed_forward is None or self.feed_forward.captures_start))

    def _pending(self, q: int, y: torch.Tensor) -> StreamUpdate:
        c = self.consts
        return StreamUpdate(y, c[f"gain{q}"], c[f"mix{q}"], c[f"out{q}"])

    def forward(self, h, delta, batch, mem, shared):
        trace = getattr(batch, "trace", None)
        timed = trace is not None and trace.active
        x = self.norm1.read_forward(h, delta, self.consts["in1"])
        if timed:
            with trace.range("layer.attn_block"):
                a = self.mixer.forward(x, batch, mem, shared)
        else:
            a = self.mixer.forward(x, batch, mem, shared)
        pending = self._pending(1, a)
        if self.feed_forward is None:
            return h, pending
        x = self.norm2.read_forward(h, pending, self.consts["in2"])
        if timed:
            with trace.range("layer.mlp_block"):
                m = self.feed_forward.forward(x, batch)
        else:
            m = self.feed_forward.forward(x, batch)
        return h, self._pending(2, m)


register_part("block", "hyper", HyperBlock)
