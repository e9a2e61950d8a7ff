"""Tusasun: the description of the model in terms of parts.

A pre-norm decoder over several float32 residual streams per token (hyper-connections), every sublayer's output under
a scale per channel, norms with a weight stored around zero; mixers are a Griffin-style recurrent block (real-gated
linear recurrent unit), attention without rotation (soft-capped scores plus a learned bias by distance, biases on the
projections, normed queries and keys) or a gated delta rule with a decay per key channel; feed-forwards are mixtures
of squared-ReLU experts chosen by sigmoid scores that scale the expert's input, beside a gated shared expert; a span of
layers may run several times with the same weights and memory of its own per pass; the head is a matrix of its own
behind the final norm of the streams' sum.  Tensor names: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.hc1.*``, ``l<i>.hc2.*``, ``l<i>.mix.*``, ``l<i>.mlp.*``.  Nothing here computes: the parts do.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tusasun import TusasunConfig
from ..parts.base import PartSpec
from ..parts.model import LayerSpec, ModelSpec, ScheduleEntry


def describe_tusasun(cfg: TusasunConfig) -> ModelSpec:
    eps = cfg.eps
    streams = cfg.streams if cfg.streams is not None else 1
    norm = PartSpec("stream_rmsnorm", {"size": cfg.width, "eps": eps, "streams": streams, "one_plus": True})
    layers = []
    for i, L in enumerate(cfg.layers):
        m = L["mixer"]
        if L["type"] == "rglru":
            mixer = PartSpec("rglru", {"width": m["width"], "blocks": m["blocks"], "conv": m["conv"]})
        elif L["type"] == "attention":
            mixer = PartSpec("biased_attention", {
                "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["scale"],
                "eps": eps, "softcap": float(m.get("softcap") or 0.0), "bias_max": float(m.get("bias_max") or 0.0),
                "bias_rows": int(m.get("bias_rows") or 16) if m.get("bias_max") else 0})
        else:
            mixer = PartSpec("channel_delta", {
                "n_heads": m["heads"], "n_qk_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "conv": m["conv"], "eps": eps,
                "decay_rank": int(m.get("decay_rank") or 0), "gate_rank": int(m.get("gate_rank") or 0)})
        f = L.get("mlp")
        ffn = None
        if f is not None:
            ffn = PartSpec("scored_moe", {"n_experts": f["router"]["experts"], "top": f["router"]["top"],
                                          "intermediate_size": f["expert"]["ff"],
                                          "shared_size": f["shared"]["ff"] if f.get("shared") else 0})
        block = PartSpec("hyper", {"norm": norm, "mixer": mixer, "feed_forward": ffn, "streams": streams,
                                   "connections": cfg.streams is not None})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block))
    final = PartSpec(norm.kind, dict(norm.params, name="norm"))
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        layers=layers,
        final_norm=None,
        schedule=[ScheduleEntry(layer) for layer in cfg.run_order()],
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "name": "embed", "wide": True, "copies": streams}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "norm": final, "tied": False, "name": "head", "norm_prefix": "final."}),
        stop_token_ids=cfg.stop_token_ids,
    )


register_architecture("Tusasun", TusasunConfig, describe_tusasun)
