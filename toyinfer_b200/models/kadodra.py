"""Kadodra: the description of the model in terms of parts.

A decoder whose layers each read ONE norm with both their mixer and their feed-forward
(parallel block), over a float32 residual stream; mixers are latent attention (low-rank
shared key/value rows, sliding window, sinks, rotation stretched for long contexts) or
lightning attention (linear attention with a decayed float32 state); feed-forwards are
squared-ReLU dense layers or table-routed mixtures of experts; a span of layers may run
several times with the same weights and memory of its own per pass, the embedding's rows
being added again before every pass but the first; the head is the embedding table behind
the final norm, times a logit scale.  Tensor names: ``embed``, ``final.norm``,
``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``.  Nothing here computes: the parts do.
"""
from __future__ import annotations

import json

from ..config.kadodra import KadodraConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from ..parts.model import LayerSpec, ModelSpec, ScheduleEntry


def describe_kadodra(cfg: KadodraConfig) -> ModelSpec:
    eps = cfg.eps
    norm = lambda name: PartSpec("rmsnorm", {"size": cfg.width, "eps": eps, "name": name, "wide": True})
    positions = {}
    layers = []
    for i, L in enumerate(cfg.layers):
        m = L["mixer"]
        if L["type"] == "latent_attention":
            pos_name = None
            if m["rot_dim"] > 0:
                rot = m["rot"]
                # layers with the same rotation share one pair of tables
                pos_name = "rot:" + json.dumps({"dims": rot["dims"], "base": rot["base"], "scaling": rot.get("scaling")}, sort_keys=True)
                positions.setdefault(pos_name, PartSpec("rotary_half", {
                    "dim": rot["dims"], "theta": rot["base"], "max_positions": cfg.max_positions,
                    "scaling": rot.get("scaling"), "lazy": True}))
            mixer = PartSpec("latent_attention", {
                "n_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
                "scale": m["scale"], "eps": eps, "position": pos_name,
                "window": int(m["mask"]["size"]) if m.get("mask") else 0, "sinks": True})
        else:
            mixer = PartSpec("lightning", {"n_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "decay": list(m["decay"]),
                                           "eps": eps})
        f = L.get("mlp")
        if f is None:
            ffn = None
        elif f["kind"] == "dense":
            ffn = PartSpec("relu2", {"intermediate_size": f["ff"]})
        else:
            ffn = PartSpec("table_moe", {"n_experts": f["router"]["experts"], "top": f["router"]["top"],
                                         "intermediate_size": f["expert"]["ff"], "limit": f["expert"]["limit"],
                                         "vocab_size": cfg.vocab})
        block = PartSpec("parallel", {"norm": norm("norm1"), "mixer": mixer, "feed_forward": ffn})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block))
    schedule = [ScheduleEntry(layer, add_embedding=again) for layer, again in cfg.run_order()]
    return ModelSpec(
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        layers=layers,
        final_norm=None,
        schedule=schedule,
        positions=positions,
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "name": "embed", "wide": True}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "norm": norm("norm"), "tied": True, "scale": cfg.logit_scale,
                                 "norm_prefix": "final."}),
        stop_token_ids=cfg.stop_token_ids,
    )


register_architecture("Kadodra", KadodraConfig, describe_kadodra)
