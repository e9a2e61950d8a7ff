"""Configuration of the Tusasun decoder.

config.json names the design in ``architecture`` and gives: ``vocab``, ``width``, ``norm.eps``, ``streams`` (how many
residual streams a token has; with the key the layers carry connection tensors, without it there is one plain
stream), ``loop`` (start, stop, times: layers start .. stop - 1 run ``times`` times in a row with the same weights and
memory of their own per pass), and ``layers``: per layer its ``type`` (``rglru``, ``attention`` or ``channel_delta``), the
mixer's sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (null, or ``kind`` moe with ``expert`` {ff},
``router`` {experts, top} and optionally ``shared`` {ff}).  Every size and constant comes from there or from a tensor's
shape (the rows of an attention layer's distance table, the ranks of a delta-rule layer's low-rank projections);
nothing is assumed equal between layers.  ``bias_rows``, ``decay_rank`` and ``gate_rank`` may be given for the sake of
drawing random weights; a checkpoint's shapes win.
"""
from __future__ import annotations

from typing import List

from .base import Key, ModelConfig
from .kadodra import _check_fields, _number

MIXER_KEYS = {
    "rglru": {"width": int, "blocks": int, "conv": int},
    "attention": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float},
    "channel_delta": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int},
}


class TusasunConfig(ModelConfig):
    KEYS = {
        "architecture": Key("str"),
        "vocab": Key("int"),
        "width": Key("int"),
        "norm": Key("any"),
        "streams": Key("int", required=False, default=None, nullable=True),
        "loop": Key("any", required=False, default=None, nullable=True),
        "layers": Key("any"),
        "max_positions": Key("int", required=False, default=131072),
        "stop_tokens": Key("int_or_list", required=False, default=()),
    }

    def validate(self) -> List[str]:
        p: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            p.append("vocab and width must be positive")
        if not isinstance(self.norm, dict) or not _number(self.norm.get("eps")) or not self.norm["eps"] > 0:
            p.append("norm.eps: missing or not a positive number")
        if self.streams is not None and not 1 <= self.streams <= 8:
            p.append(f"streams: expected 1 to 8, got {self.streams}")
        if not isinstance(self.layers, list) or not self.layers:
            p.append("layers: expected a non-empty list")
            return p
        for i, L in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in MIXER_KEYS:
                p.append(f"{w}.type: expected one of {sorted(MIXER_KEYS)}")
                continue
            m = L.get("mixer")
            if not _check_fields(w + ".mixer", m, MIXER_KEYS[L["type"]], p):
                continue
            if L["type"] == "rglru":
                if m["blocks"] < 1 or m["width"] % m["blocks"]:
                    p.append(f"{w}.mixer: {m['width']} channels do not cut into {m['blocks']} equal gate blocks")
            else:
                if m["kv_heads"] < 1 or m["heads"] % m["kv_heads"]:
                    p.append(f"{w}.mixer: {m['heads']} heads over {m['kv_heads']} kv heads")
            if L["type"] == "attention":
                for k in ("softcap", "bias_max"):
                    if m.get(k) is not None and not (_number(m[k]) and m[k] > 0):
                        p.append(f"{w}.mixer.{k}: expected a positive number")
            if "conv" in MIXER_KEYS[L["type"]] and not 1 <= m["conv"] <= 8:
                p.append(f"{w}.mixer.conv: expected 1 to 8 taps, got {m['conv']}")
            f = L.get("mlp")
            if f is None:
                continue
            if not isinstance(f, dict) or f.get("kind") != "moe":
                p.append(f"{w}.mlp.kind: expected moe")
            elif _check_fields(w + ".mlp.expert", f.get("expert"), {"ff": int}, p) and \
                    _check_fields(w + ".mlp.router", f.get("router"), {"experts": int, "top": int}, p):
                if not 1 <= f["router"]["top"] <= f["router"]["experts"]:
                    p.append(f"{w}.mlp.router: top must lie in 1 .. experts")
                if f.get("shared") is not None:
                    _check_fields(w + ".mlp.shared", f["shared"], {"ff": int}, p)
        if self.loop is not None:
            if _check_fields("loop", self.loop, {"start": int, "stop": int, "times": int}, p):
                a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
                if not (0 <= a <= b <= len(self.layers)) or t < 1:
                    p.append(f"loop: start {a}, stop {b}, times {t} do not fit {len(self.layers)} layers")
        return p

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def run_order(self) -> List[int]:
        """The layers in the order they run: those before the loop, the loop's layers ``times`` times, those after it."""
        n = len(self.layers)
        loop = self.loop or {"start": 0, "stop": 0, "times": 1}
        a, b, times = loop["start"], loop["stop"], loop["times"]
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    @property
    def stop_token_ids(self) -> tuple:
        return tuple(self.stop_tokens)
