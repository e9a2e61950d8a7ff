"""Configuration of the Kadodra decoder.

config.json names the design in ``architecture`` and gives: ``vocab``, ``width``, ``logit_scale``,
``norm.eps``, ``loop`` (start, stop, times: layers start .. stop - 1 run ``times`` times in a row with
the same weights), and ``layers``: per layer its ``type`` (``latent_attention`` or ``lightning``), the
mixer's sizes and constants under ``mixer`` and its feed-forward under ``mlp`` (null, ``kind`` dense
with ``ff``, or ``kind`` moe with ``expert`` {ff, limit} and ``router`` {experts, top}).  Every size
and constant comes from there; nothing is assumed equal between layers.
"""
from __future__ import annotations

from typing import Any, Dict, List

from .base import Key, ModelConfig

MIXER_KEYS = {
    "latent_attention": {"heads": int, "dim": int, "rot_dim": int, "vdim": int, "kv_rank": int, "scale": float},
    "lightning": {"heads": int, "dim": int, "vdim": int, "decay": list},
}


def _number(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _check_fields(where: str, d: Any, fields: Dict[str, type], problems: List[str]) -> bool:
    if not isinstance(d, dict):
        problems.append(f"{where}: expected an object")
        return False
    ok = True
    for name, kind in fields.items():
        v = d.get(name)
        if kind is int:
            good = isinstance(v, int) and not isinstance(v, bool)
        elif kind is float:
            good = _number(v)
        else:
            good = isinstance(v, kind)
        if not good:
            problems.append(f"{where}.{name}: missing or not {kind.__name__}")
            ok = False
    return ok


class KadodraConfig(ModelConfig):
    KEYS = {
        "architecture": Key("str"),
        "vocab": Key("int"),
        "width": Key("int"),
        "logit_scale": Key("float", required=False, default=1.0),
        "norm": Key("any"),
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
            if L["type"] == "latent_attention":
                if m["rot_dim"] % 2:
                    p.append(f"{w}.mixer.rot_dim: must be even, got {m['rot_dim']}")
                if m["rot_dim"] > 0:
                    rot = m.get("rot")
                    if _check_fields(w + ".mixer.rot", rot, {"base": float, "dims": int}, p):
                        if rot["dims"] != m["rot_dim"]:
                            p.append(f"{w}.mixer.rot.dims: {rot['dims']} does not equal rot_dim {m['rot_dim']}")
                        if rot.get("scaling") is not None:
                            _check_fields(w + ".mixer.rot.scaling", rot["scaling"],
                                          {"factor": float, "original": int, "fast": float, "slow": float}, p)
                mask = m.get("mask")
                if mask is not None and not (isinstance(mask, dict) and isinstance(mask.get("size"), int) and mask["size"] > 0):
                    p.append(f"{w}.mixer.mask.size: expected a positive integer")
            else:
                if len(m["decay"]) != m["heads"] or not all(_number(x) and 0.0 <= x <= 1.0 for x in m["decay"]):
                    p.append(f"{w}.mixer.decay: expected {m['heads']} numbers in [0, 1]")
            f = L.get("mlp")
            if f is None:
                continue
            if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
                p.append(f"{w}.mlp.kind: expected dense or moe")
            elif f["kind"] == "dense":
                _check_fields(w + ".mlp", f, {"ff": int}, p)
            else:
                if _check_fields(w + ".mlp.expert", f.get("expert"), {"ff": int, "limit": float}, p) and \
                        _check_fields(w + ".mlp.router", f.get("router"), {"experts": int, "top": int}, p):
                    if not 1 <= f["router"]["top"] <= f["router"]["experts"]:
                        p.append(f"{w}.mlp.router: top must lie in 1 .. experts")
        if self.loop is not None:
            if _check_fields("loop", self.loop, {"start": int, "stop": int, "times": int}, p):
                a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
                if not (0 <= a <= b <= len(self.layers)) or t < 1:
                    p.append(f"loop: start {a}, stop {b}, times {t} do not fit {len(self.layers)} layers")
        return p

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def run_order(self):
        """(layer, whether the embedding's rows are added before it) in the order the layers run: the layers before
        the loop, the loop's layers ``times`` times (from the second pass on the embedding's rows are added once,
        right before the pass's first layer), the layers after it."""
        n = len(self.layers)
        loop = self.loop or {"start": 0, "stop": 0, "times": 1}
        a, b, times = loop["start"], loop["stop"], loop["times"]
        order = [(i, False) for i in range(a)]
        for rep in range(times):
            order += [(i, rep > 0 and i == a) for i in range(a, b)]
        order += [(i, False) for i in range(b, n)]
        return order

    @property
    def stop_token_ids(self) -> tuple:
        return tuple(self.stop_tokens)
