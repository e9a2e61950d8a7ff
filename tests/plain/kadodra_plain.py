"""Plain, slow Kadodra: whole sequences, no cache, one function per mechanism.

The oracle of the Kadodra tests.  It shares no code with toyinfer_b200: the configuration is
a dict as config.json holds it, the weights a dict of tensors by checkpoint name, and every
mechanism is written token by token with elementary torch operations in float64.

The design in this file's notation (x is the residual stream, one row per token):

* a layer:    n = rms(x) * w_norm1;  x <- x + mixer(n) + ff(n)        (both read one norm)
* loop:       layers [start, stop) run ``times`` times with the same weights; before every
              pass but the first the embedding rows are added to x
* latent attention: q = Wq n, head by head [dim plain | rot_dim rotated];  d = Wdkv n;
              c = rms(d[:rank]) * w;  r = d[rank:] rotated, one for all heads;
              k_h = [Wuk_h c | r], v_h = Wuv_h c;  a token sees itself and the
              ``window - 1`` tokens before it;  weights exp(s_j) / (exp(sink_h) + sum_j exp(s_j))
* rotation:   pair (i, i + dims/2), angle pos * f_i; f_i is blended between theta^(-2i/dims)
              and the same divided by ``factor`` along a ramp over i, and cos and sin carry the
              magnitude 0.1 ln(factor) + 1
* lightning:  q, k, v = silu(W. n); per head S <- decay_h S + k v^T, o = S^T q; then
              rms over all heads' outputs together, times sigmoid(Wg n), times Wo
* dense ff:   Wdown relu(Wup n)^2
* table moe:  the token id picks ``top`` experts from a table, each weighs 1/top; an expert is
              Wdown (g' sigmoid(1.702 g') (u' + 1)) with g' = min(Wgate n, limit) and
              u' = clamp(Wup n, -limit, limit)
* output:     logits = E (rms(x) * w_final) * logit_scale with E the embedding table
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.to(F64)


# ---------------------------------------------------------------------------
# rotation
# ---------------------------------------------------------------------------
def scaled_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[List[float], float]:
    """Per pair i < dims/2 the angular frequency, and the magnitude that multiplies cos and sin."""
    half = dims // 2
    plain = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return plain, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_index(turns: float) -> float:      # the pair index whose wave turns ``turns`` times over ``original`` positions
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_index(float(scaling["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(plain):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, pos: int, freqs: Sequence[float], magnitude: float) -> torch.Tensor:
    """x[..., dims] at one position; pairs (i, i + dims/2)."""
    half = len(freqs)
    out = x.to(F64).clone()
    for i in range(half):
        a = pos * freqs[i]
        c, s = math.cos(a) * magnitude, math.sin(a) * magnitude
        u, v = x[..., i].to(F64), x[..., i + half].to(F64)
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ---------------------------------------------------------------------------
# mixers (n: [T, width], one sequence from position 0)
# ---------------------------------------------------------------------------
def latent_attention(n: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, start: int = 0) -> torch.Tensor:
    """n: the rows of one sequence whose first row stands at position ``start`` (nothing before it is seen)."""
    T = n.shape[0]
    H, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    rot = m.get("rot")
    freqs, mag = scaled_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rd else ([], 1.0)
    assert not rd or int(rot["dims"]) == rd
    n = n.to(F64)
    q = (n @ w[p + "q"].to(F64).T).view(T, H, dim + rd)
    d = n @ w[p + "dkv"].to(F64).T
    c = rms_norm(d[:, :rank], w[p + "dkv.norm"], eps)
    r = d[:, rank:]
    uk = w[p + "uk"].to(F64).view(H, dim, rank)
    uv = w[p + "uv"].to(F64).view(H, vd, rank)
    sink = w[p + "sink"].to(F64) if (p + "sink") in w else None
    r_rot = torch.stack([rotate(r[t], start + t, freqs, mag) for t in range(T)])
    k_plain = torch.einsum("hdr,tr->thd", uk, c)          # every head's unrotated key part, per token
    val = torch.einsum("hvr,tr->thv", uv, c)
    out = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        first = 0 if window <= 0 else max(0, t - window + 1)
        for h in range(H):
            q_rot = rotate(q[t, h, dim:], start + t, freqs, mag)
            s = (k_plain[first:t + 1, h] @ q[t, h, :dim] + r_rot[first:t + 1] @ q_rot) * m["scale"]
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            denom = e.sum() + (0.0 if sink is None else torch.exp(sink[h] - top))
            out[t, h] = (e / denom) @ val[first:t + 1, h]
    return out.reshape(T, H * vd) @ w[p + "o"].to(F64).T


def lightning(n: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
              state: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = n.shape[0]
    H, dim, vd = m["heads"], m["dim"], m["vdim"]
    n = n.to(F64)
    silu = lambda z: z / (1.0 + torch.exp(-z))
    q = silu(n @ w[p + "q"].to(F64).T).view(T, H, dim)
    k = silu(n @ w[p + "k"].to(F64).T).view(T, H, dim)
    v = silu(n @ w[p + "v"].to(F64).T).view(T, H, vd)
    S = torch.zeros(H, dim, vd, dtype=F64) if state is None else state
    o = torch.zeros(T, H, vd, dtype=F64)
    for t in range(T):
        for h in range(H):
            S[h] = float(m["decay"][h]) * S[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    y = rms_norm(o.reshape(T, H * vd), w[p + "norm"], eps)
    g = 1.0 / (1.0 + torch.exp(-(n @ w[p + "g"].to(F64).T)))
    return (y * g) @ w[p + "o"].to(F64).T


# ---------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------
def dense_ff(n: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    n = n.to(F64)
    u = torch.clamp(n @ w[p + "up"].to(F64).T, min=0.0)
    return (u * u) @ w[p + "down"].to(F64).T


def expert(n: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    n = n.to(F64)
    g = torch.clamp(n @ w[p + "gate"].to(F64).T, max=limit)
    u = torch.clamp(n @ w[p + "up"].to(F64).T, min=-limit, max=limit)
    y = g * (1.0 / (1.0 + torch.exp(-1.702 * g))) * (u + 1.0)
    return y @ w[p + "down"].to(F64).T


def table_moe(n: torch.Tensor, ids: Sequence[int], w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    top = int(f["router"]["top"])
    table = w[p + "table"]
    out = torch.zeros(n.shape[0], n.shape[1], dtype=F64)
    for t, tok in enumerate(ids):
        for j in range(top):
            e = int(table[tok, j])
            out[t] += expert(n[t:t + 1], w, f"{p}e{e}.", float(f["expert"]["limit"]))[0] / top
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def run_order(cfg: dict) -> List[Tuple[int, bool]]:
    """(layer, whether the embedding rows are added before it) in the order the layers run."""
    L = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for rep in range(times):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    order += [(i, False) for i in range(b, L)]
    return order


def forward(w: Dict[str, torch.Tensor], cfg: dict, ids: Sequence[int], keep_layers: bool = False):
    """logits [T, vocab] in float64 (and, when asked, the residual stream after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    emb = w["embed"].to(F64)[list(ids)]
    x = emb.clone()
    streams = []
    for layer, add_emb in run_order(cfg):
        L = cfg["layers"][layer]
        p = f"l{layer}."
        if add_emb:
            x = x + emb
        n = rms_norm(x, w[p + "norm1"], eps)
        if L["type"] == "latent_attention":
            a = latent_attention(n, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "lightning":
            a = lightning(n, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        f = L.get("mlp")
        if f is None:
            y = torch.zeros_like(a)
        elif f["kind"] == "dense":
            y = dense_ff(n, w, p + "mlp.")
        elif f["kind"] == "moe":
            y = table_moe(n, ids, w, p + "mlp.", f)
        else:
            raise ValueError(f["kind"])
        x = x + (a + y)
        streams.append(x.clone())
    n = rms_norm(x, w["final.norm"], eps)
    logits = (n @ w["embed"].to(F64).T) * float(cfg["logit_scale"])
    return (logits, torch.stack(streams)) if keep_layers else logits
